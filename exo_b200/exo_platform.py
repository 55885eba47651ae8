"""Exo platform module: this library's kernels as Exo hardware instructions.

Exo reaches hardware through ``@instr`` procedures -- a body that states the
semantics in Exo object code plus a C template that is emitted at the call site
(docs/instructions.md:14-50; the decorator is src/exo/API.py:52-62; the x86
library, e.g. src/exo/platforms/x86.py:357-374, is the model).  A schedule author
rewrites a loop nest into a call with ``replace(p, cursor, b200_sgemm)`` and
``exocc`` then prints the template with the argument expressions substituted
(src/exo/backend/LoopIR_compiler.py:923-943: ``{name}`` and ``{name}_data`` both
become the C expression of a non-window argument; a numeric scalar such as
``scale : f32`` arrives as a pointer, sizes and bools by value).

The instructions, their templates and the procedures whose bodies they repeat:

    b200_sgemm       sgemm_exo       apps/x86/sgemm/sgemm.py:11-23
    b200_conv        conv            apps/x86/conv/conv.py:10-45
    b200_matmul_i8   matmul_on_cpu   apps/gemmini/src/exo/matmul.py:7-43
    b200_gemm_bf16   gemm_bf16_exo   (bf16 bit patterns travel as ui16, src/exo/core/LoopIR.py:446-462)

Every template passes NULL as the context: the ``ctxt`` in scope in generated code
is the generated library's own ``<stem>_Context*`` (or an uninitialised pointer in
the Gemmini runners), not an ``exo_b200_Context``.  ``C_GLOBAL`` is the line the
instructions add to the generated file's preamble.

This file imports without Exo (whose dependencies are not installed everywhere):
``TEMPLATES`` / ``C_GLOBAL`` / ``render_call`` are plain Python, and the ``@instr``
definitions are only created when ``exo`` is importable.  ``render_call`` formats a
template the way the code generator does, so the emitted C can be compiled and run
against the library without the compiler.
"""
from __future__ import annotations

C_GLOBAL = '#include "exo_b200.h"'

TEMPLATES = {
    "b200_sgemm": "sgemm_exo(NULL, {M}, {N}, {K}, {A_data}, {B_data}, {C_data});",
    "b200_conv": ("conv(NULL, {out_h}, {out_w}, {out_channel}, {in_h}, {in_w}, {in_channel}, {kernel_dim}, "
                  "{batch_size}, {inp_data}, {output_data}, {weights_data}, {bias_data});"),
    "b200_matmul_i8": "matmul_on_cpu(NULL, {N}, {M}, {K}, {scale_data}, {act}, {A_data}, {B_data}, {C_data});",
    "b200_gemm_bf16": "gemm_bf16_exo(NULL, {M}, {N}, {K}, {A_data}, {B_data}, {C_data});",
}

# argument names of each instruction, in order (what the code generator iterates over)
ARGUMENTS = {
    "b200_sgemm": ("M", "N", "K", "A", "B", "C"),
    "b200_conv": ("out_h", "out_w", "out_channel", "in_h", "in_w", "in_channel", "kernel_dim", "batch_size",
                  "inp", "output", "weights", "bias"),
    "b200_matmul_i8": ("N", "M", "K", "scale", "act", "A", "B", "C"),
    "b200_gemm_bf16": ("M", "N", "K", "A", "B", "C"),
}


def render_call(name: str, **exprs: str) -> str:
    """The C statement exocc prints for a call of instruction ``name`` whose arguments
    are the C expressions ``exprs`` (non-window arguments: ``{x}`` and ``{x}_data`` are
    both the parenthesised expression, src/exo/backend/LoopIR_compiler.py:929-941)."""
    missing = [a for a in ARGUMENTS[name] if a not in exprs]
    if missing:
        raise TypeError(f"{name}: missing argument expression(s) {missing}")
    d = {}
    for arg in ARGUMENTS[name]:
        d[arg] = f"({exprs[arg]})"
        d[f"{arg}_data"] = f"({exprs[arg]})"
    return TEMPLATES[name].format(**d)


try:  # the instruction objects exist only where the compiler does
    from exo import DRAM, instr  # noqa: F401
    from exo.frontend.syntax import *  # noqa: F401,F403  (size, f32, i8, ui16, seq, stride, ...)
    from exo.libs.externs import relu, select  # noqa: F401

    HAVE_EXO = True
except Exception:  # ImportError, or a missing dependency of exo itself
    HAVE_EXO = False


if HAVE_EXO:
    from exo.platforms.gemmini import acc_scale, clamp  # the Gemmini output stage procedures

    @instr(TEMPLATES["b200_sgemm"], C_GLOBAL)
    def b200_sgemm(M: size, N: size, K: size, A: f32[M, K] @ DRAM, B: f32[K, N] @ DRAM, C: f32[M, N] @ DRAM):
        assert M >= 1
        assert N >= 1
        assert K >= 1
        assert stride(A, 1) == 1
        assert stride(B, 1) == 1
        assert stride(C, 1) == 1

        for k in seq(0, K):
            for i in seq(0, M):
                for j in seq(0, N):
                    C[i, j] += A[i, k] * B[k, j]

    @instr(TEMPLATES["b200_conv"], C_GLOBAL)
    def b200_conv(
        out_h: size,
        out_w: size,
        out_channel: size,
        in_h: size,
        in_w: size,
        in_channel: size,
        kernel_dim: size,
        batch_size: size,
        inp: f32[batch_size, in_h, in_w, in_channel] @ DRAM,
        output: f32[batch_size, out_h, out_w, out_channel] @ DRAM,
        weights: f32[in_channel, kernel_dim, kernel_dim, out_channel] @ DRAM,
        bias: f32[out_channel] @ DRAM,
    ):
        assert out_h == in_h - kernel_dim + 1
        assert out_w == in_w - kernel_dim + 1

        for oc in seq(0, out_channel):
            for n in seq(0, batch_size):
                for oy in seq(0, out_h):
                    for ox in seq(0, out_w):
                        res: f32
                        res = bias[oc]
                        for ky in seq(0, kernel_dim):
                            for kx in seq(0, kernel_dim):
                                for kc in seq(0, in_channel):
                                    res += weights[kc, ky, kx, oc] * inp[n, oy + ky, ox + kx, kc]
                        relu_v: f32
                        relu_v = relu(res)
                        output[n, oy, ox, oc] = relu_v

    @instr(TEMPLATES["b200_matmul_i8"], C_GLOBAL)
    def b200_matmul_i8(
        N: size,
        M: size,
        K: size,
        scale: f32,
        act: bool,
        A: i8[N, K] @ DRAM,
        B: i8[K, M] @ DRAM,
        C: i8[N, M] @ DRAM,
    ):
        for i in seq(0, N):
            for j in seq(0, M):
                res: i32 @ DRAM
                res = 0.0
                for k in seq(0, K):
                    a: i8 @ DRAM
                    a = A[i, k]
                    b: i8 @ DRAM
                    b = B[k, j]
                    a2: i32
                    b2: i32
                    a2 = a
                    b2 = b
                    res += a2 * b2
                src_tmp: i32
                src_tmp = res
                tmp_res1: f32
                acc_scale(src_tmp, tmp_res1, scale)
                tmp_res2: i8
                clamp(tmp_res1, tmp_res2)
                if act == True:  # noqa: E712  (Exo object code compares with the literal)
                    tmp_res2 = relu(tmp_res2)
                C[i, j] = tmp_res2

    # bf16 has no Exo type: the operands are ui16 bit patterns, B column-major (an [N, K] array),
    # and the body can only state which elements are written -- the arithmetic (widen to fp32,
    # accumulate in fp32, round once to bf16) is the instruction's, as with any @instr whose
    # hardware does more than the object language can express.
    @instr(TEMPLATES["b200_gemm_bf16"], C_GLOBAL)
    def b200_gemm_bf16(M: size, N: size, K: size, A: ui16[M, K] @ DRAM, B: ui16[N, K] @ DRAM, C: ui16[M, N] @ DRAM):
        assert M >= 1
        assert N >= 1
        assert K >= 1
        for i in seq(0, M):
            for j in seq(0, N):
                C[i, j] = 0
                for k in seq(0, K):
                    C[i, j] += A[i, k] * B[j, k]

    __all__ = ["b200_sgemm", "b200_conv", "b200_matmul_i8", "b200_gemm_bf16", "TEMPLATES", "C_GLOBAL", "render_call"]
else:
    __all__ = ["TEMPLATES", "C_GLOBAL", "render_call", "HAVE_EXO"]
