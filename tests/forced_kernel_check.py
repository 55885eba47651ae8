"""Runs one GEMM with the kernel choice forced through the library's EXOB200_*
switches and checks it against the oracle.

The switches are read once per process, so tests/test_gpu_kernel_variants.py
runs this module as a child process per variant:

    EXOB200_TC2_TALL=1 python -m tests.forced_kernel_check bf16 2048 2048 2048

Outputs sit between guard bands (tests/guard.py).  Prints one line starting
with "OK" on success; any failure is an exception (non-zero exit).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def bf16_tolerance(ref, K):
    """The bf16 bound of tests/test_gpu_parity.py: one bf16 ulp of the reference
    plus an absolute floor near zero."""
    return 2.0 ** -7 * np.abs(ref) + 1e-3 * np.sqrt(K) * 4e-4


def check_bf16(M, N, K):
    import torch

    import exo_b200
    import oracle
    from tests import inputs
    from tests.guard import Guarded

    lib, port = exo_b200.library(), oracle.port()
    A = inputs.normal_bf16(51, (M, K))
    Bt = inputs.normal_bf16(52, (N, K))
    out = Guarded(torch, (M, N), torch.int16)
    lib.gemm_bf16_exo(None, M, N, K, torch.from_numpy(A.view(np.int16)).cuda(),
                      torch.from_numpy(Bt.view(np.int16)).cuda(), out.view)
    torch.cuda.synchronize()
    assert out.bands_intact(), "a store landed outside the output"
    Cbits = out.view.cpu().numpy().view(np.uint16)
    assert not (Cbits == 0xA5A5).any(), "an output element was not written"
    C = inputs.bf16_bits_to_f32(Cbits)
    port.set_threads(os.cpu_count() or 1)
    ref = inputs.bf16_bits_to_f32(port.gemm_bf16(A, Bt))  # reference fp32 chain on widened inputs, rounded once
    err = np.abs(C - ref)
    assert (err <= bf16_tolerance(ref, K)).all(), f"max err {err.max():.3e}"
    same = float((C == ref).mean())
    assert same > 0.9, same
    print(f"OK bf16 {M}x{N}x{K}: max err {err.max():.3e}, {same:.4f} of the outputs bit-identical")


def check_i8(N, M, K):
    import torch

    import exo_b200
    import oracle
    from tests import inputs
    from tests.guard import Guarded

    lib, port = exo_b200.library(), oracle.port()
    A = inputs.int8(N + K, (N, K))
    B = inputs.int8(M + K + 1, (K, M))
    port.set_threads(os.cpu_count() or 1)
    for scale, act in ((1.0 / 256, False), (0.0007, True)):
        out = Guarded(torch, (N, M), torch.int8)
        lib.matmul_on_cpu(None, N, M, K, float(scale), act, torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(),
                          out.view)
        torch.cuda.synchronize()
        assert out.bands_intact(), "a store landed outside the output"
        want = port.matmul_i8(A, B, scale, act)
        assert np.array_equal(out.view.cpu().numpy(), want), "int8 output differs from the oracle"
    print(f"OK i8 {N}x{M}x{K}: bit-exact")


def check_ffma(M, N, K):
    """The exact-fp32 tile engine under a forced tile size (EXOB200_FFMA_TILE, EXOB200_FFMA_SCALAR): SGEMM,
    SSYRK on the upper triangle (N x N from an N x K operand) and a padded, strided convolution whose
    implicit GEMM has about the same extents, each bit for bit against the oracle."""
    import torch

    import exo_b200
    import oracle
    from tests import inputs
    from tests.guard import Guarded

    lib, port = exo_b200.library(), oracle.port()
    port.set_threads(os.cpu_count() or 1)
    bits = lambda x: np.ascontiguousarray(x).view(np.uint32)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()

    A = inputs.uniform_f32(7 + M, (M, K))
    B = inputs.uniform_f32(8 + N, (K, N))
    C0 = inputs.uniform_f32(9 + K, (M, N))
    out = Guarded(torch, (M, N), torch.float32)
    out.view.copy_(dev(C0))
    lib.sgemm_exo_ffma(None, M, N, K, dev(A), dev(B), out.view)
    torch.cuda.synchronize()
    assert out.bands_intact(), "a store landed outside the output"
    assert np.array_equal(bits(out.view.cpu().numpy()), bits(port.sgemm(A, B, C0.copy()))), "sgemm differs"

    S0 = inputs.uniform_f32(10 + N, (N, N))
    dS = dev(S0)
    lib.ssyrk_exo_ffma(None, N, K, dev(B.T), dS)
    torch.cuda.synchronize()
    assert np.array_equal(bits(dS.cpu().numpy()), bits(port.ssyrk(np.ascontiguousarray(B.T), S0.copy()))), "ssyrk differs"

    b, k, pad, stride, ci = 2, 3, 1, 2, max(1, K // 9)
    h = w = max(4, int(round((M / b) ** 0.5)) * stride)
    co = N
    inp = inputs.uniform_f32(11, (b, h, w, ci))
    wts = inputs.uniform_f32(12, (k, k, ci, co))
    bias = inputs.uniform_f32(13, (co,))
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    cout = Guarded(torch, (b * oh * ow, co), torch.float32)
    lib.conv_nhwc_strided_exo(None, b, h, w, ci, co, k, pad, stride, True, dev(inp), cout.view, dev(wts), dev(bias))
    torch.cuda.synchronize()
    assert cout.bands_intact(), "a store landed outside the output"
    want = port.conv_nhwc_strided(inp, wts, bias, pad, stride, True).reshape(b * oh * ow, co)
    assert np.array_equal(bits(cout.view.cpu().numpy()), bits(want)), "conv differs"
    print(f"OK ffma {M}x{N}x{K}: sgemm, ssyrk and conv bit-exact")


def check_sgemm(M, N, K):
    """sgemm_exo_ffma alone (for switches that only move the SGEMM's kernel choice), bit for bit."""
    import torch

    import exo_b200
    import oracle
    from tests import inputs
    from tests.guard import Guarded

    lib, port = exo_b200.library(), oracle.port()
    port.set_threads(os.cpu_count() or 1)
    A = inputs.uniform_f32(17 + M, (M, K))
    B = inputs.uniform_f32(18 + N, (K, N))
    C0 = inputs.uniform_f32(19 + K, (M, N))
    out = Guarded(torch, (M, N), torch.float32)
    out.view.copy_(torch.from_numpy(C0).cuda())
    lib.sgemm_exo_ffma(None, M, N, K, torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), out.view)
    torch.cuda.synchronize()
    assert out.bands_intact(), "a store landed outside the output"
    want = port.sgemm(A, B, C0.copy())
    assert np.array_equal(out.view.cpu().numpy().view(np.uint32), want.view(np.uint32)), "sgemm differs"
    print(f"OK sgemm {M}x{N}x{K}: bit-exact")


if __name__ == "__main__":
    kind = sys.argv[1]
    dims = [int(x) for x in sys.argv[2:5]]
    {"bf16": check_bf16, "i8": check_i8, "ffma": check_ffma, "sgemm": check_sgemm}[kind](*dims)
