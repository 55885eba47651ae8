"""The Exo platform module (exo_b200/exo_platform.py): its C templates, formatted the
way exocc formats an @instr call (src/exo/backend/LoopIR_compiler.py:923-943), must
compile against include/exo_b200.h and compute what the instruction bodies state.
Exo itself is not importable here (its dependencies are not installed), so the
@instr objects are not built; what exocc would print for a call is rendered with
render_call(), put into a C file shaped like a generated one, and compiled with gcc."""
import ast
import os
import subprocess

import pytest

from exo_b200 import exo_platform as plat

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "exo_b200")

STUB = r"""
#include <math.h>
#include <stdint.h>
#include <stdbool.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
%(c_global)s

/* what a generated procedure looks like: ctxt first, sizes as int_fast32_t, scalars by pointer */
static void use_sgemm(void *ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const float* A, const float* B, float* C) {
  (void)ctxt;
  %(sgemm)s
}
static void use_conv(void *ctxt, int_fast32_t out_h, int_fast32_t out_w, int_fast32_t out_channel, int_fast32_t in_h,
                     int_fast32_t in_w, int_fast32_t in_channel, int_fast32_t kernel_dim, int_fast32_t batch_size,
                     const float* inp, float* output, const float* weights, const float* bias) {
  (void)ctxt;
  %(conv)s
}
static void use_matmul(void *ctxt, int_fast32_t N, int_fast32_t M, int_fast32_t K, const float* scale, bool act,
                       const int8_t* A, const int8_t* B, int8_t* C) {
  (void)ctxt;
  %(matmul)s
}
static void use_bf16(void *ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const uint16_t* A, const uint16_t* B,
                     uint16_t* C) {
  (void)ctxt;
  %(bf16)s
}

static float bf2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static uint16_t f2bf(float f) { uint32_t u; memcpy(&u, &f, 4); u += 0x7FFFu + ((u >> 16) & 1u); return (uint16_t)(u >> 16); }

int main(void) {
  long bad = 0;
  void *garbage = (void *)(size_t)0x12340;  /* a generated caller's ctxt: never handed on */
  { /* C += A B, one fmaf chain per element in increasing k */
    enum { M = 37, N = 52, K = 29 };
    static float A[M * K], B[K * N], C[M * N], W[M * N];
    for (int i = 0; i < M * K; i++) A[i] = (float)((i * 7) %% 13 - 6) / 8.0f;
    for (int i = 0; i < K * N; i++) B[i] = (float)((i * 5) %% 11 - 5) / 4.0f;
    for (int i = 0; i < M * N; i++) C[i] = W[i] = (float)(i %% 9) / 16.0f;
    use_sgemm(garbage, M, N, K, A, B, C);
    for (int i = 0; i < M; i++) for (int j = 0; j < N; j++) {
      float c = W[i * N + j];
      for (int k = 0; k < K; k++) c = fmaf(A[i * K + k], B[k * N + j], c);
      if (memcmp(&c, &C[i * N + j], 4)) bad++;
    }
    if (exo_b200_last_error()) { printf("sgemm: %%s\n", exo_b200_last_error_string()); return 1; }
  }
  { /* conv: weights [Ci, Kh, Kw, Co], bias, ReLU */
    enum { NB = 2, IH = 7, IW = 9, CI = 4, CO = 8, KD = 3, OH = IH - KD + 1, OW = IW - KD + 1 };
    static float inp[NB * IH * IW * CI], w[CI * KD * KD * CO], bias[CO], out[NB * OH * OW * CO];
    for (int i = 0; i < NB * IH * IW * CI; i++) inp[i] = (float)((i * 3) %% 17 - 8) / 8.0f;
    for (int i = 0; i < CI * KD * KD * CO; i++) w[i] = (float)((i * 5) %% 7 - 3) / 4.0f;
    for (int i = 0; i < CO; i++) bias[i] = (float)(i - 4) / 2.0f;
    use_conv(garbage, OH, OW, CO, IH, IW, CI, KD, NB, inp, out, w, bias);
    for (int n = 0; n < NB; n++) for (int oy = 0; oy < OH; oy++) for (int ox = 0; ox < OW; ox++) for (int oc = 0; oc < CO; oc++) {
      float r = bias[oc];
      for (int ky = 0; ky < KD; ky++) for (int kx = 0; kx < KD; kx++) for (int kc = 0; kc < CI; kc++)
        r = fmaf(w[((kc * KD + ky) * KD + kx) * CO + oc], inp[((n * IH + oy + ky) * IW + ox + kx) * CI + kc], r);
      r = r > 0.0f ? r : 0.0f;
      if (memcmp(&r, &out[((n * OH + oy) * OW + ox) * CO + oc], 4)) bad++;
    }
  }
  { /* int8 matmul, scale by pointer, act by value */
    enum { N = 40, M = 48, K = 32 };
    static int8_t A[N * K], B[K * M], C[N * M];
    float scale = 0.03f;
    for (int i = 0; i < N * K; i++) A[i] = (int8_t)((i * 7) %% 31 - 15);
    for (int i = 0; i < K * M; i++) B[i] = (int8_t)((i * 3) %% 29 - 14);
    use_matmul(garbage, N, M, K, &scale, true, A, B, C);
    for (int i = 0; i < N; i++) for (int j = 0; j < M; j++) {
      int32_t acc = 0;
      for (int k = 0; k < K; k++) acc += (int32_t)A[i * K + k] * (int32_t)B[k * M + j];
      float t = nearbyintf((float)acc * scale);
      t = t > 127.0f ? 127.0f : (t < -128.0f ? -128.0f : t);
      int8_t q = (int8_t)t; if (q < 0) q = 0;
      if (q != C[i * M + j]) bad++;
    }
  }
  { /* bf16: B column-major, fp32 accumulate, one rounding */
    enum { M = 16, N = 24, K = 32 };
    static uint16_t A[M * K], B[N * K], C[M * N];
    for (int i = 0; i < M * K; i++) A[i] = f2bf((float)((i * 5) %% 9 - 4) / 8.0f);
    for (int i = 0; i < N * K; i++) B[i] = f2bf((float)((i * 7) %% 11 - 5) / 16.0f);
    use_bf16(garbage, M, N, K, A, B, C);
    for (int i = 0; i < M; i++) for (int j = 0; j < N; j++) {
      float c = 0.0f;  /* small dyadic values: every partial sum is exact, so the order cannot matter */
      for (int k = 0; k < K; k++) c += bf2f(A[i * K + k]) * bf2f(B[j * K + k]);
      if (f2bf(c) != C[i * N + j]) bad++;
    }
  }
  if (exo_b200_last_error()) { printf("error: %%s\n", exo_b200_last_error_string()); return 1; }
  printf("%%ld mismatches\n", bad);
  return bad != 0;
}
"""


def stub_source():
    return STUB % {
        "c_global": plat.C_GLOBAL,
        "sgemm": plat.render_call("b200_sgemm", M="M", N="N", K="K", A="A", B="B", C="C"),
        "conv": plat.render_call("b200_conv", out_h="out_h", out_w="out_w", out_channel="out_channel", in_h="in_h",
                                 in_w="in_w", in_channel="in_channel", kernel_dim="kernel_dim",
                                 batch_size="batch_size", inp="inp", output="output", weights="weights", bias="bias"),
        "matmul": plat.render_call("b200_matmul_i8", N="N", M="M", K="K", scale="scale", act="act", A="A", B="B", C="C"),
        "bf16": plat.render_call("b200_gemm_bf16", M="M", N="N", K="K", A="A", B="B", C="C"),
    }


def build_stub(tmp_path):
    from exo_b200 import build

    build.build()
    src = tmp_path / "generated_like.c"
    src.write_text(stub_source())
    exe = tmp_path / "generated_like"
    subprocess.run(["gcc", "-std=gnu11", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o",
                    str(exe), "-L", LIBDIR, "-lexo_b200", f"-Wl,-rpath,{LIBDIR}", "-lm"], check=True)
    return str(exe)


def test_module_imports_without_exo_and_templates_cover_every_argument():
    assert set(plat.TEMPLATES) == set(plat.ARGUMENTS) == {"b200_sgemm", "b200_conv", "b200_matmul_i8", "b200_gemm_bf16"}
    for name, args in plat.ARGUMENTS.items():
        call = plat.render_call(name, **{a: a.upper() for a in args})
        for a in args:
            assert f"({a.upper()})" in call, (name, a)
        assert call.endswith(");") and "NULL" in call  # the generated caller's ctxt is never handed on
    with pytest.raises(TypeError):
        plat.render_call("b200_sgemm", M="M")


def test_instruction_bodies_are_the_reference_loop_nests():
    """Without Exo the @instr functions are not created, but their source must still be
    valid Python syntax (Exo parses the function's AST) and hold the four definitions."""
    tree = ast.parse(open(plat.__file__).read())
    names = {n.name for n in ast.walk(tree) if isinstance(n, ast.FunctionDef)}
    assert {"b200_sgemm", "b200_conv", "b200_matmul_i8", "b200_gemm_bf16"} <= names
    for fn in (n for n in ast.walk(tree) if isinstance(n, ast.FunctionDef) and n.name.startswith("b200_")):
        deco = fn.decorator_list[0]
        assert isinstance(deco, ast.Call) and deco.func.id == "instr"
        assert [a.arg for a in fn.args.args] == list(plat.ARGUMENTS[fn.name])


def test_rendered_calls_compile_against_the_header(tmp_path):
    build_stub(tmp_path)


@pytest.mark.gpu
def test_rendered_calls_compute_the_instruction_semantics(tmp_path):
    exe = build_stub(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("0 mismatches")
