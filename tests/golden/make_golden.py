"""Generates tests/golden/reference_vectors.npz from the reference's own
exocc-generated C (oracle/_ref/libexo_ref.so, built by oracle/build_ref.py
from the reference checkout).  Run where that checkout exists:

    python oracle/build_ref.py && python tests/golden/make_golden.py

The fixture then travels with the repository, so machines without the
reference can still pin the oracle port and the CUDA kernels to it.
Small outputs are stored whole; large ones as SHA-256 plus a strided sample.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from tests import cases, inputs  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")


def main():
    r = oracle.ref()
    d = {}
    for (M, N, K) in cases.SGEMM_CASES:
        A, B, C0 = cases.sgemm_inputs(M, N, K)
        d[f"sgemm_{M}x{N}x{K}"] = r.sgemm(A, B, C0.copy())
    for (M, N, K) in cases.SGEMM_DIGEST_CASES:
        A, B, C0 = cases.sgemm_inputs(M, N, K)
        C = r.sgemm(A, B, C0.copy())
        d[f"sgemm_{M}x{N}x{K}_sha256"] = np.array(cases.digest(C))
        d[f"sgemm_{M}x{N}x{K}_sample"] = cases.sample(C)
    # conv_specialized on the reference harness's own deterministic fill
    src, wts, bias = inputs.conv_instance_fill(5, 82, 102, 128, 128, 3)
    out = r.conv_specialized(src, wts, bias)
    d["conv_specialized_sha256"] = np.array(cases.digest(out))
    d["conv_specialized_sample"] = cases.sample(out)
    d["conv_specialized_inputs_sha256"] = np.array(cases.digest(src) + cases.digest(wts) + cases.digest(bias))
    # ... and on seeded uniform inputs
    src = inputs.uniform_f32(11, (5, 82, 102, 128))
    wts = inputs.uniform_f32(12, (128, 3, 3, 128))
    bias = inputs.uniform_f32(13, (128,))
    out = r.conv_specialized(src, wts, bias)
    d["conv_specialized_uniform_sha256"] = np.array(cases.digest(out))
    d["conv_specialized_uniform_sample"] = cases.sample(out)
    # int8 matmul 512^3
    for name in cases.I8_CASES:
        A, B, scale, act = cases.i8_inputs(name)
        d[f"i8_{name}"] = r.matmul_i8("512x512x512", A, B, scale, act)
    A, B = cases.i8_tie_inputs()
    d["i8_ties_s256"] = r.matmul_i8("512x512x512", A, B, 1.0 / 256, False)
    d["i8_ties_s512_relu"] = r.matmul_i8("512x512x512", A, B, 1.0 / 512, True)
    # the reference runner's own vector (run_matmul.c: scale 2.0, act false)
    for name, (N, M, K) in oracle.REF_MATMUL_SHAPES.items():
        x, y = inputs.gemmini_matmul_fill(N, M, K)
        C = r.matmul_i8(name, x, y, 2.0, False)
        d[f"i8_runner_{name}_sha256"] = np.array(cases.digest(C))
        d[f"i8_runner_{name}_sample"] = cases.sample(C)
        A = inputs.int8(700 + N % 97, (N, K), -16, 15)
        B = inputs.int8(701 + M % 89, (K, M), -16, 15)
        C = r.matmul_i8(name, A, B, 1.0 / 64, True)
        d[f"i8_shape_{name}_sha256"] = np.array(cases.digest(C))
        d[f"i8_shape_{name}_sample"] = cases.sample(C)
    # int8 conv: runner vector (scale 1.0, act false) and a seeded fractional case
    for name, (b, od, co, kd, ci, ind) in oracle.REF_CONV_I8_SHAPES.items():
        inp, w, bias = inputs.gemmini_conv_fill(b, ind, ci, co, kd)
        out = r.conv_i8(name, inp, w, bias, 1.0, False)
        d[f"i8conv_runner_{name}_sha256"] = np.array(cases.digest(out))
        d[f"i8conv_runner_{name}_sample"] = cases.sample(out)
        inp = inputs.int8(800 + ci, (b, ind, ind, ci), -16, 15)
        w = inputs.int8(801 + co, (kd, kd, ci, co), -16, 15)
        bias = inputs.int32(802, (1, co), -5000, 5000)
        out = r.conv_i8(name, inp, w, bias, 1.0 / 128, True)
        d[f"i8conv_seeded_{name}_sha256"] = np.array(cases.digest(out))
        d[f"i8conv_seeded_{name}_sample"] = cases.sample(out)
    np.savez_compressed(OUT, **d)
    print(f"wrote {OUT}: {len(d)} arrays, {os.path.getsize(OUT) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
