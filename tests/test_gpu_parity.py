"""GPU parity tests: every kernel, called through the C ABI (ctypes), against
the CPU oracle and the committed fixtures on the same seeded inputs.

Bars: bit-exact for the fp32 FFMA paths (SGEMM, conv) and all int8 work;
stated tolerances for 3xTF32 and bf16."""
import os

import numpy as np
import pytest

import oracle
from tests import cases, inputs

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.fixture(scope="module")
def lib():
    import exo_b200

    return exo_b200.library()


@pytest.fixture(scope="module")
def torch():
    import torch

    return torch


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ------------------------------------------------------------- SGEMM (FFMA)
@pytest.mark.parametrize("shape", cases.SGEMM_CASES)
def test_sgemm_ffma_host_pointers_bit_exact(lib, port, golden, shape):
    M, N, K = shape
    A, B, C0 = cases.sgemm_inputs(M, N, K)
    C = C0.copy()
    lib.sgemm_exo(None, M, N, K, A, B, C)
    assert np.array_equal(bits(C), bits(golden[f"sgemm_{M}x{N}x{K}"]))
    assert np.array_equal(bits(C), bits(port.sgemm(A, B, C0.copy())))


@pytest.mark.parametrize("shape", cases.SGEMM_DIGEST_CASES + [(129, 257, 40), (33, 128, 16), (32, 8192, 300)]
                         + cases.SGEMM_EXTRA_CASES)
def test_sgemm_ffma_device_pointers_bit_exact(lib, port, torch, golden, shape):
    M, N, K = shape
    A, B, C0 = cases.sgemm_inputs(M, N, K)
    dA, dB, dC = dev(torch, A), dev(torch, B), dev(torch, C0)
    lib.sgemm_exo_ffma(None, M, N, K, dA, dB, dC)
    torch.cuda.synchronize()
    C = dC.cpu().numpy()
    key = f"sgemm_{M}x{N}x{K}_sha256"
    if key in golden:
        assert cases.digest(C) == str(golden[key])
    else:
        assert np.array_equal(bits(C), bits(port.sgemm(A, B, C0.copy())))


def test_sgemm_ffma_signed_zero_and_specials(lib, port):
    """-0.0 in C must survive a ragged K tail; inf/nan propagate like the chain."""
    M, N, K = 9, 70, 19
    A, B, C0 = cases.sgemm_inputs(M, N, K, seed=5)
    A[3, :] = 0.0
    C0[3, :] = -0.0
    B[:, 5] = -np.abs(B[:, 5])  # every product in column 5 of row 3 is -0: the -0 in C survives
    A[4, 2] = np.inf
    A[5, 1] = np.nan
    C = C0.copy()
    lib.sgemm_exo(None, M, N, K, A, B, C)
    want = port.sgemm(A, B, C0.copy(), naive=True)
    # NaN payloads are not part of the contract (x86 propagates an operand's payload,
    # the GPU returns the canonical NaN); everything else, signed zeros and
    # infinities included, is compared bit for bit.
    assert np.array_equal(np.isnan(C), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.isnan(want).any() and np.isinf(want).any()
    assert np.array_equal(bits(C)[ok], bits(want)[ok])
    assert np.signbit(C[3, 5]) and C[3, 5] == 0 and not np.signbit(C[3]).all()


def test_sgemm_ffma_full_size_rows_against_oracle(lib, port, torch):
    """4096^3 is beyond what the CPU oracle finishes in seconds; because every
    output row depends only on its own row of A, a sample of rows run through
    the oracle at full N and K checks the full-size launch bit for bit.  (8192^3:
    tests/test_gpu_kernel_variants.py.)"""
    M = N = K = 4096
    g = torch.Generator(device="cuda").manual_seed(7)
    dA = torch.rand((M, K), generator=g, device="cuda") * 2 - 1
    dB = torch.rand((K, N), generator=g, device="cuda") * 2 - 1
    dC = torch.rand((M, N), generator=g, device="cuda") * 2 - 1
    rows = [0, 1, 127, 128, 2049, 4095]
    C0 = dC[rows].cpu().numpy()
    lib.sgemm_exo(None, M, N, K, dA, dB, dC)
    torch.cuda.synchronize()
    port.set_threads(os.cpu_count() or 1)
    try:
        want = port.sgemm(dA[rows].cpu().numpy(), dB.cpu().numpy(), C0.copy())
    finally:
        port.set_threads(1)
    assert np.array_equal(bits(dC[rows].cpu().numpy()), bits(want))


# -------------------------------------------------------------------- SSYRK
# sizes of the reference's comparison benchmark (apps/x86/ssyrk/bench_ssyrk.cpp:60-65: n = 64 .. 2048,
# k = 16 .. 2048, powers of two) plus ragged ones
SSYRK_CASES = [(64, 16), (64, 2048), (100, 33), (129, 7), (256, 512), (1000, 77), (1024, 1024), (2048, 16), (2048, 2048)]


@pytest.mark.parametrize("shape", SSYRK_CASES)
def test_ssyrk_ffma_bit_exact_on_the_upper_triangle(lib, port, torch, shape):
    """C += A A^T for j >= i, one fmaf chain per element in increasing k: bit-identical to
    the oracle (itself equal to the SGEMM oracle on (A, A^T)); the strict lower triangle of
    C keeps its bits."""
    N, K = shape
    A = inputs.uniform_f32(1000 + N + K, (N, K))
    C0 = inputs.uniform_f32(2000 + N, (N, N))
    dC = dev(torch, C0)
    lib.ssyrk_exo(None, N, K, dev(torch, A), dC)
    torch.cuda.synchronize()
    port.set_threads(os.cpu_count() or 1)
    try:
        want = port.ssyrk(A, C0.copy())
    finally:
        port.set_threads(1)
    assert np.array_equal(bits(dC.cpu().numpy()), bits(want))
    if N <= 256:  # host pointers too
        C = C0.copy()
        lib.ssyrk_exo_ffma(None, N, K, A, C)
        assert np.array_equal(bits(C), bits(want))


@pytest.mark.parametrize("shape", [(64, 16), (100, 33), (256, 512), (1000, 77), (2048, 2048), (300, 4100)])
def test_ssyrk_3xtf32_within_tolerance(lib, torch, shape):
    N, K = shape
    A = inputs.uniform_f32(1000 + N + K, (N, K))
    C0 = inputs.uniform_f32(2000 + N, (N, N))
    dC = dev(torch, C0)
    lib.ssyrk_exo_3xtf32(None, N, K, dev(torch, A), dC)
    torch.cuda.synchronize()
    C = dC.cpu().numpy()
    A64 = A.astype(np.float64)
    ref = C0.astype(np.float64) + A64 @ A64.T
    # Tolerance, stated: the 3xTF32 SGEMM bound plus 2.4e-8 * min(K, 256) * S.  The tensor core adds into
    # its fp32 accumulator without round-to-nearest (up to 2^-24 of the running sum per accumulation
    # step, three steps per 8 elements of K); for sums of random sign the running sum is small against
    # S = |C0| + sum |a||a| and the SGEMM bound's middle term covers it, but on the diagonal of A A^T
    # every product is positive, the running sum IS S, and the bias is coherent.  The kernel drains its
    # accumulator every 256 elements of K, which caps the term.
    bound = (tf32x3_bound(K) + 2.4e-8 * min(K, 256)) * (np.abs(C0).astype(np.float64) + np.abs(A64) @ np.abs(A64).T)
    up = np.triu(np.ones((N, N), bool))
    assert (np.abs(C - ref)[up] <= bound[up] + 1e-30).all()
    assert np.array_equal(bits(C)[~up], bits(C0)[~up])  # the strict lower triangle is untouched


# ------------------------------------------------------------ SGEMM (3xTF32)
# Tolerance, stated: per element, with S = |C0| + sum_k |a_ik| |b_kj|,
#     |C_gpu - C_fp64| <= (1.5e-6 + 1e-6 * min(K, 1024) / 1024 + 1e-7 * K / 1024) * S.
# The constant term: each product carries a relative error of about 2^-21 from
# the dropped lo*lo term and the TF32 rounding of lo.  The second term: the tensor
# core adds into its fp32 accumulator without round-to-nearest, a bias that grows
# linearly with the number of accumulation steps (measured before chunking: 3.1e-3
# absolute at K = 4096 on uniform[-1,1) inputs, where S is about 1024); the kernel
# therefore drains its accumulator into C every 1024 elements of K, which caps that
# term.  The last term: one round-to-nearest fp32 add into C per chunk.
def tf32x3_bound(K):
    return 1.5e-6 + 1e-6 * min(K, 1024) / 1024.0 + 1e-7 * K / 1024.0


@pytest.mark.parametrize("shape", [(128, 256, 32), (256, 512, 1024), (1000, 1000, 1000), (17, 4099, 513),
                                   (4096, 64, 4096), (1, 8192, 2048), (300, 77, 129), (2048, 1000, 999),
                                   (1030, 2049, 513), (512, 512, 8192), (256, 300, 2500)])
def test_sgemm_3xtf32_within_tolerance(lib, torch, shape):
    M, N, K = shape
    A, B, C0 = cases.sgemm_inputs(M, N, K)
    dA, dB, dC = dev(torch, A), dev(torch, B), dev(torch, C0)
    lib.sgemm_exo_3xtf32(None, M, N, K, dA, dB, dC)
    torch.cuda.synchronize()
    C = dC.cpu().numpy().astype(np.float64)
    ref = C0.astype(np.float64) + A.astype(np.float64) @ B.astype(np.float64)
    bound = tf32x3_bound(K) * (np.abs(C0).astype(np.float64) + np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64))
    err = np.abs(C - ref)
    print(f"3xTF32 {shape}: max err {err.max():.3e}, worst err/bound {(err / (bound + 1e-30)).max():.3f}")
    assert (err <= bound + 1e-30).all(), f"max err {err.max():.3e}, worst ratio {(err / bound).max():.3f}"


# --------------------------------------------------------------------- conv
def test_conv_specialized_fixture(lib, golden):
    src = inputs.uniform_f32(11, (5, 82, 102, 128))
    wts = inputs.uniform_f32(12, (128, 3, 3, 128))
    bias = inputs.uniform_f32(13, (128,))
    out = np.empty((5, 80, 100, 128), np.float32)
    lib.conv_specialized(None, src, out, wts, bias)
    assert cases.digest(out) == str(golden["conv_specialized_uniform_sha256"])


def test_conv_specialized_reference_fill(lib, port, golden):
    src, wts, bias = inputs.conv_instance_fill(5, 82, 102, 128, 128, 3)
    out = np.empty((5, 80, 100, 128), np.float32)
    lib.conv_specialized(None, src, out, wts, bias)
    if cases.digest(src) + cases.digest(wts) + cases.digest(bias) == str(golden["conv_specialized_inputs_sha256"]):
        assert cases.digest(out) == str(golden["conv_specialized_sha256"])
    else:
        port.set_threads(os.cpu_count() or 1)
        try:
            assert np.array_equal(bits(out), bits(port.conv(src, wts, bias)))
        finally:
            port.set_threads(1)


@pytest.mark.parametrize("cfg", [
    # batch, h, w, ci, co, k, pad, relu
    (4, 56, 56, 64, 64, 3, 1, True),     # the 3x3 workload
    (8, 28, 28, 256, 512, 1, 0, True),   # the 1x1 workload
    (2, 9, 11, 8, 16, 3, 1, True),
    (1, 7, 5, 3, 5, 3, 0, False),        # ragged channels: scalar loads
    (3, 6, 6, 4, 130, 5, 2, True),
    (1, 6, 6, 1, 4, 3, 1, True),         # one input channel: a k-tile of 16 walks through 16 taps
    (2, 8, 8, 20, 12, 3, 1, True),       # Ci = 20: vector loads, a k-tile straddles a tap boundary mid-way
])
def test_conv_nhwc_bit_exact(lib, port, torch, cfg):
    b, h, w, ci, co, k, pad, relu = cfg
    inp = inputs.uniform_f32(101, (b, h, w, ci))
    wts = inputs.uniform_f32(102, (k, k, ci, co))
    bias = inputs.uniform_f32(103, (co,))
    oh, ow = h + 2 * pad - k + 1, w + 2 * pad - k + 1
    out = torch.empty((b, oh, ow, co), dtype=torch.float32, device="cuda")
    lib.conv_nhwc_exo(None, b, h, w, ci, co, k, pad, relu, dev(torch, inp), out, dev(torch, wts), dev(torch, bias))
    torch.cuda.synchronize()
    port.set_threads(os.cpu_count() or 1)
    try:
        want = port.conv_nhwc(inp, wts, bias, pad, relu)
    finally:
        port.set_threads(1)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))


@pytest.mark.parametrize("cfg", [
    # batch, h, w, ci, co, k, pad, stride: the two stride-2 layers of the reference's conv bench
    # (apps/x86/conv/bench_conv.cpp:47-49) and ragged ones
    (4, 224, 224, 3, 64, 7, 3, 2),
    (4, 28, 28, 128, 128, 3, 1, 2),
    (2, 11, 9, 5, 7, 3, 0, 3),
    (1, 10, 10, 8, 16, 2, 1, 2),
])
def test_conv_strided_bit_exact(lib, port, torch, cfg):
    b, h, w, ci, co, k, pad, stride = cfg
    inp = inputs.uniform_f32(141, (b, h, w, ci))
    wts = inputs.uniform_f32(142, (k, k, ci, co))
    bias = inputs.uniform_f32(143, (co,))
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    out = torch.empty((b, oh, ow, co), dtype=torch.float32, device="cuda")
    lib.conv_nhwc_strided_exo(None, b, h, w, ci, co, k, pad, stride, True, dev(torch, inp), out, dev(torch, wts),
                              dev(torch, bias))
    torch.cuda.synchronize()
    port.set_threads(os.cpu_count() or 1)
    try:
        want = port.conv_nhwc_strided(inp, wts, bias, pad, stride, True)
    finally:
        port.set_threads(1)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))


def test_conv_equals_im2col_plus_sgemm(lib, port):
    """The decomposition of tests/test_im2col.py: marshal, then SGEMM into a
    bias-initialised C, then ReLU -- done with the GPU SGEMM -- equals the
    implicit-GEMM convolution bit for bit."""
    b, h, w, ci, co, k, pad = 4, 56, 56, 64, 64, 3, 1
    inp = inputs.uniform_f32(201, (b, h, w, ci))
    wts = inputs.uniform_f32(202, (k, k, ci, co))
    bias = inputs.uniform_f32(203, (co,))
    out = np.empty((b, h, w, co), np.float32)
    lib.conv_nhwc_exo(None, b, h, w, ci, co, k, pad, True, inp, out, wts, bias)
    col = port.im2col_nhwc(inp, k, pad)
    C = np.tile(bias, (col.shape[0], 1)).astype(np.float32)
    lib.sgemm_exo(None, col.shape[0], co, col.shape[1], col, np.ascontiguousarray(wts.reshape(-1, co)), C)
    C = np.where(C > 0, C, np.float32(0)).astype(np.float32)
    assert np.array_equal(bits(out), bits(C.reshape(out.shape)))


def test_conv_generic_entry_matches_specialized_layout(lib, port):
    inp = inputs.uniform_f32(301, (2, 10, 12, 16))
    wts = inputs.uniform_f32(302, (16, 3, 3, 32))  # [Ci, Kh, Kw, Co]
    bias = inputs.uniform_f32(303, (32,))
    out = np.empty((2, 8, 10, 32), np.float32)
    lib.conv(None, 8, 10, 32, 10, 12, 16, 3, 2, inp, out, wts, bias)
    assert np.array_equal(bits(out), bits(port.conv(inp, wts, bias)))


# --------------------------------------------------------------------- int8
@pytest.mark.parametrize("name", list(cases.I8_CASES))
def test_i8_matmul_512_fixture(lib, golden, name):
    A, B, scale, act = cases.i8_inputs(name)
    C = np.empty((512, 512), np.int8)
    s = np.array([scale], np.float32)
    lib.cpu_matmul_512x512x512(None, s, act, A, B, C)
    assert np.array_equal(C, golden[f"i8_{name}"])
    C2 = np.empty_like(C)
    lib.matmul_512x512x512(None, s, act, A, B, C2)
    assert np.array_equal(C2, C)


def test_i8_ties_and_uninitialised_ctxt(lib, golden):
    import ctypes

    A, B = cases.i8_tie_inputs()
    C = np.empty((512, 512), np.int8)
    # the reference runner passes an uninitialised context pointer (run_matmul.c:49-52)
    garbage = ctypes.c_void_p(0xDEADBEEF0)
    fn = lib.dll.cpu_matmul_512x512x512
    s = np.array([1.0 / 256], np.float32)
    fn(garbage, s.ctypes.data, False, A.ctypes.data, B.ctypes.data, C.ctypes.data)
    assert lib.dll.exo_b200_last_error() == 0
    assert np.array_equal(C, golden["i8_ties_s256"])
    lib.matmul_on_cpu(None, 512, 512, 512, 1.0 / 512, True, A, B, C)
    assert np.array_equal(C, golden["i8_ties_s512_relu"])


@pytest.mark.parametrize("name", list(oracle.REF_MATMUL_SHAPES))
def test_i8_reference_shapes(lib, golden, name):
    N, M, K = oracle.REF_MATMUL_SHAPES[name]
    x, y = inputs.gemmini_matmul_fill(N, M, K)
    C = np.empty((N, M), np.int8)
    getattr(lib, f"cpu_matmul_{name}")(None, np.array([2.0], np.float32), False, x, y, C)
    assert cases.digest(C) == str(golden[f"i8_runner_{name}_sha256"])
    A = inputs.int8(700 + N % 97, (N, K), -16, 15)
    B = inputs.int8(701 + M % 89, (K, M), -16, 15)
    getattr(lib, f"matmul_{name}")(None, np.array([1.0 / 64], np.float32), True, A, B, C)
    assert cases.digest(C) == str(golden[f"i8_shape_{name}_sha256"])


@pytest.mark.parametrize("shape", [(1, 1, 1), (5, 7, 17), (64, 48, 16), (130, 300, 256), (257, 129, 4096),
                                   (128, 256, 128), (1000, 520, 272)])
@pytest.mark.parametrize("scale,act", [(1.0 / 256, False), (0.3, True), (2.0 ** -7, True)])
def test_i8_generic_shapes(lib, port, torch, shape, scale, act):
    N, M, K = shape
    A = inputs.int8(N + K, (N, K), -20, 20)
    B = inputs.int8(M + K + 1, (K, M), -20, 20)
    dC = torch.empty((N, M), dtype=torch.int8, device="cuda")
    lib.matmul_on_cpu(None, N, M, K, float(scale), act, dev(torch, A), dev(torch, B), dC)
    torch.cuda.synchronize()
    assert np.array_equal(dC.cpu().numpy(), port.matmul_i8(A, B, scale, act))


def test_i8_large_accumulator_rounding(lib):
    K = 4096
    A = np.full((128, K), 127, np.int8)
    B = np.full((K, 256), 127, np.int8)
    B[:5, 1] = 126
    B[:3, 2] = 125
    A[1, :7] = 126
    acc = A.astype(np.int64) @ B.astype(np.int64)
    scale = np.float32(2.0 ** -19)
    want = np.clip(np.rint(acc.astype(np.float32) * scale), -128, 127).astype(np.int8)
    C = np.empty((128, 256), np.int8)
    lib.matmul_on_cpu(None, 128, 256, K, float(scale), False, A, B, C)
    assert np.array_equal(C, want)


def test_i8_4096_cubed(lib, port, torch):
    """The full-size int8 workload, bit-exact against the oracle on a row sample
    (rows are independent), with the saturation rate the workload implies."""
    n = 4096
    A = inputs.int8(41, (n, n))
    B = inputs.int8(42, (n, n))
    dC = torch.empty((n, n), dtype=torch.int8, device="cuda")
    for act in (False, True):
        lib.matmul_on_cpu(None, n, n, n, 1.0 / 256, act, dev(torch, A), dev(torch, B), dC)
        torch.cuda.synchronize()
        C = dC.cpu().numpy()
        rows = np.r_[0:8, 127:131, 2047:2050, 4088:4096]
        port.set_threads(os.cpu_count() or 1)
        try:
            want = port.matmul_i8(np.ascontiguousarray(A[rows]), B, 1.0 / 256, act)
        finally:
            port.set_threads(1)
        assert np.array_equal(C[rows], want)


@pytest.mark.parametrize("name", list(oracle.REF_CONV_I8_SHAPES))
def test_i8_conv_reference_shapes(lib, golden, name):
    b, od, co, kd, ci, ind = oracle.REF_CONV_I8_SHAPES[name]
    inp, w, bias = inputs.gemmini_conv_fill(b, ind, ci, co, kd)
    out = np.empty((b, od, od, co), np.int8)
    getattr(lib, f"conv_{name}_cpu")(None, out, bias, inp, w, False, np.array([1.0], np.float32))
    assert cases.digest(out) == str(golden[f"i8conv_runner_{name}_sha256"])
    inp = inputs.int8(800 + ci, (b, ind, ind, ci), -16, 15)
    w = inputs.int8(801 + co, (kd, kd, ci, co), -16, 15)
    bias = inputs.int32(802, (1, co), -5000, 5000)
    getattr(lib, f"conv_{name}")(None, out, bias, inp, w, True, np.array([1.0 / 128], np.float32))
    assert cases.digest(out) == str(golden[f"i8conv_seeded_{name}_sha256"])
    lib.conv_on_cpu_stride_1(None, b, od, co, kd, ci, ind, out, bias, inp, w, True, 1.0 / 128)
    assert cases.digest(out) == str(golden[f"i8conv_seeded_{name}_sha256"])


@pytest.mark.parametrize("cfg", [
    # batch, in_dim, ci, co, k     (tensor path: ci % 16 == 0 and co % 16 == 0; else SIMT)
    (2, 19, 32, 48, 3), (1, 9, 16, 16, 5), (3, 12, 144, 272, 3), (2, 10, 64, 64, 1), (1, 130, 16, 32, 3),
    (2, 11, 24, 40, 3),
])
def test_i8_conv_generic_shapes(lib, port, torch, cfg):
    b, ind, ci, co, k = cfg
    od = ind - k + 1
    inp = inputs.int8(900 + ind, (b, ind, ind, ci), -20, 20)
    w = inputs.int8(901 + co, (k, k, ci, co), -20, 20)
    bias = inputs.int32(902, (1, co), -3000, 3000)
    out = torch.empty((b, od, od, co), dtype=torch.int8, device="cuda")
    for scale, act in [(1.0 / 64, True), (0.013, False)]:
        lib.conv_on_cpu_stride_1(None, b, od, co, k, ci, ind, out, dev(torch, bias), dev(torch, inp), dev(torch, w),
                                 act, float(scale))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), port.conv_i8(inp, w, bias, scale, act))


# ------------------------------------------------------- conv on tensor cores
@pytest.mark.parametrize("cfg", [
    (4, 56, 56, 64, 64, 3, 1, True),     # the 3x3 workload
    (8, 28, 28, 256, 512, 1, 0, True),   # the 1x1 workload
    (2, 9, 11, 8, 16, 3, 1, True),
    (1, 20, 150, 12, 36, 3, 2, False),   # rows wider than a tile, channels not a multiple of 32
    (3, 6, 6, 4, 130, 5, 2, True),
])
def test_conv_3xtf32_within_tolerance(lib, port, torch, cfg):
    """Same bound as the 3xTF32 SGEMM with K = kdim^2 * Ci and S = |bias| + sum |x||w|
    (ReLU is 1-Lipschitz, so the bound carries through it)."""
    b, h, w, ci, co, k, pad, relu = cfg
    inp = inputs.uniform_f32(111, (b, h, w, ci))
    wts = inputs.uniform_f32(112, (k, k, ci, co))
    bias = inputs.uniform_f32(113, (co,))
    oh, ow = h + 2 * pad - k + 1, w + 2 * pad - k + 1
    out = torch.empty((b, oh, ow, co), dtype=torch.float32, device="cuda")
    lib.conv_nhwc_exo_3xtf32(None, b, h, w, ci, co, k, pad, relu, dev(torch, inp), out, dev(torch, wts),
                             dev(torch, bias))
    torch.cuda.synchronize()
    port.set_threads(os.cpu_count() or 1)
    try:
        want = port.conv_nhwc(inp, wts, bias, pad, relu)
        S = port.conv_nhwc(np.abs(inp), np.abs(wts), np.abs(bias), pad, False)
    finally:
        port.set_threads(1)
    err = np.abs(out.cpu().numpy().astype(np.float64) - want.astype(np.float64))
    bound = (tf32x3_bound(k * k * ci) + 2e-7) * S.astype(np.float64)  # + the fp32 chain's own rounding
    assert (err <= bound).all(), f"max err {err.max():.3e}, worst ratio {(err / bound).max():.3f}"


# --------------------------------------------------------------------- bf16
# Tolerance, stated: |C_gpu - C_ref| <= 2^-7 |C_ref| + 1e-3 * sqrt(K) * 4e-4 where C_ref is
# the reference fp32 SGEMM chain on the widened inputs rounded once to bf16 (one bf16 ulp
# of slack for a different fp32 accumulation order plus an absolute floor near zero).
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 512), (384, 300, 1000), (130, 70, 72), (2048, 2048, 2048),
                                   (130, 70, 71), (257, 129, 1001), (3, 5, 1)])  # K % 8 != 0: padded operand copies
def test_gemm_bf16_against_reference_sgemm(lib, port, torch, shape):
    M, N, K = shape
    A = inputs.normal_bf16(51, (M, K))
    Bt = inputs.normal_bf16(52, (N, K))  # column-major K x N
    dC = torch.empty((M, N), dtype=torch.int16, device="cuda")
    lib.gemm_bf16_exo(None, M, N, K, dev(torch, A.view(np.int16)), dev(torch, Bt.view(np.int16)), dC)
    torch.cuda.synchronize()
    C = inputs.bf16_bits_to_f32(dC.cpu().numpy().view(np.uint16))
    port.set_threads(os.cpu_count() or 1)
    try:
        ref = inputs.bf16_bits_to_f32(port.gemm_bf16(A, Bt))
    finally:
        port.set_threads(1)
    tol = 2.0 ** -7 * np.abs(ref) + 1e-3 * np.sqrt(K) * 4e-4
    err = np.abs(C - ref)
    assert (err <= tol).all(), f"max err {err.max():.3e} at ref {ref.reshape(-1)[err.argmax()]:.3e}"
    # and most outputs are bit-identical to the reference rounding
    assert (C == ref).mean() > 0.9


def test_gemm_bf16_unaligned_bases(lib, port, torch):
    """A, B and C that start 2 bytes into an allocation (not 16-byte aligned): TMA cannot
    address them, so the operands go through the padded copy and C through scalar stores."""
    M, N, K = 200, 136, 264
    A = inputs.normal_bf16(53, (M, K))
    Bt = inputs.normal_bf16(54, (N, K))

    def shifted(a):
        flat = torch.full((a.size + 1,), 0x7FC0, dtype=torch.int16, device="cuda")
        view = flat[1:].view(a.shape)
        view.copy_(torch.from_numpy(a.view(np.int16)))
        assert view.data_ptr() % 16 != 0
        return view

    dC = torch.full((M * N + 1,), 0x7FC0, dtype=torch.int16, device="cuda")[1:].view(M, N)
    lib.gemm_bf16_exo(None, M, N, K, shifted(A), shifted(Bt), dC)
    torch.cuda.synchronize()
    C = inputs.bf16_bits_to_f32(dC.cpu().numpy().view(np.uint16))
    ref = inputs.bf16_bits_to_f32(port.gemm_bf16(A, Bt))
    assert (np.abs(C - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-3 * np.sqrt(K) * 4e-4).all()


def test_two_streams_share_the_default_context_scratch(lib, port, torch):
    """Two device-pointer calls that both use the default context's scratch (the 3xTF32 split
    copies; the K-major copy of B for an int8 matmul whose B pitch TMA cannot read in place),
    issued back to back on two different streams: the second call's pre-pass must wait for the
    first call's GEMM to finish reading the scratch.  Both results are checked."""
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    M, N, K = 1024, 1024, 2048
    A1, B1, C1 = cases.sgemm_inputs(M, N, K, seed=601)
    A2, B2, C2 = cases.sgemm_inputs(M, N, K, seed=602)
    d = [dev(torch, x) for x in (A1, B1, C1, A2, B2, C2)]
    n, m, k = 2048, 1000, 2048  # m % 16 != 0: B goes through the transposing pre-pass into scratch
    A8a, B8a = inputs.int8(611, (n, k), -20, 20), inputs.int8(612, (k, m), -20, 20)
    A8b, B8b = inputs.int8(613, (n, k), -20, 20), inputs.int8(614, (k, m), -20, 20)
    d8 = [dev(torch, x) for x in (A8a, B8a, A8b, B8b)]
    o1 = torch.empty((n, m), dtype=torch.int8, device="cuda")
    o2 = torch.empty((n, m), dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    for _ in range(3):  # a few rounds: the race, if present, is a matter of timing
        d[2].copy_(torch.from_numpy(C1))
        d[5].copy_(torch.from_numpy(C2))
        torch.cuda.synchronize()
        with torch.cuda.stream(s1):
            lib.sgemm_exo_3xtf32(None, M, N, K, d[0], d[1], d[2])
        with torch.cuda.stream(s2):
            lib.sgemm_exo_3xtf32(None, M, N, K, d[3], d[4], d[5])
        with torch.cuda.stream(s1):
            lib.matmul_on_cpu(None, n, m, k, 1.0 / 64, True, d8[0], d8[1], o1)
        with torch.cuda.stream(s2):
            lib.matmul_on_cpu(None, n, m, k, 1.0 / 64, True, d8[2], d8[3], o2)
        torch.cuda.synchronize()
        for (A, B, C0, got) in ((A1, B1, C1, d[2]), (A2, B2, C2, d[5])):
            ref = C0.astype(np.float64) + A.astype(np.float64) @ B.astype(np.float64)
            bound = tf32x3_bound(K) * (np.abs(C0) + np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64))
            assert (np.abs(got.cpu().numpy() - ref) <= bound).all()
        port.set_threads(os.cpu_count() or 1)
        try:
            assert np.array_equal(o1.cpu().numpy(), port.matmul_i8(A8a, B8a, 1.0 / 64, True))
            assert np.array_equal(o2.cpu().numpy(), port.matmul_i8(A8b, B8b, 1.0 / 64, True))
        finally:
            port.set_threads(1)


def test_context_of_another_device_is_made_current(lib, port, torch):
    """A context created for device 1 used while device 0 is current: the call switches to the
    context's device for its duration (and back), so the kernel runs where the operands are."""
    import exo_b200

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    M, N, K = 130, 200, 64
    A, B, C0 = cases.sgemm_inputs(M, N, K, seed=71)
    ctx = exo_b200.Context(device=1)
    dA, dB, dC = (torch.from_numpy(x).to("cuda:1") for x in (A, B, C0))
    torch.cuda.set_device(0)
    lib.dll.sgemm_exo(ctx.handle, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr())
    assert lib.dll.exo_b200_last_error() == 0
    assert torch.cuda.current_device() == 0
    lib.synchronize(ctx)
    assert np.array_equal(bits(dC.cpu().numpy()), bits(port.sgemm(A, B, C0.copy())))
    # operands of device 0 through the device-1 context are refused, not dereferenced
    d0 = torch.from_numpy(C0).to("cuda:0")
    lib.dll.sgemm_exo(ctx.handle, M, N, K, dA.data_ptr(), dB.data_ptr(), d0.data_ptr())
    assert lib.dll.exo_b200_last_error() == exo_b200.ERR_INVALID_ARGUMENT
    ctx.close()


def test_measured_peaks_are_plausible(lib):
    """The probe kernels behind the roofline denominators: packed fp32 FMA from registers and
    tcgen05.mma with operands resident in shared memory.  Bounds are loose physical ones for a
    B200 (148 SMs x 128 lanes x 2 x 1.965 GHz = 74.4 TFLOP/s fp32; int8 about twice bf16)."""
    simt = lib.dll.exo_b200_measure_peak(0, 20)
    i8 = lib.dll.exo_b200_measure_peak(1, 20)
    bf16 = lib.dll.exo_b200_measure_peak(2, 20)
    tf32 = lib.dll.exo_b200_measure_peak(3, 20)
    assert lib.dll.exo_b200_last_error() == 0, lib.dll.exo_b200_last_error_string()
    print(f"measured peaks: fp32 SIMT {simt:.1f}, int8 {i8:.0f}, bf16 {bf16:.0f}, tf32 {tf32:.0f} T(FL)OP/s")
    assert 45.0 < simt < 80.0
    assert 1000.0 < bf16 < 2600.0
    assert 1.5 * bf16 < i8 < 2.5 * bf16
    assert 0.35 * bf16 < tf32 < 0.65 * bf16
    assert lib.dll.exo_b200_measure_peak(9, 20) < 0 and lib.dll.exo_b200_last_error() != 0


def test_error_side_channel_on_gpu(lib):
    import exo_b200

    A = np.zeros((8, 8), np.float32)
    with pytest.raises(exo_b200.ExoB200Error):
        lib.sgemm_exo(None, -1, 8, 8, A, A, A)
    lib.sgemm_exo(None, 8, 8, 8, A, A, A)  # a good call clears the error
    assert lib.dll.exo_b200_last_error() == 0


def test_bounded_wait_times_out_and_context_survives(lib):
    """Failure detection on the device without a fault: a wait that nothing will
    ever satisfy must run out, surface as EXO_B200_ERR_TIMEOUT through the status
    word, and leave the context usable for the next call."""
    import time

    import exo_b200

    t0 = time.time()
    code = lib.dll.exo_b200_selftest_bounded_wait(None, 20000)  # 20 ms limit
    dt = time.time() - t0
    assert code == exo_b200.ERR_TIMEOUT
    assert b"wait ran out" in lib.dll.exo_b200_last_error_string()
    assert dt < 5.0
    A = np.eye(8, dtype=np.float32)
    C = np.zeros((8, 8), np.float32)
    lib.sgemm_exo(None, 8, 8, 8, A, A, C)
    assert np.array_equal(C, A)
    assert lib.dll.exo_b200_synchronize(None) == 0


def test_gemm_bf16_large_uses_tall_pair_kernel(lib, torch):
    """Problems with at least 296 tiles of 512 x 256 run on the kernel whose CTA pairs own a
    512 x 256 tile (two accumulators per CTA sharing each B stage).  Ragged in M, N and K;
    every element must be written; a row sample (tile and half-tile boundaries, last rows) is
    checked against float64 within the bf16 tolerance."""
    M, N, K = 20 * 512 + 130, 16 * 256 + 72, 520
    A = inputs.normal_bf16(81, (M, K))
    Bt = inputs.normal_bf16(82, (N, K))
    dC = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")  # NaN pattern
    lib.gemm_bf16_exo(None, M, N, K, dev(torch, A.view(np.int16)), dev(torch, Bt.view(np.int16)), dC)
    torch.cuda.synchronize()
    C = dC.cpu().numpy().view(np.uint16)
    assert not (C == 0x7FC0).any()
    rows = np.array([0, 127, 128, 255, 256, 383, 384, 511, 512, 5000, 10239, 10240, M - 2, M - 1])
    ref = inputs.bf16_bits_to_f32(A[rows]).astype(np.float64) @ inputs.bf16_bits_to_f32(Bt).astype(np.float64).T
    got = inputs.bf16_bits_to_f32(C[rows]).astype(np.float64)
    assert (np.abs(got - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-3 * np.sqrt(K) * 4e-4).all()
    # and column samples over every row
    cols = np.array([0, 255, 256, 4095, 4096, N - 1])
    refc = inputs.bf16_bits_to_f32(A).astype(np.float64) @ inputs.bf16_bits_to_f32(Bt[cols]).astype(np.float64).T
    gotc = inputs.bf16_bits_to_f32(C[:, cols]).astype(np.float64)
    assert (np.abs(gotc - refc) <= 2.0 ** -7 * np.abs(refc) + 1e-3 * np.sqrt(K) * 4e-4).all()


# ------------------------------------------------ host-pointer row pipeline
def test_host_pointer_pipeline_matches_device_pointer_path(lib, torch):
    """Large host-pointer calls run as a chunked copy-in / multiply / copy-out pipeline;
    the result must be bit-identical to the single-launch device-pointer path
    (rows are independent and every kernel is deterministic)."""
    rng = np.random.default_rng(0)
    # fp32, C += (C is an input too), ragged last chunk
    M, N, K = 6100, 1024, 1024
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    C = C0.copy()
    lib.sgemm_exo(None, M, N, K, A, B, C)
    dC = dev(torch, C0)
    lib.sgemm_exo(None, M, N, K, dev(torch, A), dev(torch, B), dC)
    torch.cuda.synchronize()
    assert np.array_equal(bits(C), bits(dC.cpu().numpy()))
    # bf16
    M, N, K = 8192, 2048, 2048
    Ab = inputs.normal_bf16(61, (M, K))
    Bb = inputs.normal_bf16(62, (N, K))
    Cb = np.zeros((M, N), np.uint16)
    lib.gemm_bf16_exo(None, M, N, K, Ab, Bb, Cb)
    dCb = torch.empty((M, N), dtype=torch.int16, device="cuda")
    lib.gemm_bf16_exo(None, M, N, K, dev(torch, Ab.view(np.int16)), dev(torch, Bb.view(np.int16)), dCb)
    torch.cuda.synchronize()
    assert np.array_equal(Cb, dCb.cpu().numpy().view(np.uint16))
    # int8
    n, m, k = 16500, 2048, 2048
    A8 = inputs.int8(63, (n, k), -30, 30)
    B8 = inputs.int8(64, (k, m), -30, 30)
    C8 = np.zeros((n, m), np.int8)
    lib.matmul_on_cpu(None, n, m, k, 1.0 / 128, True, A8, B8, C8)
    dC8 = torch.empty((n, m), dtype=torch.int8, device="cuda")
    lib.matmul_on_cpu(None, n, m, k, 1.0 / 128, True, dev(torch, A8), dev(torch, B8), dC8)
    torch.cuda.synchronize()
    assert np.array_equal(C8, dC8.cpu().numpy())


def test_host_pointer_block_pipeline_matches_device_pointer_path(lib, port, torch):
    """With A, B and C all on the host and B large, the bf16 GEMM uploads both operands
    piecewise and sends 2048 x 4096 output blocks back as they become computable (ragged
    last row chunk and column block here).  Bit-identical to the device-pointer call; a
    sample of rows is also checked against the oracle."""
    M, N, K = 8192 + 640, 8192 + 328, 2048
    Ab = inputs.normal_bf16(71, (M, K))
    Bb = inputs.normal_bf16(72, (N, K))
    Cb = np.full((M, N), 0x7FC0, np.uint16)  # NaN pattern: every element must be overwritten
    lib.gemm_bf16_exo(None, M, N, K, Ab, Bb, Cb)
    dCb = torch.empty((M, N), dtype=torch.int16, device="cuda")
    lib.gemm_bf16_exo(None, M, N, K, dev(torch, Ab.view(np.int16)), dev(torch, Bb.view(np.int16)), dCb)
    torch.cuda.synchronize()
    assert np.array_equal(Cb, dCb.cpu().numpy().view(np.uint16))
    rows = np.array([0, 1, 2047, 2048, 4095, 6144, 8191, 8192, M - 1])
    ref = inputs.bf16_bits_to_f32(Ab[rows]).astype(np.float64) @ inputs.bf16_bits_to_f32(Bb).astype(np.float64).T
    got = inputs.bf16_bits_to_f32(Cb[rows]).astype(np.float64)
    assert (np.abs(got - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-3 * np.sqrt(K) * 4e-4).all()


def test_unaligned_device_pointers(lib, port, torch):
    """Operands that start at an odd offset inside an allocation (4 bytes for fp32, 1 byte
    for int8) must take the scalar / SIMT paths and still match the oracle bit for bit."""
    M, N, K = 130, 260, 96
    A, B, C0 = cases.sgemm_inputs(M, N, K, seed=77)

    def shifted(a, dtype):
        flat = torch.empty(a.size + 1, dtype=dtype, device="cuda")
        view = flat[1:].view(a.shape)
        view.copy_(torch.from_numpy(a))
        assert view.data_ptr() % 16 != 0
        return view

    dA, dB, dC = shifted(A, torch.float32), shifted(B, torch.float32), shifted(C0, torch.float32)
    lib.sgemm_exo(None, M, N, K, dA, dB, dC)
    torch.cuda.synchronize()
    want = port.sgemm(A, B, C0.copy())
    assert np.array_equal(bits(dC.cpu().numpy()), bits(want))
    # 3xTF32 repacks its operands, so alignment does not matter there either
    dC2 = shifted(C0, torch.float32)
    lib.sgemm_exo_3xtf32(None, M, N, K, dA, dB, dC2)
    torch.cuda.synchronize()
    ref = C0.astype(np.float64) + A.astype(np.float64) @ B.astype(np.float64)
    bound = tf32x3_bound(K) * (np.abs(C0) + np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64))
    assert (np.abs(dC2.cpu().numpy() - ref) <= bound).all()
    # int8
    n, m, k = 130, 256, 128
    A8, B8 = inputs.int8(5, (n, k), -20, 20), inputs.int8(6, (k, m), -20, 20)
    dA8, dB8 = shifted(A8, torch.int8), shifted(B8, torch.int8)
    dC8 = torch.empty(n * m + 1, dtype=torch.int8, device="cuda")[1:].view(n, m)
    lib.matmul_on_cpu(None, n, m, k, 1.0 / 32, True, dA8, dB8, dC8)
    torch.cuda.synchronize()
    assert np.array_equal(dC8.cpu().numpy(), port.matmul_i8(A8, B8, 1.0 / 32, True))


def test_explicit_context_stream_and_path(lib, port, torch):
    """ctxt != NULL: an exo_b200_Context carrying its own stream and SGEMM path."""
    import exo_b200

    M, N, K = 512, 384, 1024
    A, B, C0 = cases.sgemm_inputs(M, N, K, seed=88)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        dA, dB, dC = dev(torch, A), dev(torch, B), dev(torch, C0)
        ctx = exo_b200.Context(stream=side.cuda_stream)  # default path: exact FFMA
        lib.sgemm_exo(ctx, M, N, K, dA, dB, dC)
        lib.synchronize(ctx)
        assert np.array_equal(bits(dC.cpu().numpy()), bits(port.sgemm(A, B, C0.copy())))
        # same context switched to the tensor path: within the 3xTF32 bound, and not the exact bits
        lib.dll.exo_b200_context_set_sgemm_path(ctx.handle, exo_b200.SGEMM_3XTF32)
        dC2 = dev(torch, C0)
        lib.sgemm_exo(ctx, M, N, K, dA, dB, dC2)
        lib.synchronize(ctx)
        ref = C0.astype(np.float64) + A.astype(np.float64) @ B.astype(np.float64)
        bound = tf32x3_bound(K) * (np.abs(C0) + np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64))
        got = dC2.cpu().numpy()
        assert (np.abs(got - ref) <= bound).all()
        ctx.close()
    # a pointer that is not a context is rejected, not dereferenced as one
    junk = np.zeros(64, np.uint8)
    lib.dll.sgemm_exo(junk.ctypes.data, M, N, K, A.ctypes.data, B.ctypes.data, C0.ctypes.data)
    assert lib.dll.exo_b200_last_error() == exo_b200.ERR_INVALID_ARGUMENT


def test_conv_reference_layout_on_tensor_path(lib, port, torch):
    """conv (weights [Ci, Kh, Kw, Co], the x86 app's layout) with the context switched to
    3xTF32: the weight pre-pass has to reorder K to (ky, kx, ci) from either layout."""
    import exo_b200

    inp = inputs.uniform_f32(401, (2, 20, 22, 32))
    wts = inputs.uniform_f32(402, (32, 3, 3, 48))  # [Ci, Kh, Kw, Co]
    bias = inputs.uniform_f32(403, (48,))
    ctx = exo_b200.Context(sgemm_path=exo_b200.SGEMM_3XTF32)
    out = torch.empty((2, 18, 20, 48), dtype=torch.float32, device="cuda")
    lib.conv(ctx, 18, 20, 48, 20, 22, 32, 3, 2, dev(torch, inp), out, dev(torch, wts), dev(torch, bias))
    lib.synchronize(ctx)
    want = port.conv(inp, wts, bias)
    S = port.conv_nhwc(np.abs(inp), np.ascontiguousarray(np.abs(wts).transpose(1, 2, 0, 3)), np.abs(bias), 0, False)
    err = np.abs(out.cpu().numpy().astype(np.float64) - want.astype(np.float64))
    bound = (tf32x3_bound(9 * 32) + 2e-7) * S.astype(np.float64)
    assert (err <= bound).all(), f"max err {err.max():.3e}, worst ratio {(err / bound).max():.3f}"
    assert err.max() > 0  # it really took the tensor path (the FFMA path would be bit-exact)
    ctx.close()


def test_conv_weight_cache_is_opt_in_and_invalidated(lib, port, torch):
    """With exo_b200_context_cache_weights on, the TF32 split of the weights is reused while the same
    weight tensor is passed; after an in-place update the caller invalidates.  Results stay within the
    3xTF32 bound in every phase, and the cache is off unless asked for."""
    import exo_b200

    b, h, w, ci, co, k, pad = 2, 14, 14, 32, 64, 3, 1
    inp = inputs.uniform_f32(131, (b, h, w, ci))
    w1 = inputs.uniform_f32(132, (k, k, ci, co))
    w2 = inputs.uniform_f32(133, (k, k, ci, co))
    bias = inputs.uniform_f32(134, (co,))
    ctx = exo_b200.Context(sgemm_path=exo_b200.SGEMM_3XTF32)
    d_in, d_w, d_b = dev(torch, inp), dev(torch, w1), dev(torch, bias)
    out = torch.empty((b, h, w, co), dtype=torch.float32, device="cuda")

    def check(weights):
        lib.conv_nhwc_exo(ctx, b, h, w, ci, co, k, pad, True, d_in, out, d_w, d_b)
        lib.synchronize(ctx)
        want = port.conv_nhwc(inp, weights, bias, pad, True)
        S = port.conv_nhwc(np.abs(inp), np.abs(weights), np.abs(bias), pad, False).astype(np.float64)
        err = np.abs(out.cpu().numpy().astype(np.float64) - want)
        return bool((err <= (tf32x3_bound(k * k * ci) + 2e-7) * S).all())

    assert check(w1)                       # cache off (default): every call splits the weights
    d_w.copy_(torch.from_numpy(w2))
    assert check(w2)                       # ... so an in-place update is simply seen
    lib.dll.exo_b200_context_cache_weights(ctx.handle, 1)
    assert check(w2) and check(w2)         # second call reuses the split
    d_w.copy_(torch.from_numpy(w1))        # in-place update: the caller's promise is to invalidate
    lib.dll.exo_b200_context_invalidate(ctx.handle)
    assert check(w1)
    d_w2 = dev(torch, w2)                  # another tensor: a different key, no invalidation needed
    d_w = d_w2
    assert check(w2)
    lib.dll.exo_b200_context_cache_weights(ctx.handle, 0)
    ctx.close()


@pytest.mark.gpu
def test_concurrent_host_threads_share_the_default_context(lib, port):
    """Host threads calling with host buffers and ctxt = NULL at the same time (what an
    OpenMP caller of the generated C would do) take turns inside the library; every
    result is still bit-identical to the oracle."""
    import threading
    shapes = [(192, 130, 77), (64, 64, 300), (257, 33, 129), (100, 200, 50)]
    work = []
    for i, (M, N, K) in enumerate(shapes):
        A, B, C = cases.sgemm_inputs(M, N, K, seed=40 + i)
        want = C.copy()
        port.sgemm(A, B, want)
        work.append((M, N, K, A, B, C, want))
    errors = []

    # by-pointer scalars (the int8 scale given as a Python float) are per-call temporaries of the
    # wrapper: concurrent callers must not free each other's
    A8, B8 = inputs.int8(51, (64, 48), -20, 20), inputs.int8(52, (48, 80), -20, 20)
    scales = [1.0 / 64, 0.3, 2.0, 0.011]
    want8 = [port.matmul_i8(A8, B8, s, True) for s in scales]

    def run(mine, item):
        M, N, K, A, B, C, want = item
        try:
            for _ in range(5):
                got = C.copy()
                lib.sgemm_exo_ffma(None, M, N, K, A, B, got)
                if not np.array_equal(bits(got), bits(want)):
                    errors.append((M, N, K))
                got8 = np.empty((64, 80), np.int8)
                lib.matmul_on_cpu(None, 64, 80, 48, scales[mine], True, A8, B8, got8)
                if not np.array_equal(got8, want8[mine]):
                    errors.append(("i8", scales[mine]))
        except Exception as e:  # noqa: BLE001 - reported through the list
            errors.append(repr(e))

    threads = [threading.Thread(target=run, args=(i, w)) for i, w in enumerate(work)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
