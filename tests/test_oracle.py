"""The oracle port (oracle/exo_oracle.c) against (a) the committed fixtures
generated from the reference's exocc output and (b), where it was built, the
compiled reference itself.  CPU only."""
import os

import numpy as np
import pytest

import oracle
from tests import cases, inputs

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32 if a.dtype == np.float32 else a.dtype)


@pytest.mark.parametrize("shape", cases.SGEMM_CASES)
def test_sgemm_port_matches_fixture(port, golden, shape):
    M, N, K = shape
    A, B, C0 = cases.sgemm_inputs(M, N, K)
    C = port.sgemm(A, B, C0.copy())
    assert np.array_equal(bits(C), bits(golden[f"sgemm_{M}x{N}x{K}"]))


@pytest.mark.parametrize("shape", cases.SGEMM_DIGEST_CASES)
def test_sgemm_port_matches_digest(port, golden, shape):
    M, N, K = shape
    A, B, C0 = cases.sgemm_inputs(M, N, K)
    port.set_threads(os.cpu_count() or 1)  # threads split rows: the bits do not depend on them
    try:
        C = port.sgemm(A, B, C0.copy())
    finally:
        port.set_threads(1)
    assert cases.digest(C) == str(golden[f"sgemm_{M}x{N}x{K}_sha256"])
    assert np.array_equal(bits(cases.sample(C)), bits(golden[f"sgemm_{M}x{N}x{K}_sample"]))


def test_sgemm_blocked_equals_naive_chain(port):
    A, B, C0 = cases.sgemm_inputs(37, 1100, 300)
    assert np.array_equal(bits(port.sgemm(A, B, C0.copy())), bits(port.sgemm(A, B, C0.copy(), naive=True)))


def test_sgemm_threads_do_not_change_bits(port):
    A, B, C0 = cases.sgemm_inputs(64, 200, 300)
    one = port.sgemm(A, B, C0.copy())
    port.set_threads(4)
    try:
        four = port.sgemm(A, B, C0.copy())
    finally:
        port.set_threads(1)
    assert np.array_equal(bits(one), bits(four))


def test_ssyrk_port_equals_sgemm_port_on_the_triangle(port):
    """The reference has no SSYRK kernel (only an MKL benchmark); the restatement is pinned
    to the SGEMM restatement on (A, A^T), which is itself pinned to the reference."""
    A = inputs.uniform_f32(31, (97, 130))
    C0 = inputs.uniform_f32(32, (97, 97))
    got = port.ssyrk(A, C0.copy())
    full = port.sgemm(A, np.ascontiguousarray(A.T), C0.copy())
    up = np.triu(np.ones((97, 97), bool))
    assert np.array_equal(bits(got)[up], bits(full)[up])
    assert np.array_equal(bits(got)[~up], bits(C0)[~up])


def test_sgemm_close_to_fp64(port):
    """The reference's own tolerance for SGEMM is 3 decimals (tests/test_x86.py:151-161)."""
    A, B, C0 = cases.sgemm_inputs(100, 100, 1000)
    C = port.sgemm(A, B, C0.copy())
    np.testing.assert_almost_equal(C, C0.astype(np.float64) + A.astype(np.float64) @ B.astype(np.float64), decimal=3)


def test_conv_specialized_fixture(port, golden):
    src, wts, bias = inputs.conv_instance_fill(5, 82, 102, 128, 128, 3)
    if cases.digest(src) + cases.digest(wts) + cases.digest(bias) != str(golden["conv_specialized_inputs_sha256"]):
        pytest.skip("libm on this machine rounds cos/sin/tanh differently from the fixture's")
    out = port.conv(src, wts, bias)
    assert cases.digest(out) == str(golden["conv_specialized_sha256"])


def test_conv_specialized_uniform_fixture(port, golden):
    src = inputs.uniform_f32(11, (5, 82, 102, 128))
    wts = inputs.uniform_f32(12, (128, 3, 3, 128))
    bias = inputs.uniform_f32(13, (128,))
    out = port.conv(src, wts, bias)
    assert cases.digest(out) == str(golden["conv_specialized_uniform_sha256"])
    assert np.array_equal(bits(cases.sample(out)), bits(golden["conv_specialized_uniform_sample"]))


def test_conv_layouts_agree(port):
    """conv (CiKhKwCo, caller-padded) == conv_nhwc (KhKwCiCo, pad in the kernel)
    == im2col + SGEMM with C pre-set to bias, then ReLU."""
    inp = inputs.uniform_f32(21, (2, 9, 11, 8))
    w = inputs.uniform_f32(22, (3, 3, 8, 16))
    bias = inputs.uniform_f32(23, (16,))
    out = port.conv_nhwc(inp, w, bias, pad=1, relu=True)
    padded = np.zeros((2, 11, 13, 8), np.float32)
    padded[:, 1:-1, 1:-1, :] = inp
    out2 = port.conv(padded, np.ascontiguousarray(w.transpose(2, 0, 1, 3)), bias)
    assert np.array_equal(bits(out), bits(out2))
    col = port.im2col_nhwc(inp, 3, 1)
    C = np.tile(bias, (col.shape[0], 1)).astype(np.float32)
    port.sgemm(col, np.ascontiguousarray(w.reshape(-1, 16)), C)
    C = np.where(C > 0, C, np.float32(0)).astype(np.float32)
    assert np.array_equal(bits(C.reshape(out.shape)), bits(out))


def test_strided_conv_restatement_reduces_to_the_unit_stride_one(port):
    """stride 1 is the pinned conv_nhwc; stride 2 equals every second output of it when the sizes line up."""
    inp = inputs.uniform_f32(41, (2, 9, 11, 4))
    w = inputs.uniform_f32(42, (3, 3, 4, 8))
    bias = inputs.uniform_f32(43, (8,))
    full = port.conv_nhwc(inp, w, bias, 1, True)
    assert np.array_equal(bits(port.conv_nhwc_strided(inp, w, bias, 1, 1, True)), bits(full))
    assert np.array_equal(bits(port.conv_nhwc_strided(inp, w, bias, 1, 2, True)), bits(np.ascontiguousarray(full[:, ::2, ::2])))


@pytest.mark.parametrize("name", list(cases.I8_CASES))
def test_i8_port_matches_fixture(port, golden, name):
    A, B, scale, act = cases.i8_inputs(name)
    assert np.array_equal(port.matmul_i8(A, B, scale, act), golden[f"i8_{name}"])


def test_i8_ties(port, golden):
    A, B = cases.i8_tie_inputs()
    got = port.matmul_i8(A, B, 1.0 / 256, False)
    assert np.array_equal(got, golden["i8_ties_s256"])
    assert np.array_equal(port.matmul_i8(A, B, 1.0 / 512, True), golden["i8_ties_s512_relu"])
    # the fixture really contains ties resolved to even in both directions
    acc = A.astype(np.int64) @ B.astype(np.int64)
    tie = (acc % 256 == 128) & (np.abs(acc) < 127 * 256)
    assert tie.sum() > 100
    q = acc[tie] / 256.0
    assert np.array_equal(got[tie].astype(np.int64) % 2, np.zeros(tie.sum(), np.int64))
    assert ((got[tie] > q).any() and (got[tie] < q).any())


def test_i8_large_acc_rounding(port):
    """|acc| > 2^24 so that int32 -> fp32 itself rounds; small scale keeps the
    result in range.  Checked against exact integer arithmetic done here."""
    K = 4096
    A = np.full((4, K), 127, np.int8)
    B = np.full((K, 8), 127, np.int8)
    B[:5, 1] = 126
    B[:3, 2] = 125
    A[1, :7] = 126
    acc = A.astype(np.int64) @ B.astype(np.int64)
    assert (np.abs(acc) > 2 ** 24).all()
    scale = np.float32(2.0 ** -19)
    want = np.clip(np.rint(acc.astype(np.float32) * scale), -128, 127).astype(np.int8)
    assert np.array_equal(port.matmul_i8(A, B, float(scale), False), want)


@pytest.mark.parametrize("name", list(oracle.REF_MATMUL_SHAPES))
def test_i8_reference_shapes(port, golden, name):
    N, M, K = oracle.REF_MATMUL_SHAPES[name]
    x, y = inputs.gemmini_matmul_fill(N, M, K)
    assert cases.digest(port.matmul_i8(x, y, 2.0, False)) == str(golden[f"i8_runner_{name}_sha256"])
    A = inputs.int8(700 + N % 97, (N, K), -16, 15)
    B = inputs.int8(701 + M % 89, (K, M), -16, 15)
    assert cases.digest(port.matmul_i8(A, B, 1.0 / 64, True)) == str(golden[f"i8_shape_{name}_sha256"])


@pytest.mark.parametrize("name", list(oracle.REF_CONV_I8_SHAPES))
def test_i8_conv_reference_shapes(port, golden, name):
    b, od, co, kd, ci, ind = oracle.REF_CONV_I8_SHAPES[name]
    inp, w, bias = inputs.gemmini_conv_fill(b, ind, ci, co, kd)
    assert cases.digest(port.conv_i8(inp, w, bias, 1.0, False)) == str(golden[f"i8conv_runner_{name}_sha256"])
    inp = inputs.int8(800 + ci, (b, ind, ind, ci), -16, 15)
    w = inputs.int8(801 + co, (kd, kd, ci, co), -16, 15)
    bias = inputs.int32(802, (1, co), -5000, 5000)
    assert cases.digest(port.conv_i8(inp, w, bias, 1.0 / 128, True)) == str(golden[f"i8conv_seeded_{name}_sha256"])


def test_bf16_helpers(port):
    x = inputs.uniform_f32(5, (1000,))
    b = port.bf16_round(x)
    assert np.array_equal(b, inputs.f32_to_bf16_bits(x))
    assert np.array_equal(bits(port.bf16_widen(b)), bits(inputs.bf16_bits_to_f32(b)))
    A = inputs.normal_bf16(6, (33, 64))
    Bt = inputs.normal_bf16(7, (17, 64))
    C = port.bf16_widen(port.gemm_bf16(A, Bt))
    ref = inputs.bf16_bits_to_f32(A).astype(np.float64) @ inputs.bf16_bits_to_f32(Bt).astype(np.float64).T
    assert np.abs(C - ref).max() <= 2.0 ** -8 * np.abs(ref).max() + 1e-6


# --- direct comparison with the compiled reference, where available -------
@pytest.mark.ref
@pytest.mark.parametrize("shape", [(7, 65, 513), (264, 64, 512), (265, 129, 1030), (1, 4099, 77)])
def test_sgemm_port_equals_compiled_reference(port, ref, shape):
    M, N, K = shape
    A, B, C0 = cases.sgemm_inputs(M, N, K, seed=99)
    assert np.array_equal(bits(port.sgemm(A, B, C0.copy())), bits(ref.sgemm(A, B, C0.copy())))


@pytest.mark.ref
def test_i8_port_equals_compiled_reference(port, ref):
    A = inputs.int8(31, (512, 512), -30, 30)
    B = inputs.int8(32, (512, 512), -30, 30)
    for scale, act in [(1 / 256, True), (0.0173, False), (1.0, False)]:
        assert np.array_equal(port.matmul_i8(A, B, scale, act), ref.matmul_i8("512x512x512", A, B, scale, act))
