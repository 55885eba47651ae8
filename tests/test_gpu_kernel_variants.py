"""Every shipped tensor-core kernel variant against the oracle, the headline
kernel at the headline shape, and guard bands around ragged outputs.

The bf16 and int8 GEMMs have three kernels each way (single CTA, CTA pair with a
256 x 256 tile, CTA pair with a 512 x 256 tile); which one a call takes depends
on the tile count.  The default dispatch only reaches the pair kernels at sizes
the CPU oracle cannot finish, so the variants are forced through the library's
EXOB200_* switches -- read once per process, hence one child process per case
(tests/forced_kernel_check.py) -- on the 2048^3 sub-block that the large bf16
workload prescribes for its reference comparison, and on ragged shapes.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import cases, inputs
from tests.forced_kernel_check import bf16_tolerance
from tests.guard import Guarded

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_forced(env, *args):
    e = dict(os.environ)
    e.update(env)
    r = subprocess.run([sys.executable, "-m", "tests.forced_kernel_check", *map(str, args)], cwd=ROOT, env=e,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    assert r.stdout.strip().splitlines()[-1].startswith("OK"), r.stdout
    return r.stdout


VARIANTS_BF16 = {
    "pair_512x256": {"EXOB200_TC2": "1", "EXOB200_TC2_TALL": "1"},  # gemm_tc2t_kernel: the headline kernel
    "pair_256x256": {"EXOB200_TC2": "1", "EXOB200_TC2_TALL": "0"},  # gemm_tc2_kernel<bf16>
    "single_cta": {"EXOB200_TC2": "0"},                            # gemm_tc_kernel<bf16>
    "pair_512x256_direct_stores": {"EXOB200_TC2": "1", "EXOB200_TC2_TALL": "1", "EXOB200_TC2T_DIRECT": "1"},
}


@pytest.mark.parametrize("variant", list(VARIANTS_BF16))
@pytest.mark.parametrize("shape", [(2048, 2048, 2048), (1100, 776, 520), (513, 264, 72), (300, 1001, 136),
                                   (5000, 2040, 72)])  # 80 tiles of 512 x 256: a last round of 6, split into halves
def test_bf16_kernel_variant_against_reference_sgemm(variant, shape):
    """The 2048^3 sub-block (and two ragged shapes: M, N and K all off the tile
    sizes) through each kernel, against the reference fp32 SGEMM chain on the
    widened inputs rounded once to bf16."""
    run_forced(VARIANTS_BF16[variant], "bf16", *shape)


# The exact-fp32 engine's tile configurations (the default dispatch picks one per shape from a cost table;
# here each is forced onto the same ragged shape: M, N and K off every tile size, several tiles each way).
FFMA_TILES = ["128", "12864", "6464", "64", "32", "3224", "1664", "8128"]


@pytest.mark.parametrize("scalar", ["0", "1"])
@pytest.mark.parametrize("tile", FFMA_TILES)
def test_ffma_tile_configuration_bit_exact(tile, scalar):
    if scalar == "1" and tile not in ("128", "6464"):
        pytest.skip("the one-FMA-per-instruction build is a timing aid; two configurations cover its code")
    run_forced({"EXOB200_FFMA_TILE": tile, "EXOB200_FFMA_SCALAR": scalar}, "ffma", 300, 333, 77)


@pytest.mark.parametrize("shape", [(17, 4099, 513), (32, 8192, 300), (12, 1000, 700)])
def test_skinny_kernel_beyond_its_default_range(shape):
    """The skinny-M kernel is only dispatched for at most 8 rows and at least 8192 columns; it accepts up to
    32 rows, so that range is forced here."""
    run_forced({"EXOB200_SKINNY_MAX_M": "32"}, "sgemm", *shape)


@pytest.mark.parametrize("variant,env", [("pair_256x256", {"EXOB200_TC2": "1", "EXOB200_TC2_TALL": "0"}),
                                         ("pair_512x256", {"EXOB200_TC2": "1", "EXOB200_TC2_TALL": "1"}),
                                         ("single_cta", {"EXOB200_TC2": "0"}),
                                         ("single_cta_transposed_b", {"EXOB200_TC2": "0", "EXOB200_I8_TRANSPOSE": "1"})])
@pytest.mark.parametrize("shape", [(2048, 2048, 2048), (1000, 528, 272), (5000, 2048, 272)])
def test_i8_kernel_variant_bit_exact(variant, env, shape):
    run_forced(env, "i8", *shape)


def test_bf16_headline_shape_rows_against_oracle(port, torch_mod):
    """The large bf16 workload itself (M=32768, N=16384, K=8192: 64 tiles of
    512 x 256 per CTA pair, 128 k-blocks, 32 trips round the four-stage ring) on
    device buffers.  Rows of C are independent, so a sample of rows -- first and
    last of the problem, of a 512-row tile, of its 256-row halves and of each
    CTA's 128 rows -- is run through the oracle at full N and K."""
    torch = torch_mod
    import exo_b200

    lib = exo_b200.library()
    M, N, K = 32768, 16384, 8192
    g = torch.Generator(device="cuda").manual_seed(2024)
    A = (torch.randn((M, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    B = (torch.randn((N, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)  # column-major K x N
    out = Guarded(torch, (M, N), torch.bfloat16)
    lib.gemm_bf16_exo(None, M, N, K, A, B, out.view)
    torch.cuda.synchronize()
    assert out.bands_intact()
    rows = [0, 1, 127, 128, 255, 256, 383, 384, 511, 512, 16383, 16384, 20000, 31020, 31237, 32255, 32256, M - 129, M - 2,
            M - 1]  # the last four tile rows hold the half tiles of the split last round
    idx = torch.tensor(rows, device="cuda")
    got_bits = out.view[idx].view(torch.int16).cpu().numpy().view(np.uint16)
    A_rows = A[idx].view(torch.int16).cpu().numpy().view(np.uint16)
    B_host = B.view(torch.int16).cpu().numpy().view(np.uint16)
    port.set_threads(os.cpu_count() or 1)
    try:
        ref = inputs.bf16_bits_to_f32(port.gemm_bf16(A_rows, B_host))
    finally:
        port.set_threads(1)
    got = inputs.bf16_bits_to_f32(got_bits)
    err = np.abs(got - ref)
    assert (err <= bf16_tolerance(ref, K)).all(), f"max err {err.max():.3e}"
    assert (got == ref).mean() > 0.9
    # every element of the output was written (a bf16 0xA5A5 is about -2.9e-16: no sum of these inputs lands there)
    flat = out.view.view(torch.int16).view(-1)
    step = 1 << 26
    for s in range(0, flat.numel(), step):
        assert not bool((flat[s:s + step] == 0xA5A5 - 65536).any())


def test_sgemm_ffma_8192_cubed_rows_against_oracle(port, torch_mod):
    """The largest square of the fp32 shape sweep on the exact path: a row sample
    of the full-size launch, bit for bit."""
    torch = torch_mod
    import exo_b200

    lib = exo_b200.library()
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(8192)
    dA = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
    dB = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
    dC = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
    rows = [0, 1, 63, 64, 127, 128, 4095, 4096, 8063, 8064, n - 2, n - 1]
    C0 = dC[rows].cpu().numpy()
    lib.sgemm_exo(None, n, n, n, dA, dB, dC)
    torch.cuda.synchronize()
    port.set_threads(os.cpu_count() or 1)
    try:
        want = port.sgemm(dA[rows].cpu().numpy(), dB.cpu().numpy(), C0.copy())
    finally:
        port.set_threads(1)
    assert np.array_equal(dC[rows].cpu().numpy().view(np.uint32), want.view(np.uint32))


# ----------------------------------------------------------------- guard bands
def _f32_bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("shape", [(130, 70, 72), (385, 1000, 264), (129, 257, 40)])
def test_guard_bands_bf16(port, torch_mod, shape):
    torch = torch_mod
    import exo_b200

    lib = exo_b200.library()
    M, N, K = shape
    A, Bt = inputs.normal_bf16(91, (M, K)), inputs.normal_bf16(92, (N, K))
    out = Guarded(torch, (M, N), torch.int16)
    lib.gemm_bf16_exo(None, M, N, K, torch.from_numpy(A.view(np.int16)).cuda(), torch.from_numpy(Bt.view(np.int16)).cuda(),
                      out.view)
    torch.cuda.synchronize()
    assert out.bands_intact()
    got = inputs.bf16_bits_to_f32(out.view.cpu().numpy().view(np.uint16))
    ref = inputs.bf16_bits_to_f32(port.gemm_bf16(A, Bt))
    assert (np.abs(got - ref) <= bf16_tolerance(ref, K)).all()


@pytest.mark.parametrize("shape", [(130, 304, 272), (257, 129, 4096), (5, 7, 17), (1000, 520, 272)])
def test_guard_bands_int8(port, torch_mod, shape):
    torch = torch_mod
    import exo_b200

    lib = exo_b200.library()
    N, M, K = shape
    A, B = inputs.int8(N + K, (N, K), -20, 20), inputs.int8(M + K + 1, (K, M), -20, 20)
    out = Guarded(torch, (N, M), torch.int8)
    lib.matmul_on_cpu(None, N, M, K, 0.013, True, torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), out.view)
    torch.cuda.synchronize()
    assert out.bands_intact()
    assert np.array_equal(out.view.cpu().numpy(), port.matmul_i8(A, B, 0.013, True))


@pytest.mark.parametrize("shape", [(300, 77, 129), (1030, 2049, 513), (130, 260, 96)])
@pytest.mark.parametrize("path", ["ffma", "3xtf32"])
def test_guard_bands_sgemm(port, torch_mod, shape, path):
    torch = torch_mod
    import exo_b200

    lib = exo_b200.library()
    M, N, K = shape
    A, B, C0 = cases.sgemm_inputs(M, N, K, seed=31)
    out = Guarded(torch, (M, N), torch.float32)
    out.view.copy_(torch.from_numpy(C0))
    fn = lib.sgemm_exo_ffma if path == "ffma" else lib.sgemm_exo_3xtf32
    fn(None, M, N, K, torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), out.view)
    torch.cuda.synchronize()
    assert out.bands_intact()
    got = out.view.cpu().numpy()
    if path == "ffma":
        assert np.array_equal(_f32_bits(got), _f32_bits(port.sgemm(A, B, C0.copy())))
    else:
        ref = C0.astype(np.float64) + A.astype(np.float64) @ B.astype(np.float64)
        S = np.abs(C0) + np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
        bound = 1.5e-6 + 1e-6 * min(K, 1024) / 1024.0 + 1e-7 * K / 1024.0
        assert (np.abs(got - ref) <= bound * S).all()


@pytest.mark.parametrize("cfg", [(2, 9, 11, 8, 16, 3, 1), (1, 20, 150, 12, 36, 3, 2), (3, 6, 6, 4, 130, 5, 2),
                                 (1, 7, 5, 3, 5, 3, 0)])
@pytest.mark.parametrize("path", ["ffma", "3xtf32"])
def test_guard_bands_conv_fp32(port, torch_mod, cfg, path):
    torch = torch_mod
    import exo_b200

    lib = exo_b200.library()
    b, h, w, ci, co, k, pad = cfg
    inp = inputs.uniform_f32(121, (b, h, w, ci))
    wts = inputs.uniform_f32(122, (k, k, ci, co))
    bias = inputs.uniform_f32(123, (co,))
    oh, ow = h + 2 * pad - k + 1, w + 2 * pad - k + 1
    out = Guarded(torch, (b, oh, ow, co), torch.float32)
    fn = lib.conv_nhwc_exo if path == "ffma" else lib.conv_nhwc_exo_3xtf32
    fn(None, b, h, w, ci, co, k, pad, True, torch.from_numpy(inp).cuda(), out.view, torch.from_numpy(wts).cuda(),
       torch.from_numpy(bias).cuda())
    torch.cuda.synchronize()
    assert out.bands_intact()
    want = port.conv_nhwc(inp, wts, bias, pad, True)
    got = out.view.cpu().numpy()
    if path == "ffma":
        assert np.array_equal(_f32_bits(got), _f32_bits(want))
    else:
        S = port.conv_nhwc(np.abs(inp), np.abs(wts), np.abs(bias), pad, False).astype(np.float64)
        bound = 1.5e-6 + 1e-6 * min(k * k * ci, 1024) / 1024.0 + 1e-7 * k * k * ci / 1024.0 + 2e-7
        assert (np.abs(got.astype(np.float64) - want) <= bound * S).all()


@pytest.mark.parametrize("cfg", [(2, 19, 32, 48, 3), (3, 12, 144, 272, 3), (2, 11, 24, 40, 3), (1, 130, 16, 32, 3)])
def test_guard_bands_conv_int8(port, torch_mod, cfg):
    torch = torch_mod
    import exo_b200

    lib = exo_b200.library()
    b, ind, ci, co, k = cfg
    od = ind - k + 1
    inp = inputs.int8(900 + ind, (b, ind, ind, ci), -20, 20)
    w = inputs.int8(901 + co, (k, k, ci, co), -20, 20)
    bias = inputs.int32(902, (1, co), -3000, 3000)
    out = Guarded(torch, (b, od, od, co), torch.int8)
    lib.conv_on_cpu_stride_1(None, b, od, co, k, ci, ind, out.view, torch.from_numpy(bias).cuda(),
                             torch.from_numpy(inp).cuda(), torch.from_numpy(w).cuda(), True, 1.0 / 64)
    torch.cuda.synchronize()
    assert out.bands_intact()
    assert np.array_equal(out.view.cpu().numpy(), port.conv_i8(inp, w, bias, 1.0 / 64, True))
