"""matmul_on_cpu_static -- the int8 matmul for callers that cannot allocate.

Some users of this library need a matmul at a point where device allocation is
off the table: under a framework arena that owns all device memory, inside a
fixed memory budget, or in a loop where the synchronisation hidden inside
cudaMalloc would break a latency budget.  For them the library keeps the
scratch of one kernel (the K-major copy of B) in a fixed array inside the
library image.  This test calls that entry point through the C ABI twice in a
row (different shapes, so the second call sees the first call's leftovers in
the shared array) and requires bit-identical results to the regular entry
point and to the CPU oracle.

The file name sorts last on purpose: a run that stops at the first failure has
already run every other test by the time it gets here.
"""
import ctypes

import numpy as np
import pytest

import oracle
from tests import inputs

pytestmark = pytest.mark.gpu


def _call_static(lib, stream, N, M, K, scale, act, dA, dB, dC):
    s = np.array([scale], np.float32)
    lib.dll.matmul_on_cpu_static(ctypes.c_void_p(stream), N, M, K, ctypes.c_void_p(s.ctypes.data), act,
                                 ctypes.c_void_p(dA.data_ptr()), ctypes.c_void_p(dB.data_ptr()),
                                 ctypes.c_void_p(dC.data_ptr()))
    return lib.dll.exo_b200_last_error()


def test_static_scratch_matches_regular_entry_point_twice():
    import torch

    import exo_b200

    lib = exo_b200.library()
    stream = torch.cuda.current_stream().cuda_stream
    # first call: fills most of the 4 MiB array; second: smaller, ragged M, other values
    for (N, M, K, lo, hi, scale, act) in [(384, 2048, 2048, -128, 127, 1.0 / 256, False),
                                          (200, 328, 1040, -9, 9, 0.37, True)]:
        A = inputs.int8(N + 1, (N, K), lo, hi)
        B = inputs.int8(M + 2, (K, M), lo, hi)
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        want = torch.empty((N, M), dtype=torch.int8, device="cuda")
        lib.matmul_on_cpu(None, N, M, K, float(scale), act, dA, dB, want)
        got = torch.full((N, M), 77, dtype=torch.int8, device="cuda")
        assert _call_static(lib, stream, N, M, K, scale, act, dA, dB, got) == 0, \
            lib.dll.exo_b200_last_error_string()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert np.array_equal(got.cpu().numpy(), oracle.port().matmul_i8(A, B, scale, act))
        assert lib.dll.exo_b200_synchronize(None) == 0  # no device-side timeout was recorded


def test_static_scratch_rejects_what_does_not_fit():
    import torch

    import exo_b200

    lib = exo_b200.library()
    N, M, K = 16, 4096, 2048  # K * M = 8 Mi > 4 Mi
    dA = torch.zeros((N, K), dtype=torch.int8, device="cuda")
    dB = torch.zeros((K, M), dtype=torch.int8, device="cuda")
    dC = torch.full((N, M), 5, dtype=torch.int8, device="cuda")
    code = _call_static(lib, 0, N, M, K, 1.0, False, dA, dB, dC)
    assert code == exo_b200.ERR_UNSUPPORTED
    assert b"static scratch" in lib.dll.exo_b200_last_error_string()
    torch.cuda.synchronize()
    assert bool((dC == 5).all())
    # host buffers would need staging allocations: rejected too
    hA = np.zeros((16, 16), np.int8)
    s = np.array([1.0], np.float32)
    lib.dll.matmul_on_cpu_static(None, 16, 16, 16, s.ctypes.data, False, hA.ctypes.data, hA.ctypes.data, hA.ctypes.data)
    assert lib.dll.exo_b200_last_error() == exo_b200.ERR_INVALID_ARGUMENT


def test_static_scratch_rejects_operands_of_another_device():
    """The scratch array and the launch belong to the current device, so operands that live
    on a different GPU are refused instead of being dereferenced from the wrong device."""
    import torch

    import exo_b200

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = exo_b200.library()
    with torch.cuda.device(1):
        dA = torch.zeros((16, 16), dtype=torch.int8, device="cuda:1")
        dC = torch.full((16, 16), 5, dtype=torch.int8, device="cuda:1")
    torch.cuda.set_device(0)
    code = _call_static(lib, 0, 16, 16, 16, 1.0, False, dA, dA, dC)
    assert code == exo_b200.ERR_INVALID_ARGUMENT
    assert b"device" in lib.dll.exo_b200_last_error_string()
    assert bool((dC == 5).all())
