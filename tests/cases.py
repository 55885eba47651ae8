"""The parity cases shared by the fixture generator (tests/golden/make_golden.py),
the oracle tests and the GPU parity tests.  Each case rebuilds its inputs from
a seed (tests/inputs.py), so a fixture only has to hold outputs."""
import hashlib

import numpy as np

from tests import inputs

# (M, N, K): covers K-blocks > 512, all panel kernels of the reference
# schedule (N % 64, M % 6), the scalar corner, GEMV-like shapes.
SGEMM_CASES = [
    (1, 1, 1), (5, 63, 7), (6, 64, 512), (17, 130, 33), (100, 100, 1000),
    (263, 65, 1025), (17, 4099, 513), (530, 129, 600), (1, 2048, 1030), (256, 256, 256),
]
# shapes added after the fixture was generated are checked against the oracle port only
SGEMM_EXTRA_CASES = [(1500, 8, 515), (2048, 16, 64), (1025, 13, 130), (3000, 1, 33), (20000, 5, 40), (4, 512, 300), (2, 8192, 1024), (3, 70, 1000), (4, 33, 31), (2, 4099, 97), (5, 64, 40), (32, 100, 513), (64, 64, 64), (65, 129, 17),
                     (1, 6404, 700), (2, 7000, 515),
                     (8, 8192, 300), (5, 8196, 129), (7, 8193, 65),
                     (1100, 11, 77), (1024, 12, 64),
                     (8, 32768, 70), (6, 40001, 33), (16, 16384, 40), (13, 70, 90)]  # the engine's 8- and 16-row tiles  # + the tall kernel with three column quads  # + the skinny kernel (a handful of rows, >= 8192 columns)  # the TMA-fed GEMV kernel with a partial last strip and a ragged K tail
# large outputs are held as SHA-256 + a strided sample: the remaining shapes of the fp32 shape sweep
SGEMM_DIGEST_CASES = [(1000, 1000, 1000), (1024, 1024, 1024), (512, 512, 512), (2048, 2048, 2048),
                      (4096, 64, 4096), (1, 8192, 8192)]

# name -> (N, M, K, value range, scale, act)
I8_CASES = {
    "full_s256": (512, 512, 512, (-128, 127), 1.0 / 256, False),
    "full_s256_relu": (512, 512, 512, (-128, 127), 1.0 / 256, True),
    "small_s256": (512, 512, 512, (-8, 7), 1.0 / 256, False),
    "small_s03_relu": (512, 512, 512, (-8, 7), 0.3, True),
    "unit_s1": (512, 512, 512, (-1, 1), 1.0, True),
    "small_s2": (512, 512, 512, (-2, 2), 2.0, False),
}


def sgemm_inputs(M, N, K, seed=None):
    seed = seed if seed is not None else (M * 1000003 + N * 1009 + K)
    A = inputs.uniform_f32(seed, (M, K))
    B = inputs.uniform_f32(seed + 1, (K, N))
    C0 = inputs.uniform_f32(seed + 2, (M, N))
    return A, B, C0


def i8_inputs(name):
    N, M, K, (lo, hi), scale, act = I8_CASES[name]
    seed = sum(map(ord, name))
    A = inputs.int8(seed, (N, K), lo, hi)
    B = inputs.int8(seed + 1, (K, M), lo, hi)
    return A, B, scale, act


def i8_tie_inputs():
    """Crafted so that acc/256 hits exact .5 ties with even and odd quotients,
    and |acc| > 2^24 rows (K = 4096) for the int32 -> float rounding; see the
    measurement notes on the int8 epilogue."""
    K = 512
    A = np.zeros((512, K), np.int8)
    B = np.zeros((K, 512), np.int8)
    # row i, col j: acc = (i - 256) * 128 + j * 256  -> acc/256 = (i-256)/2 + j
    A[:, 0] = np.clip(np.arange(512) - 256, -128, 127).astype(np.int8)
    A[:, 1] = (np.arange(512) - 256 - A[:, 0].astype(np.int64)).astype(np.int8)
    B[0, :] = 127
    B[1, :] = 127
    A[:, 2] = 1
    B[2, :] = (np.arange(512) % 7 - 3).astype(np.int8)
    A[:, 3] = (np.arange(512) - 256 - A[:, 0].astype(np.int64) - A[:, 1].astype(np.int64)).astype(np.int8)
    B[3, :] = 1
    return A, B


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def sample(a: np.ndarray, step: int = 1009) -> np.ndarray:
    return np.ascontiguousarray(a).reshape(-1)[::step].copy()
