"""Deterministic test inputs that do not depend on numpy's RNG streams.

A counter-based generator: element i of a tensor is a splitmix64-style hash of
(seed, i), so every machine produces the same bits.  Distributions follow the
workload definitions: fp32 uniform in [-1, 1) on a 2^-23 grid, int8 uniform in
[-128, 127], bf16 N(0,1) * 0.02 (Box-Muller in float64, rounded to bf16).
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _hash(seed: int, n: int, stream: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        x += np.uint64((seed * 0xD1B54A32D192ED03 + stream * 0x8CB92BA72F3D8DD7) & 0xFFFFFFFFFFFFFFFF)
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return x


def uniform_f32(seed: int, shape) -> np.ndarray:
    n = int(np.prod(shape))
    bits = (_hash(seed, n) >> np.uint64(40)).astype(np.float32)  # 24 bits
    return (bits * np.float32(2.0 ** -23) - np.float32(1.0)).reshape(shape)


def int8(seed: int, shape, lo: int = -128, hi: int = 127) -> np.ndarray:
    n = int(np.prod(shape))
    h = _hash(seed, n) >> np.uint64(33)
    span = hi - lo + 1
    return ((h % np.uint64(span)).astype(np.int64) + lo).astype(np.int8).reshape(shape)


def int32(seed: int, shape, lo: int, hi: int) -> np.ndarray:
    n = int(np.prod(shape))
    h = _hash(seed, n) >> np.uint64(33)
    return ((h % np.uint64(hi - lo + 1)).astype(np.int64) + lo).astype(np.int32).reshape(shape)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))
    return (u >> np.uint64(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16(seed: int, shape, std: float = 0.02) -> np.ndarray:
    """bf16 bit patterns (uint16) of N(0,1)*std."""
    n = int(np.prod(shape))
    u1 = ((_hash(seed, n, 1) >> np.uint64(11)).astype(np.float64) + 1.0) * 2.0 ** -53
    u2 = (_hash(seed, n, 2) >> np.uint64(11)).astype(np.float64) * 2.0 ** -53
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return f32_to_bf16_bits((z * std).astype(np.float32)).reshape(shape)


def conv_instance_fill(n, ih, iw, ci, co, k):
    """The deterministic fill of the reference's conv harness
    (apps/x86/conv/conv_instance.hpp:52-60): src = cos(i/10), weights =
    sin(2i), bias = tanh(i) over a float counter, evaluated in float64 from the
    float32 argument and rounded once (a correctly rounded cosf/sinf/tanhf)."""
    def gen(count, f):
        i = np.arange(count, dtype=np.float32)
        return f(i).astype(np.float32)
    src = gen(n * ih * iw * ci, lambda i: np.cos((i / np.float32(10)).astype(np.float64)))
    wts = gen(co * ci * k * k, lambda i: np.sin((i * np.float32(2)).astype(np.float64)))
    bias = gen(co, lambda i: np.tanh(i.astype(np.float64)))
    return src.reshape(n, ih, iw, ci), wts.reshape(ci, k, k, co), bias


def gemmini_matmul_fill(N, M, K):
    """apps/gemmini/test/run_matmul.c:37-47: x[i,j] = i + 2j, y[i,j] = 3j + i,
    wrapped to int8."""
    i = np.arange(N, dtype=np.int64)[:, None]
    j = np.arange(K, dtype=np.int64)[None, :]
    x = (i + 2 * j).astype(np.int8)
    i = np.arange(K, dtype=np.int64)[:, None]
    j = np.arange(M, dtype=np.int64)[None, :]
    y = (3 * j + i).astype(np.int8)
    return x, y


def gemmini_conv_fill(batch, in_dim, in_c, out_c, kdim):
    """apps/gemmini/test/run_conv.c:41-68 (its index arithmetic taken literally,
    flat arrays reinterpreted in the kernels' NHWC / KhKwCiCo layouts)."""
    bias = (-np.arange(out_c, dtype=np.int32)).reshape(1, out_c)
    inp = np.zeros(batch * in_dim * in_dim * in_c, np.int8)
    j = np.arange(in_dim)[:, None, None]
    k = np.arange(in_dim)[None, :, None]
    r = np.arange(out_c)[None, None, :]
    blk = (j + k + r * 3).astype(np.int8)
    for i in range(batch):
        base = in_dim * in_dim * out_c * i
        idx = (in_dim * out_c * j + out_c * k + r + base).reshape(-1)
        ok = idx < inp.size
        inp[idx[ok]] = blk.reshape(-1)[ok]
    w = np.zeros(out_c * kdim * kdim * in_c, np.int8)
    i = np.arange(out_c)[:, None, None, None]
    j = np.arange(kdim)[None, :, None, None]
    k = np.arange(kdim)[None, None, :, None]
    r = np.arange(in_c)[None, None, None, :]
    val = np.broadcast_to((i + k * 3 + r).astype(np.int8), (out_c, kdim, kdim, in_c))
    idx = kdim * kdim * in_c * i + kdim * in_c * j + in_c * k + r
    w[idx.reshape(-1)] = val.reshape(-1)
    return (inp.reshape(batch, in_dim, in_dim, in_c), w.reshape(kdim, kdim, in_c, out_c), bias)
