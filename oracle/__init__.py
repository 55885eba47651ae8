"""TEST INFRASTRUCTURE: the CPU oracle for the GEMM / convolution hot path.

Two checkers live here, neither of which the product package may import:

* ``port``  -- ``exo_oracle.c``, a restatement of the reference algorithms
  (compiled on demand with gcc into ``oracle/libexo_oracle.so``);
* ``ref``   -- ``oracle/_ref/libexo_ref.so``, the reference's own
  exocc-generated C compiled by ``oracle/build_ref.py`` (present only where a
  reference checkout was available at build time; needs AVX-512F to run).

Both are exposed as numpy-in / numpy-out functions.  Parity of ``port``
against ``ref`` and against the committed fixtures is tested in
``tests/test_oracle.py``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SRC = os.path.join(HERE, "exo_oracle.c")
PORT_SO = os.path.join(HERE, "libexo_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libexo_ref.so")

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p


def build_port(force: bool = False) -> str:
    """Compile exo_oracle.c (a second or two)."""
    if force or not os.path.exists(PORT_SO) or os.path.getmtime(PORT_SO) < os.path.getmtime(PORT_SRC):
        flags = ["-mfma", "-mavx2"] if _cpu_has("fma") and _cpu_has("avx2") else []
        subprocess.run(["gcc", "-O3", "-fPIC", "-shared", "-fopenmp", *flags, PORT_SRC,
                        "-o", PORT_SO, "-lm"], check=True)
    return PORT_SO


def _cpu_has(flag: str) -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return flag in line.split()
    except OSError:
        pass
    return False


def _ptr(a: np.ndarray) -> _vp:
    assert a.flags["C_CONTIGUOUS"]
    return _vp(a.ctypes.data)


class Port:
    """ctypes view of libexo_oracle.so (the restatement)."""

    def __init__(self):
        self.lib = ctypes.CDLL(build_port())
        L = self.lib
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        L.oracle_sgemm.argtypes = [_i64] * 3 + [_vp] * 3
        L.oracle_sgemm_naive.argtypes = [_i64] * 3 + [_vp] * 3
        L.oracle_ssyrk.argtypes = [_i64] * 2 + [_vp] * 2
        L.oracle_conv.argtypes = [_i64] * 8 + [_vp] * 4
        L.oracle_conv_nhwc.argtypes = [_i64] * 7 + [ctypes.c_bool] + [_vp] * 4
        L.oracle_conv_nhwc_strided.argtypes = [_i64] * 8 + [ctypes.c_bool] + [_vp] * 4
        L.oracle_im2col_nhwc.argtypes = [_i64] * 6 + [_vp] * 2
        L.oracle_matmul_i8.argtypes = [_i64] * 3 + [_vp, ctypes.c_bool] + [_vp] * 3
        L.oracle_conv_i8.argtypes = [_i64] * 6 + [_vp] * 4 + [ctypes.c_bool, _vp]
        L.oracle_gemm_bf16.argtypes = [_i64] * 3 + [_vp] * 3
        L.oracle_bf16_widen.argtypes = [_i64, _vp, _vp]
        L.oracle_bf16_round.argtypes = [_i64, _vp, _vp]
        for name in ("oracle_sgemm", "oracle_sgemm_naive", "oracle_ssyrk", "oracle_conv_nhwc_strided", "oracle_conv", "oracle_conv_nhwc",
                     "oracle_im2col_nhwc", "oracle_matmul_i8", "oracle_conv_i8",
                     "oracle_gemm_bf16", "oracle_bf16_widen", "oracle_bf16_round",
                     "oracle_set_threads"):
            getattr(L, name).restype = None

    def set_threads(self, n: int) -> None:
        self.lib.oracle_set_threads(int(n))

    def sgemm(self, A, B, C, naive=False):
        """C += A @ B in place (fp32 arrays); returns C."""
        M, K = A.shape
        K2, N = B.shape
        assert K == K2 and C.shape == (M, N)
        assert A.dtype == B.dtype == C.dtype == np.float32
        fn = self.lib.oracle_sgemm_naive if naive else self.lib.oracle_sgemm
        fn(M, N, K, _ptr(A), _ptr(B), _ptr(C))
        return C

    def ssyrk(self, A, C):
        """C += A @ A.T on the upper triangle (j >= i), in place; returns C."""
        N, K = A.shape
        assert C.shape == (N, N) and A.dtype == C.dtype == np.float32
        self.lib.oracle_ssyrk(N, K, _ptr(A), _ptr(C))
        return C

    def conv(self, inp, weights, bias):
        """Reference layout: inp NHWC, weights [Ci,Kh,Kw,Co]; no pad; ReLU."""
        n, ih, iw, ci = inp.shape
        ci2, kh, kw, co = weights.shape
        assert ci == ci2 and kh == kw
        oh, ow = ih - kh + 1, iw - kw + 1
        out = np.empty((n, oh, ow, co), np.float32)
        self.lib.oracle_conv(oh, ow, co, ih, iw, ci, kh, n, _ptr(inp), _ptr(out), _ptr(weights),
                             _ptr(bias))
        return out

    def conv_nhwc(self, inp, weights, bias, pad, relu=True):
        """weights [Kh,Kw,Ci,Co], symmetric zero padding."""
        n, ih, iw, ci = inp.shape
        kh, kw, ci2, co = weights.shape
        assert ci == ci2 and kh == kw
        oh, ow = ih + 2 * pad - kh + 1, iw + 2 * pad - kw + 1
        out = np.empty((n, oh, ow, co), np.float32)
        self.lib.oracle_conv_nhwc(n, ih, iw, ci, co, kh, pad, bool(relu), _ptr(inp), _ptr(out),
                                  _ptr(weights), _ptr(bias) if bias is not None else None)
        return out

    def conv_nhwc_strided(self, inp, weights, bias, pad, stride, relu=True):
        """weights [Kh,Kw,Ci,Co], symmetric zero padding, stride >= 1."""
        n, ih, iw, ci = inp.shape
        kh, kw, ci2, co = weights.shape
        assert ci == ci2 and kh == kw and stride >= 1
        oh, ow = (ih + 2 * pad - kh) // stride + 1, (iw + 2 * pad - kw) // stride + 1
        out = np.empty((n, oh, ow, co), np.float32)
        self.lib.oracle_conv_nhwc_strided(n, ih, iw, ci, co, kh, pad, stride, bool(relu), _ptr(inp), _ptr(out),
                                          _ptr(weights), _ptr(bias) if bias is not None else None)
        return out

    def im2col_nhwc(self, inp, kdim, pad):
        n, ih, iw, ci = inp.shape
        oh, ow = ih + 2 * pad - kdim + 1, iw + 2 * pad - kdim + 1
        col = np.empty((n * oh * ow, kdim * kdim * ci), np.float32)
        self.lib.oracle_im2col_nhwc(n, ih, iw, ci, kdim, pad, _ptr(inp), _ptr(col))
        return col

    def matmul_i8(self, A, B, scale, act):
        N, K = A.shape
        K2, M = B.shape
        assert K == K2 and A.dtype == B.dtype == np.int8
        C = np.empty((N, M), np.int8)
        s = np.array([scale], np.float32)
        self.lib.oracle_matmul_i8(N, M, K, _ptr(s), bool(act), _ptr(A), _ptr(B), _ptr(C))
        return C

    def conv_i8(self, inp, weights, bias, scale, act):
        b, ind, ind2, ci = inp.shape
        kh, kw, ci2, co = weights.shape
        assert ind == ind2 and kh == kw and ci == ci2
        od = ind - kh + 1
        out = np.empty((b, od, od, co), np.int8)
        s = np.array([scale], np.float32)
        bias = np.ascontiguousarray(bias.reshape(-1), np.int32)
        self.lib.oracle_conv_i8(b, od, co, kh, ci, ind, _ptr(out), _ptr(bias), _ptr(inp),
                                _ptr(weights), bool(act), _ptr(s))
        return out

    def gemm_bf16(self, A, Bt):
        """A: uint16 [M,K] bf16 bits; Bt: uint16 [N,K] (= column-major KxN)."""
        M, K = A.shape
        N, K2 = Bt.shape
        assert K == K2 and A.dtype == Bt.dtype == np.uint16
        C = np.empty((M, N), np.uint16)
        self.lib.oracle_gemm_bf16(M, N, K, _ptr(A), _ptr(Bt), _ptr(C))
        return C

    def bf16_widen(self, a):
        out = np.empty(a.shape, np.float32)
        self.lib.oracle_bf16_widen(a.size, _ptr(a), _ptr(out))
        return out

    def bf16_round(self, a):
        out = np.empty(a.shape, np.uint16)
        self.lib.oracle_bf16_round(a.size, _ptr(a), _ptr(out))
        return out


# Shapes baked into the reference's generated int8 functions
# (apps/gemmini/src/exo/matmul.py:166-170,228-232,284-288,349-353,414-418,487-507
#  and apps/gemmini/src/exo/conv.py:58-66 ff.): name -> (N, M, K) / conv dims.
REF_MATMUL_SHAPES = {
    "512x512x512": (512, 512, 512),
    "4": (12544, 256, 64),
    "6": (12544, 64, 256),
    "14": (3136, 512, 128),
    "16": (3136, 128, 512),
    "27": (784, 1024, 256),
}
# name -> (batch, out_dim, out_channel, kernel_dim, in_channel, in_dim)
REF_CONV_I8_SHAPES = {
    "3": (4, 56, 64, 3, 64, 58),
    "17": (4, 28, 128, 3, 128, 30),
    "30": (4, 14, 256, 3, 256, 16),
}


class Ref:
    """ctypes view of the compiled reference C (oracle/_ref/libexo_ref.so).

    sgemm_exo keeps its tiles in function-local statics, so it is not
    reentrant: one call at a time per process."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        if not _cpu_has("avx512f"):
            raise RuntimeError("compiled reference needs AVX-512F on this host")
        self.lib = ctypes.CDLL(REF_SO)
        L = self.lib
        L.sgemm_exo.argtypes = [_vp] + [_i64] * 3 + [_vp] * 3
        L.sgemm_exo.restype = None
        L.conv_specialized.argtypes = [_vp] * 5
        L.conv_specialized.restype = None
        for name in REF_MATMUL_SHAPES:
            f = getattr(L, f"cpu_matmul_{name}")
            f.argtypes = [_vp, _vp, ctypes.c_bool, _vp, _vp, _vp]
            f.restype = None
        for name in REF_CONV_I8_SHAPES:
            f = getattr(L, f"conv_{name}_cpu")
            f.argtypes = [_vp, _vp, _vp, _vp, _vp, ctypes.c_bool, _vp]
            f.restype = None

    def sgemm(self, A, B, C):
        M, K = A.shape
        _, N = B.shape
        assert A.dtype == B.dtype == C.dtype == np.float32 and C.shape == (M, N)
        self.lib.sgemm_exo(None, M, N, K, _ptr(A), _ptr(B), _ptr(C))
        return C

    def conv_specialized(self, inp, weights, bias):
        assert inp.shape == (5, 82, 102, 128) and weights.shape == (128, 3, 3, 128)
        out = np.empty((5, 80, 100, 128), np.float32)
        self.lib.conv_specialized(None, _ptr(inp), _ptr(out), _ptr(weights), _ptr(bias))
        return out

    def matmul_i8(self, name, A, B, scale, act):
        N, M, K = REF_MATMUL_SHAPES[name]
        assert A.shape == (N, K) and B.shape == (K, M)
        C = np.empty((N, M), np.int8)
        s = np.array([scale], np.float32)
        getattr(self.lib, f"cpu_matmul_{name}")(None, _ptr(s), bool(act), _ptr(A), _ptr(B), _ptr(C))
        return C

    def conv_i8(self, name, inp, weights, bias, scale, act):
        b, od, co, kd, ci, ind = REF_CONV_I8_SHAPES[name]
        assert inp.shape == (b, ind, ind, ci) and weights.shape == (kd, kd, ci, co)
        out = np.empty((b, od, od, co), np.int8)
        s = np.array([scale], np.float32)
        bias = np.ascontiguousarray(bias.reshape(-1), np.int32)
        getattr(self.lib, f"conv_{name}_cpu")(None, _ptr(out), _ptr(bias), _ptr(inp), _ptr(weights),
                                              bool(act), _ptr(s))
        return out


_port = None
_ref = None


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref_available() -> bool:
    return os.path.exists(REF_SO) and _cpu_has("avx512f")


def ref() -> Ref:
    global _ref
    if _ref is None:
        _ref = Ref()
    return _ref
