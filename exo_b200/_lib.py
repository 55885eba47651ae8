"""Loads libexo_b200.so and declares the C prototypes of include/exo_b200.h.

The product path has no CPU implementation: if the CUDA library has not been
built (``python -m exo_b200.build``) importing this module raises."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libexo_b200.so")

i64 = ctypes.c_int64  # int_fast32_t is 8 bytes on glibc x86-64
vp = ctypes.c_void_p
cbool = ctypes.c_bool

_MM_INSTANCES = ("512x512x512", "4", "6", "14", "16", "27")
_CONV_INSTANCES = ("3", "17", "30")

# name -> argtypes; every compute entry point returns void
PROTOTYPES = {
    "sgemm_exo": [vp, i64, i64, i64, vp, vp, vp],
    "sgemm_exo_ffma": [vp, i64, i64, i64, vp, vp, vp],
    "sgemm_exo_3xtf32": [vp, i64, i64, i64, vp, vp, vp],
    "conv_specialized": [vp, vp, vp, vp, vp],
    "conv": [vp] + [i64] * 8 + [vp] * 4,
    "conv_nhwc_exo": [vp] + [i64] * 7 + [cbool] + [vp] * 4,
    "conv_nhwc_exo_3xtf32": [vp] + [i64] * 7 + [cbool] + [vp] * 4,
    "conv_nhwc_strided_exo": [vp] + [i64] * 8 + [cbool] + [vp] * 4,
    "matmul_on_cpu": [vp, i64, i64, i64, vp, cbool, vp, vp, vp],
    "conv_on_cpu_stride_1": [vp] + [i64] * 6 + [vp] * 4 + [cbool, vp],
    "gemm_bf16_exo": [vp, i64, i64, i64, vp, vp, vp],
    "matmul_on_cpu_static": [vp, i64, i64, i64, vp, cbool, vp, vp, vp],
    "ssyrk_exo": [vp, i64, i64, vp, vp],
    "ssyrk_exo_ffma": [vp, i64, i64, vp, vp],
    "ssyrk_exo_3xtf32": [vp, i64, i64, vp, vp],
    # the Gemmini library's "auto" entry points (include/exo_b200_gemmini_shim.h)
    "tiled_matmul_auto": [ctypes.c_size_t] * 3 + [vp] * 4 + [ctypes.c_size_t] * 4 + [ctypes.c_float] * 3
                         + [ctypes.c_int, ctypes.c_float, ctypes.c_float] + [cbool] * 5 + [ctypes.c_uint8, ctypes.c_int],
    "tiled_conv_auto": [ctypes.c_int] * 12 + [cbool] * 5 + [vp] * 4 + [ctypes.c_int, ctypes.c_float]
                       + [ctypes.c_int] * 4,
}
for _n in _MM_INSTANCES:
    PROTOTYPES[f"cpu_matmul_{_n}"] = [vp, vp, cbool, vp, vp, vp]
    PROTOTYPES[f"matmul_{_n}"] = [vp, vp, cbool, vp, vp, vp]
for _n in _CONV_INSTANCES:
    PROTOTYPES[f"conv_{_n}_cpu"] = [vp, vp, vp, vp, vp, cbool, vp]
    PROTOTYPES[f"conv_{_n}"] = [vp, vp, vp, vp, vp, cbool, vp]

SUPPORT = {
    "exo_b200_context_create": ([ctypes.c_int, vp], vp),
    "exo_b200_context_destroy": ([vp], None),
    "exo_b200_context_set_stream": ([vp, vp], None),
    "exo_b200_context_set_sgemm_path": ([vp, ctypes.c_int], None),
    "exo_b200_set_default_stream": ([vp], None),
    "exo_b200_context_cache_weights": ([vp, ctypes.c_int], None),
    "exo_b200_context_invalidate": ([vp], None),
    "exo_b200_synchronize": ([vp], ctypes.c_int),
    "exo_b200_selftest_bounded_wait": ([vp, ctypes.c_int], ctypes.c_int),
    "exo_b200_measure_peak": ([ctypes.c_int, ctypes.c_int], ctypes.c_double),
    "exo_b200_sgemm_kernel_choice": ([i64, i64, i64], ctypes.c_int),
    "exo_b200_last_error": ([], ctypes.c_int),
    "exo_b200_last_error_string": ([], ctypes.c_char_p),
    "exo_b200_version": ([], ctypes.c_char_p),
}

_dll = None


def load() -> ctypes.CDLL:
    global _dll
    if _dll is not None:
        return _dll
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m exo_b200.build` "
            "(needs nvcc; there is no CPU fallback)")
    dll = ctypes.CDLL(LIB_PATH)
    for name, argtypes in PROTOTYPES.items():
        f = getattr(dll, name)
        f.argtypes = argtypes
        f.restype = None
    for name, (argtypes, restype) in SUPPORT.items():
        f = getattr(dll, name)
        f.argtypes = argtypes
        f.restype = restype
    _dll = dll
    return dll
