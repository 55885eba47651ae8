"""exo_b200: B200-native GEMM / convolution kernels behind the C ABI of Exo's
generated code (sgemm_exo, conv_specialized / conv, the Gemmini int8 matmul and
conv) plus bf16 / 3xTF32 tensor-core entry points.

    import exo_b200
    lib = exo_b200.library()
    lib.sgemm_exo(None, M, N, K, A, B, C)      # C += A @ B, numpy or torch CUDA tensors

The compute code lives in ``libexo_b200.so`` (``python -m exo_b200.build``);
importing the package without it fails -- there is no CPU path.
"""
from .api import (Context, ERR_CUDA, ERR_INVALID_ARGUMENT, ERR_TIMEOUT, ERR_UNSUPPORTED, OK, SGEMM_3XTF32,
                  SGEMM_FFMA, ExoB200Error, Library, library)
from . import _lib

_lib.load()  # fail loudly at import time if the CUDA library is missing

__all__ = ["library", "Library", "Context", "ExoB200Error", "OK", "ERR_INVALID_ARGUMENT", "ERR_CUDA",
           "ERR_TIMEOUT", "ERR_UNSUPPORTED", "SGEMM_FFMA", "SGEMM_3XTF32"]
