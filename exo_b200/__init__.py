"""exo_b200: B200-native GEMM / convolution kernels behind the C ABI of Exo's
generated code (sgemm_exo, conv_specialized / conv, the Gemmini int8 matmul and
conv) plus bf16 / 3xTF32 tensor-core entry points.

    import exo_b200
    lib = exo_b200.library()
    lib.sgemm_exo(None, M, N, K, A, B, C)      # C += A @ B, numpy or torch CUDA tensors

The compute code lives in ``libexo_b200.so`` (``python -m exo_b200.build``).
``library()`` loads it and raises if it is missing or stale -- there is no CPU
path to fall back to.  (The import itself stays light so that the build module
inside this package can run before the library exists.)
"""
from .api import (Context, ERR_CUDA, ERR_INVALID_ARGUMENT, ERR_TIMEOUT, ERR_UNSUPPORTED, OK, SGEMM_3XTF32,
                  SGEMM_FFMA, ExoB200Error, Library, library)

__all__ = ["library", "Library", "Context", "ExoB200Error", "OK", "ERR_INVALID_ARGUMENT", "ERR_CUDA",
           "ERR_TIMEOUT", "ERR_UNSUPPORTED", "SGEMM_FFMA", "SGEMM_3XTF32"]
