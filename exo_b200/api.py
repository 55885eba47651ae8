"""Python face of the C ABI, in the calling style of the reference's own ctypes
harness (tests/conftest.py:141-173, ``ProcWrapper``): positional arguments,
``None`` for the context, ints for sizes, arrays for tensors -- e.g.
``lib.sgemm_exo(None, M, N, K, A, B, C)`` exactly as one would call the library
``exocc`` generates.  Tensors may be numpy arrays (host memory: staged to the
GPU and back inside the call) or torch CUDA tensors (used in place, on torch's
current stream).  Results are written into the output argument.

Errors: the C functions return void (as the reference's do); this wrapper reads
the library's error side channel after each call and raises ``ExoB200Error``.
"""
from __future__ import annotations

import ctypes
import threading

import numpy as np

from . import _lib


class ExoB200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code


OK, ERR_INVALID_ARGUMENT, ERR_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED = range(5)
SGEMM_FFMA, SGEMM_3XTF32 = 0, 1


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch") and hasattr(x, "data_ptr")


def _convert(arg, argtype, keepalive):
    """One argument, the way ProcWrapper._convert does it, plus torch tensors,
    Python floats for by-pointer scalars, and Context objects.  Temporaries that
    the C call reads through a pointer are appended to ``keepalive``, which the
    caller owns until the C function has returned."""
    if arg is None:
        return None
    if isinstance(arg, Context):
        return arg.handle
    if isinstance(arg, np.ndarray):
        if not arg.flags["C_CONTIGUOUS"]:
            raise ValueError("arrays must be C-contiguous (dense row-major)")
        return ctypes.c_void_p(arg.ctypes.data)
    if _is_torch(arg):
        if not arg.is_contiguous():
            raise ValueError("tensors must be contiguous (dense row-major)")
        return ctypes.c_void_p(arg.data_ptr())
    if isinstance(arg, (bool, np.bool_)):
        return bool(arg)
    if isinstance(arg, (int, np.integer)):
        return int(arg)
    if isinstance(arg, float) and argtype is _lib.vp:
        # numeric scalars travel by pointer in Exo's ABI
        holder = ctypes.c_float(arg)
        keepalive.append(holder)
        return ctypes.cast(ctypes.pointer(holder), ctypes.c_void_p)
    raise ValueError(f"unrecognized type {type(arg)}")


_raw_stream = None  # torch._C._cuda_getCurrentRawStream where available: the stream handle without a Stream object


def _sync_stream_for(args):
    """Device tensors run on torch's current stream."""
    global _raw_stream
    for a in args:
        if _is_torch(a) and a.is_cuda:
            if _raw_stream is None:
                import torch

                fast = getattr(torch._C, "_cuda_getCurrentRawStream", None)
                _raw_stream = fast if fast is not None else (lambda i: torch.cuda.current_stream(i).cuda_stream)
            return _raw_stream(a.device.index)
    return None


_last_default_stream = threading.local()  # what this thread last installed as the library's default stream


class ProcWrapper:
    def __init__(self, dll, name):
        self._fn = getattr(dll, name)
        self._dll = dll
        self._name = name
        self._argtypes = _lib.PROTOTYPES[name]

    def __call__(self, *args, **kwargs):
        if kwargs:
            raise ValueError("cannot call with kwargs")
        if len(args) != len(self._argtypes):
            raise TypeError(f"{self._name} takes {len(self._argtypes)} arguments ({len(args)} given)")
        stream = _sync_stream_for(args)
        ctx = args[0] if isinstance(args[0], Context) else None
        if ctx is not None:
            if stream is not None:
                self._dll.exo_b200_context_set_stream(ctx.handle, stream)
        elif getattr(_last_default_stream, "value", -1) != stream:
            # the library keeps the default stream per host thread; tell it only when it changes
            self._dll.exo_b200_set_default_stream(stream)
            _last_default_stream.value = stream
        keepalive = []  # per call, so concurrent callers cannot free each other's scalars
        conv = [_convert(a, t, keepalive) for a, t in zip(args, self._argtypes)]
        self._fn(*conv)
        del keepalive
        code = self._dll.exo_b200_last_error()
        if code != OK:
            raise ExoB200Error(code, self._dll.exo_b200_last_error_string().decode())


class Library:
    """``lib.<proc>(ctxt, ...)`` for every entry point of include/exo_b200.h."""

    def __init__(self):
        self.dll = _lib.load()

    def __getattr__(self, item):
        if item in _lib.PROTOTYPES:
            w = ProcWrapper(self.dll, item)
            setattr(self, item, w)
            return w
        raise AttributeError(item)

    def synchronize(self, ctx: "Context | None" = None) -> None:
        code = self.dll.exo_b200_synchronize(ctx.handle if ctx else None)
        if code != OK:
            raise ExoB200Error(code, self.dll.exo_b200_last_error_string().decode())

    def version(self) -> str:
        return self.dll.exo_b200_version().decode()


class Context:
    """An explicit context: device, stream and SGEMM arithmetic path."""

    def __init__(self, device: int = -1, stream: int | None = None, sgemm_path: int = SGEMM_FFMA):
        self._dll = _lib.load()
        self.handle = self._dll.exo_b200_context_create(device, stream)
        if not self.handle:
            raise ExoB200Error(self._dll.exo_b200_last_error(),
                               self._dll.exo_b200_last_error_string().decode())
        self._dll.exo_b200_context_set_sgemm_path(self.handle, sgemm_path)

    def close(self):
        if self.handle:
            self._dll.exo_b200_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_library = None


def library() -> Library:
    global _library
    if _library is None:
        _library = Library()
    return _library
