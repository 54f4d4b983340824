"""Calling the compiled kernels: pointers, dtype codes, streams, error codes."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import KernelsUnavailable, load_library

_DT = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {10001: "unsupported dtype combination", 10002: "unsupported size", 10003: "misaligned pointer or stride",
           10004: "a bounded wait inside the kernel ran out (see the kernel's status word)",
           10005: "the problem needs more scratch than the library's built-in array holds"}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


def dt_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {dtype}") from None


def require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelsUnavailable(
                "this operation runs only as a CUDA kernel on an sm_100a device; it was given a "
                f"{t.device} tensor (there is no CPU path)")
        if not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


try:                                    # the raw handle without building a Stream object (an order of magnitude cheaper)
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:                  # pragma: no cover - older torch
    _raw_stream = None


def stream() -> ctypes.c_void_p:
    """The current CUDA stream of the current device (the capturing stream inside a graph capture)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_COUNTER = [None]


def set_launch_counter(obj) -> None:
    """``obj.kernel_launches`` is incremented for every kernel launched from here on."""
    _COUNTER[0] = obj


def count_launches(n: int) -> None:
    if _COUNTER[0] is not None:
        _COUNTER[0].kernel_launches += n


def check(code: int, what: str, launches: int = 1) -> None:
    if code == 0:
        if _COUNTER[0] is not None:
            _COUNTER[0].kernel_launches += launches
        return
    if code in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[code]}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_FN_CACHE = {}
_LIBS = {}


def _library(lib: str):
    """The loaded library; the launch options of this process are handed to it when it is loaded."""
    h = _LIBS.get(lib)
    if h is None:
        h = _LIBS[lib] = load_library(lib)
        _set_pdl(h)
    return h


def loaded(lib: str) -> bool:
    return lib in _LIBS


def _set_pdl(handle) -> None:
    from .options import OPTIONS
    f = getattr(handle, "sx_set_pdl", None)
    if f is not None:
        f(ctypes.c_int(1 if OPTIONS.pdl else 0))


def apply_pdl() -> None:
    """Tell every loaded library whether kernels are launched with programmatic dependent launch."""
    for h in _LIBS.values():
        _set_pdl(h)


def fn(lib: str, name: str):
    key = (lib, name)
    f = _FN_CACHE.get(key)
    if f is None:
        f = getattr(_library(lib), name)
        f.restype = ctypes.c_int
        _FN_CACHE[key] = f
    return f


c_int = ctypes.c_int
c_float = ctypes.c_float
c_longlong = ctypes.c_longlong
c_ulonglong = ctypes.c_ulonglong
