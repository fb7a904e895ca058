"""ctypes binding of ``libftb200_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`torchft_b200._build`.  On a machine with a
CUDA device the library is mandatory: :func:`lib` raises if it cannot be loaded so
that no GPU code path silently falls back to eager PyTorch.
"""

from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from .. import _build

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float

ERRORS = {
    -1: "bad argument",
    -2: "misaligned pointer or leading dimension",
    -3: "driver entry point unavailable / tensor-map encode failed",
    -4: "size beyond the supported maximum",
    -5: "CUDA launch error",
}

STATUS = {0: "ok", 1: "timeout", 2: "aborted", 3: "epoch mismatch", 4: "bounds"}


class KernelError(RuntimeError):
    pass


def available() -> bool:
    """True when the kernel library exists (it may still need a GPU to run)."""
    return _build.KERNEL_LIB.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        checked = os.environ.get("FTB200_KERNEL_LIB", "") == "checked"
        path = _build.KERNEL_LIB_CHECKED if checked else _build.KERNEL_LIB
        if not path.exists():
            if os.environ.get("FTB200_NO_AUTOBUILD"):
                raise KernelError(f"{path} is missing; run `python -m torchft_b200._build`")
            _build.build_kernels(checked=checked)
        _lib = ctypes.CDLL(str(path))
        return _lib


def bounds_status() -> tuple:
    """``(code, index)`` recorded by the checked-index debug build (``FTB200_KERNEL_LIB=checked``)
    since the last call: ``(0, 0)`` when every guarded index was in range, ``(4, i)`` with the
    first offending index otherwise.  Always ``(0, 0)`` on the normal library, which has no checks."""
    code, index = 0, 0
    library = lib()
    for tag in ("elementwise", "team", "gemm_2cta"):
        fn = getattr(library, f"ftb200_bounds_status_{tag}", None)
        if fn is None:
            continue
        idx = ctypes.c_longlong(0)
        st = int(fn(ctypes.byref(idx)))
        if st and not code:
            code, index = st, int(idx.value)
    return code, index


launch_count = 0  # kernels launched through this library since import (bench.py reports the delta)


def check(rc: int, what: str, launches: int = 1) -> None:
    global launch_count
    if rc != 0:
        raise KernelError(f"{what}: {ERRORS.get(rc, rc)}")
    launch_count += launches


def ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return c_void_p(s.cuda_stream)
