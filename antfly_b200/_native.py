"""ctypes bindings to the in-tree native libraries.

``cuda()`` returns the handle of ``libafb_cuda.so`` (sm_100a kernels); ``host()`` the handle of
``libafb_host.so`` (C++ runtime: KV blocks, scheduler, formats, codecs, CPU oracle).  Both are built on first
use when missing.  When a CUDA device is present and the kernel library cannot be loaded, ops raise instead
of silently falling back to PyTorch.
"""
from __future__ import annotations

import ctypes
import functools
import os
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent / "_lib"


class NativeError(RuntimeError):
    pass


def _ensure_built() -> None:
    if os.environ.get("ANTFLY_B200_NO_BUILD"):
        return
    from . import _build

    _build.build()


@functools.lru_cache(maxsize=None)
def cuda() -> ctypes.CDLL:
    path = _LIB_DIR / "libafb_cuda.so"
    if not path.exists():
        _ensure_built()
    try:
        lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    except OSError as e:  # pragma: no cover - depends on the machine
        raise NativeError(f"cannot load {path}: {e}") from e
    lib.afb_last_error.restype = ctypes.c_char_p
    lib.afb_status_read.restype = ctypes.c_int
    lib.afb_status_read.argtypes = [ctypes.c_int]
    return lib


@functools.lru_cache(maxsize=None)
def host() -> ctypes.CDLL:
    path = _LIB_DIR / "libafb_host.so"
    if not path.exists():
        _ensure_built()
    try:
        lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    except OSError as e:  # pragma: no cover
        raise NativeError(f"cannot load {path}: {e}") from e
    return lib


def cuda_available() -> bool:
    return torch.cuda.is_available()


def check(rc: int, what: str) -> None:
    """Raise when a native launcher reports failure."""
    if rc != 0:
        msg = cuda().afb_last_error()
        raise NativeError(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def status(clear: bool = True) -> int:
    """Synchronise and return the OR of the kernels' status words (0 = no bounded wait gave up)."""
    torch.cuda.synchronize()
    return int(cuda().afb_status_read(1 if clear else 0))


def poison_waits() -> int:
    """Make every bounded kernel wait (running, queued or future) give up at once; see ``afb_poison_waits``.
    For watchdogs and signal handlers: the GPU drains before the process goes away.  ``status()`` clears it."""
    try:
        return int(cuda().afb_poison_waits())
    except Exception:
        return -1


_launch_counter = 0


def count_launch(n: int = 1) -> None:
    global _launch_counter
    _launch_counter += n


def launches() -> int:
    return _launch_counter


def reset_launches() -> None:
    global _launch_counter
    _launch_counter = 0
