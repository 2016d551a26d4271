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
    """Device address of a tensor for a native launcher.  The launchers run on the calling THREAD's current device
    and stream, so a CUDA tensor of another device is refused here: launching on GPU 0's stream with pointers
    into GPU 1's memory would be an illegal-address fault.  Threads that serve a model enter
    ``device_of(model_device)`` (or ``torch.cuda.device``) first."""
    if t is None:
        return ctypes.c_void_p(0)
    if t.is_cuda and t.device.index != torch.cuda.current_device():
        raise NativeError(f"tensor on cuda:{t.device.index} passed to a kernel launcher while this thread's current "
                          f"device is cuda:{torch.cuda.current_device()}; wrap the call in device_of(tensor.device)")
    return ctypes.c_void_p(t.data_ptr())


def device_of(device):
    """Context manager that makes `device` current in this thread for the launches inside it (a no-op context for
    CPU devices).  The current CUDA device is per host thread and starts at 0 in every new thread."""
    import contextlib

    d = torch.device(device) if device is not None else None
    if d is None or d.type != "cuda":
        return contextlib.nullcontext()
    return torch.cuda.device(d)


def status(clear: bool = True) -> int:
    """Synchronise and return the OR of the kernels' status words (0 = no bounded wait gave up)."""
    torch.cuda.synchronize()
    return int(cuda().afb_status_read(1 if clear else 0))


def poison_waits(device: int | None = None) -> int:
    """Make every bounded kernel wait (running, queued or future) on `device` give up at once; see
    ``afb_poison_waits_on``.  For watchdogs and signal handlers: the GPU drains before the process goes away.
    `device` is the CUDA device index whose kernels are to be drained; a timer or signal-helper thread must pass
    it, because the current device is per thread and such a thread starts on device 0.  None = this thread's
    current device.  ``status()`` clears the poison."""
    try:
        lib = cuda()
        if device is None:
            return int(lib.afb_poison_waits())
        return int(lib.afb_poison_waits_on(ctypes.c_int(int(device))))
    except Exception:
        return -1


# Longer than the cross-GPU wait limit compiled into the kernels (AFB_PEER_WAIT_NS, 2 s).
DRAIN_SECONDS = 3.0


def drain_for_exit(device: int | None = None) -> None:
    """Called on the way out of a process that may have kernels in cross-GPU waits (watchdog, SIGTERM): poison
    the waits of `device`, then give the GPU longer than one wait limit to run dry before the caller exits."""
    import time

    poison_waits(device)
    time.sleep(DRAIN_SECONDS)


_launch_counter = 0


def count_launch(n: int = 1) -> None:
    global _launch_counter
    _launch_counter += n


def launches() -> int:
    return _launch_counter


def reset_launches() -> None:
    global _launch_counter
    _launch_counter = 0
