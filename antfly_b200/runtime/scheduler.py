"""Python face of the C++ continuous-batching scheduler (``csrc/host/scheduler.cpp``)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List

import numpy as np

from .. import _native as N

_i64 = ctypes.c_int64
_int = ctypes.c_int
_pint = ctypes.POINTER(ctypes.c_int)
_pi64 = ctypes.POINTER(ctypes.c_int64)


class QueueFull(RuntimeError):
    """Admission refused: the server answers 503 (the reference's error.QueueFull)."""


@dataclass
class StepItem:
    request_id: int
    mode: str  # "decode" or "prefill"
    q_len: int
    kv_before: int


@dataclass
class SchedulerPolicy:
    # The reference's defaults (native_generate.zig:40-57); the B200 engine passes larger budgets.
    max_step_items: int = 16
    max_step_query_tokens: int = 512
    prefill_chunk: int = 256
    min_chunk: int = 32
    decode_streak: int = 4
    max_kv_blocks: int = 0
    page: int = 16
    max_queue: int = 0


def _lib():
    lib = N.host()
    if not getattr(lib, "_sched_ready", False):
        lib.afb_sched_create.restype = ctypes.c_void_p
        lib.afb_sched_create.argtypes = [_int] * 8
        lib.afb_sched_destroy.argtypes = [ctypes.c_void_p]
        lib.afb_sched_admit.argtypes = [ctypes.c_void_p, _i64, _int, _int]
        lib.afb_sched_set_decode_width.argtypes = [ctypes.c_void_p, _i64, _int]
        lib.afb_sched_set_atomic_prefill.argtypes = [ctypes.c_void_p, _i64, _int]
        lib.afb_sched_claim_step.argtypes = [ctypes.c_void_p, _pi64, _pint, _pint, _pint, _int]
        lib.afb_sched_complete_step.argtypes = [ctypes.c_void_p, _int, _pi64, _pint, _pint]
        lib.afb_sched_fail_step.argtypes = [ctypes.c_void_p]
        lib.afb_sched_cancel.argtypes = [ctypes.c_void_p, _i64]
        lib.afb_sched_snapshot.argtypes = [ctypes.c_void_p, _pint]
        lib.afb_sched_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64)]
        lib._sched_ready = True
    return lib


class StepScheduler:
    def __init__(self, policy: SchedulerPolicy = SchedulerPolicy()):
        self.lib = _lib()
        self.policy = policy
        p = policy
        self.h = ctypes.c_void_p(self.lib.afb_sched_create(p.max_step_items, p.max_step_query_tokens, p.prefill_chunk,
                                                          p.min_chunk, p.decode_streak, p.max_kv_blocks, p.page,
                                                          p.max_queue))
        cap = max(p.max_step_items, 1)
        self._ids = np.empty(cap, dtype=np.int64)
        self._modes = np.empty(cap, dtype=np.int32)
        self._q = np.empty(cap, dtype=np.int32)
        self._kv = np.empty(cap, dtype=np.int32)

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.lib.afb_sched_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def admit(self, request_id: int, prompt_len: int, max_new_tokens: int, prompt_done: int = 0) -> None:
        """``prompt_done`` > 0: that many leading prompt tokens are already in the KV cache (shared prefix)."""
        if prompt_done > 0:
            rc = self.lib.afb_sched_admit_prefilled(self.h, request_id, prompt_len, max_new_tokens, prompt_done)
        else:
            rc = self.lib.afb_sched_admit(self.h, request_id, prompt_len, max_new_tokens)
        if rc == -2:
            raise QueueFull("generation queue is full")
        if rc != 0:
            raise ValueError("duplicate request id or empty prompt")

    def set_atomic_prefill(self, request_id: int, on: bool = True) -> None:
        """The request's prompt is prefilled in one step, never in chunks."""
        self.lib.afb_sched_set_atomic_prefill(self.h, request_id, 1 if on else 0)

    def set_decode_width(self, request_id: int, width: int) -> None:
        self.lib.afb_sched_set_decode_width(self.h, request_id, width)

    def claim_step(self) -> List[StepItem]:
        n = self.lib.afb_sched_claim_step(self.h, self._ids.ctypes.data_as(_pi64), self._modes.ctypes.data_as(_pint),
                                          self._q.ctypes.data_as(_pint), self._kv.ctypes.data_as(_pint),
                                          len(self._ids))
        if n < 0:
            raise RuntimeError("a step is already in flight")
        return [StepItem(int(self._ids[i]), "decode" if self._modes[i] == 0 else "prefill", int(self._q[i]),
                         int(self._kv[i])) for i in range(n)]

    def complete_step(self, items: List[StepItem], tokens_out: List[int], finished: List[bool]) -> None:
        n = len(items)
        ids = np.array([it.request_id for it in items], dtype=np.int64)
        tk = np.array(tokens_out, dtype=np.int32)
        fin = np.array([1 if f else 0 for f in finished], dtype=np.int32)
        self.lib.afb_sched_complete_step(self.h, n, ids.ctypes.data_as(_pi64), tk.ctypes.data_as(_pint),
                                         fin.ctypes.data_as(_pint))

    def fail_step(self) -> None:
        self.lib.afb_sched_fail_step(self.h)

    def cancel(self, request_id: int) -> bool:
        return self.lib.afb_sched_cancel(self.h, request_id) == 0

    def snapshot(self) -> dict:
        out = (ctypes.c_int * 4)()
        self.lib.afb_sched_snapshot(self.h, out)
        return {"waiting": out[0], "prefill": out[1], "decode": out[2], "in_flight": out[3]}

    def stats(self) -> dict:
        out = (ctypes.c_uint64 * 8)()
        self.lib.afb_sched_stats(self.h, out)
        keys = ["step_batches_total", "step_prefill_items_total", "step_decode_items_total",
                "step_query_tokens_total", "step_singleton_batches_total", "step_kv_block_skips_total",
                "queue_full_total", "failed_steps_total"]
        return {k: int(out[i]) for i, k in enumerate(keys)}
