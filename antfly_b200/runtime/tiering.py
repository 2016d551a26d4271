"""Memory tiers for weights: GPU memory, pinned host memory and disk, with a placement planner, per-run byte
budgets that refuse (and explain) reservations, and a background prefetcher that moves tensors up the tiers.

The planner and the budget follow the reference (zig/pkg/inference/src/runtime/tier/planner.zig:50-140,
memory.zig:87-346, prefetch.zig, shared.zig): weights are classed by name; embeddings, norms, attention and
routers want the backend tier and spill to host; output heads and unclassed tensors live on host and spill to
disk; experts want the backend and spill to host on a GPU (to disk on a CPU backend); a tensor larger than a quarter
of a budget is pushed one tier down.  A run budget tracks weight / KV / scratch bytes per tier against host,
backend, combined, KV and scratch limits; a refused reservation is recorded with the totals at that moment and
reported in one line.

What is specific here: on a B200 the backend tier is 180 GB of HBM3e and the host tier is pinned memory, so a
promotion is one ``cudaMemcpyAsync`` on a side stream that overlaps the compute stream; the disk tier is a
memory-mapped safetensors file, read on first touch by a worker thread so the page faults happen off the
serving thread.
"""
from __future__ import annotations

import enum
import heapq
import threading
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch


class Tier(enum.IntEnum):
    DISK = 0
    HOST = 1
    BACKEND = 2


class WeightClass(enum.Enum):
    EMBEDDING = "embedding"
    NORM = "norm"
    ATTENTION = "attention"
    ROUTER = "router"
    OUTPUT = "output"
    EXPERT = "expert"
    OTHER = "other"


@dataclass
class Placement:
    cls: WeightClass
    preferred: Tier
    spill: Tier


def classify_weight(name: str) -> WeightClass:
    if ".experts." in name or ".shared_expert." in name:
        return WeightClass.EXPERT
    if name.endswith(".block_sparse_moe.gate.weight") or name.endswith(".mlp.gate.weight") or \
            name.endswith("shared_expert_gate.weight"):
        return WeightClass.ROUTER
    if name in ("model.embed_tokens.weight", "wte.weight", "transformer.wte.weight"):
        return WeightClass.EMBEDDING
    if name in ("lm_head.weight", "output.weight"):
        return WeightClass.OUTPUT
    if ".self_attn." in name or ".attn." in name or ".attention." in name:
        return WeightClass.ATTENTION
    low = name.lower()
    if "layernorm" in low or "layer_norm" in low or ".norm." in low or low.endswith("norm.weight"):
        return WeightClass.NORM
    return WeightClass.OTHER


def plan_placement(name: str, gpu: bool = True, tensor_bytes: int = 0, host_budget: int = 0,
                   backend_budget: int = 0) -> Placement:
    """Where a weight should live and where it goes when that tier is full.  Without a GPU the backend tier is the
    host.  Budgets of 0 mean "no limit"."""
    top = Tier.BACKEND if gpu else Tier.HOST
    c = classify_weight(name)
    if c in (WeightClass.EMBEDDING, WeightClass.NORM, WeightClass.ATTENTION, WeightClass.ROUTER):
        p = Placement(c, top, Tier.HOST)
    elif c is WeightClass.EXPERT:
        p = Placement(c, top, Tier.HOST if gpu else Tier.DISK)
    else:
        p = Placement(c, Tier.HOST, Tier.DISK)
    if tensor_bytes and host_budget and tensor_bytes > host_budget // 4:
        if c in (WeightClass.OUTPUT, WeightClass.OTHER):
            p.preferred = p.spill = Tier.DISK
        elif c is WeightClass.EXPERT:
            p.spill = Tier.DISK
    if tensor_bytes and backend_budget and tensor_bytes > backend_budget // 4:
        if c is WeightClass.EXPERT:
            p.preferred, p.spill = Tier.HOST, Tier.DISK
        elif c in (WeightClass.OUTPUT, WeightClass.OTHER) and p.preferred is not Tier.DISK:
            p.preferred, p.spill = Tier.HOST, Tier.DISK
    return p


# -- run budget ---------------------------------------------------------------------------------------------------
class MemoryBudgetExceeded(RuntimeError):
    pass


@dataclass
class Limits:
    host: int = 0
    backend: int = 0
    combined: int = 0
    kv: int = 0
    scratch: int = 0

    @classmethod
    def from_mb(cls, host_mb=0, backend_mb=0, combined_mb=0, kv_mb=0, scratch_mb=0) -> "Limits":
        mb = 1 << 20
        return cls(int(host_mb) * mb, int(backend_mb) * mb, int(combined_mb) * mb, int(kv_mb) * mb, int(scratch_mb) * mb)


@dataclass
class Reservation:
    kind: str          # "weight" | "kv" | "scratch"
    tier: Tier
    nbytes: int


@dataclass
class Denial:
    reservation: Reservation
    limit: str
    current: int
    requested_total: int
    limit_bytes: int
    host_total: int
    backend_total: int
    kv_total: int
    scratch_total: int

    def line(self) -> str:
        r = self.reservation
        return (f"memory budget exceeded: limit={self.limit} reservation={r.kind}/{r.tier.name.lower()} "
                f"current={self.current} request={r.nbytes} next={self.requested_total} limit={self.limit_bytes} "
                f"totals(host={self.host_total} backend={self.backend_total} kv={self.kv_total} "
                f"scratch={self.scratch_total})")


class RunBudget:
    def __init__(self, limits: Limits):
        self.limits = limits
        self.bytes: Dict[Tuple[str, Tier], int] = {}
        self.denials = 0
        self.last_denial: Optional[Denial] = None
        self.peak_host = self.peak_backend = 0

    def _sum(self, kind: Optional[str] = None, tier: Optional[Tier] = None) -> int:
        return sum(v for (k, t), v in self.bytes.items() if (kind is None or k == kind) and (tier is None or t == tier))

    host_total = property(lambda self: self._sum(tier=Tier.HOST))
    backend_total = property(lambda self: self._sum(tier=Tier.BACKEND))
    kv_total = property(lambda self: self._sum(kind="kv"))
    scratch_total = property(lambda self: self._sum(kind="scratch"))

    def reserve(self, kind: str, tier: Tier, nbytes: int) -> Reservation:
        """Account ``nbytes`` or raise :class:`MemoryBudgetExceeded`; disk reservations are free."""
        r = Reservation(kind, tier, int(nbytes))
        if r.nbytes == 0 or tier is Tier.DISK:
            return r
        L = self.limits
        nh = self.host_total + (r.nbytes if tier is Tier.HOST else 0)
        nb = self.backend_total + (r.nbytes if tier is Tier.BACKEND else 0)
        nk = self.kv_total + (r.nbytes if kind == "kv" else 0)
        ns = self.scratch_total + (r.nbytes if kind == "scratch" else 0)
        for name, lim, cur, nxt in (("host_total", L.host, self.host_total, nh),
                                    ("backend_total", L.backend, self.backend_total, nb),
                                    ("combined_total", L.combined, self.host_total + self.backend_total, nh + nb),
                                    ("kv_total", L.kv, self.kv_total, nk),
                                    ("scratch_total", L.scratch, self.scratch_total, ns)):
            if lim and nxt > lim:
                self.denials += 1
                self.last_denial = Denial(r, name, cur, nxt, lim, self.host_total, self.backend_total, self.kv_total,
                                          self.scratch_total)
                raise MemoryBudgetExceeded(self.last_denial.line())
        self.bytes[(kind, tier)] = self.bytes.get((kind, tier), 0) + r.nbytes
        self.peak_host, self.peak_backend = max(self.peak_host, self.host_total), max(self.peak_backend, self.backend_total)
        return r

    def release(self, r: Reservation) -> None:
        if r.nbytes and r.tier is not Tier.DISK:
            k = (r.kind, r.tier)
            self.bytes[k] = max(0, self.bytes.get(k, 0) - r.nbytes)

    def denial_line(self) -> str:
        return self.last_denial.line() if self.last_denial else "memory budget exceeded"


# -- tiered tensor store ------------------------------------------------------------------------------------------
class DictSource:
    """Disk tier stand-in over tensors already in (pageable) memory; ``SafetensorsSource`` reads a file lazily."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.t = tensors

    def names(self) -> List[str]:
        return list(self.t)

    def nbytes(self, name: str) -> int:
        t = self.t[name]
        return t.numel() * t.element_size()

    def load(self, name: str) -> torch.Tensor:
        return self.t[name]


class SafetensorsSource:
    """Tensors of one safetensors file; each is a view of the memory map, so its pages are read on first touch."""

    def __init__(self, path: str):
        from ..formats.safetensors_io import SafetensorsFile

        self._f = SafetensorsFile(path)

    def names(self) -> List[str]:
        return list(self._f.keys())

    def nbytes(self, name: str) -> int:
        lo, hi = self._f.header[name]["data_offsets"]
        return int(hi - lo)

    def load(self, name: str) -> torch.Tensor:
        return self._f.tensor(name)


@dataclass(order=True)
class _Job:
    neg_priority: int
    seq: int
    name: str = field(compare=False)
    tier: Tier = field(compare=False)


class TieredStore:
    """Weights that do not all fit the top tier: every tensor has a home on disk, a bounded set is cached in pinned
    host memory and a bounded set on the device.  ``get`` returns a tensor at the best tier its placement and the
    budget allow, promoting it on the way and evicting the least recently used residents when a tier is full;
    ``prefetch`` asks the worker thread to do the same ahead of time (requests for a tensor that is already queued
    raise its priority instead of queueing it twice)."""

    def __init__(self, source, device, budget: Optional[RunBudget] = None, start_worker: bool = True):
        self.source, self.device = source, torch.device(device)
        self.gpu = self.device.type == "cuda"
        self.budget = budget or RunBudget(Limits())
        self.host: "OrderedDict[str, Tuple[torch.Tensor, Reservation]]" = OrderedDict()
        self.dev: "OrderedDict[str, Tuple[torch.Tensor, Reservation]]" = OrderedDict()
        self.stats = {"disk_reads": 0, "host_hits": 0, "backend_hits": 0, "promotions": 0, "evictions": 0,
                      "denials": 0, "prefetch_requests": 0, "prefetch_done": 0}
        self._lock = threading.RLock()
        self._cv = threading.Condition(self._lock)
        self._queue: List[_Job] = []
        self._pending: Dict[str, int] = {}        # name -> outstanding requests (its priority)
        self._seq = 0
        self._stop = False
        self._stream = torch.cuda.Stream(self.device) if self.gpu else None
        self._worker = None
        if start_worker:
            self._worker = threading.Thread(target=self._run, name="tier-prefetch", daemon=True)
            self._worker.start()

    # .. residency ..
    def tier_of(self, name: str) -> Tier:
        with self._lock:
            return Tier.BACKEND if name in self.dev else Tier.HOST if name in self.host else Tier.DISK

    def _make_room(self, cache, kind_tier: Tier, nbytes: int) -> Optional[Reservation]:
        """Reserve ``nbytes`` at a tier, evicting least-recently-used residents of that tier while refused."""
        while True:
            try:
                return self.budget.reserve("weight", kind_tier, nbytes)
            except MemoryBudgetExceeded:
                self.stats["denials"] += 1
                if not cache:
                    return None
                _, (_, res) = cache.popitem(last=False)
                self.budget.release(res)
                self.stats["evictions"] += 1

    def _to_host(self, name: str) -> Optional[torch.Tensor]:
        if name in self.host:
            self.host.move_to_end(name)
            self.stats["host_hits"] += 1
            return self.host[name][0]
        res = self._make_room(self.host, Tier.HOST, self.source.nbytes(name))
        if res is None:
            return None
        t = self.source.load(name).contiguous()
        self.stats["disk_reads"] += 1
        if self.gpu:
            t = t.pin_memory()
        self.host[name] = (t, res)
        self.stats["promotions"] += 1
        return t

    def get(self, name: str, tier: Tier = Tier.BACKEND) -> torch.Tensor:
        """The tensor at ``tier`` if it fits (after evictions), else at the next tier down; a tensor that fits
        nowhere is read from disk for this call only."""
        want = tier if self.gpu or tier is not Tier.BACKEND else Tier.HOST
        with self._lock:
            if want is Tier.BACKEND:
                if name in self.dev:
                    self.dev.move_to_end(name)
                    self.stats["backend_hits"] += 1
                    return self.dev[name][0]
                res = self._make_room(self.dev, Tier.BACKEND, self.source.nbytes(name))
                if res is not None:
                    h = self._to_host(name)
                    src = h if h is not None else self.source.load(name)
                    d = src.to(self.device, non_blocking=h is not None)
                    self.dev[name] = (d, res)
                    self.stats["promotions"] += 1
                    return d
            if want >= Tier.HOST:
                h = self._to_host(name)
                if h is not None:
                    return h.to(self.device) if tier is Tier.BACKEND and self.gpu else h
            self.stats["disk_reads"] += 1
            t = self.source.load(name)
            return t.to(self.device) if tier is Tier.BACKEND and self.gpu else t

    def drop(self, name: str) -> None:
        with self._lock:
            for cache in (self.dev, self.host):
                if name in cache:
                    self.budget.release(cache.pop(name)[1])

    # .. prefetch ..
    def prefetch(self, name: str, tier: Tier = Tier.BACKEND, hint: int = 1) -> int:
        """Queue a promotion; returns the tensor's outstanding request count (its priority)."""
        with self._cv:
            self.stats["prefetch_requests"] += 1
            self._pending[name] = self._pending.get(name, 0) + max(1, hint)
            self._seq += 1
            heapq.heappush(self._queue, _Job(-self._pending[name], self._seq, name, tier))
            self._cv.notify()
            return self._pending[name]

    def pending(self, name: str) -> int:
        with self._lock:
            return self._pending.get(name, 0)

    def drain(self, max_items: int = 1 << 30) -> int:
        """Run queued promotions on the calling thread (used without a worker, and by tests)."""
        n = 0
        while n < max_items:
            with self._lock:
                job = self._pop()
            if job is None:
                break
            self._do(job)
            n += 1
        return n

    def _pop(self) -> Optional[_Job]:
        while self._queue:
            job = heapq.heappop(self._queue)
            if self._pending.get(job.name, 0) and -job.neg_priority == self._pending[job.name]:
                return job                       # stale entries (superseded by a higher-priority one) are skipped
        return None

    def _do(self, job: _Job) -> None:
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                self.get(job.name, job.tier)
            self._stream.synchronize()
        else:
            self.get(job.name, job.tier)
        with self._lock:
            self._pending.pop(job.name, None)
            self.stats["prefetch_done"] += 1
            self._cv.notify_all()

    def _run(self) -> None:
        if self.gpu:
            torch.cuda.set_device(self.device)  # a new thread starts on device 0
        while True:
            with self._cv:
                job = self._pop()
                while job is None and not self._stop:
                    self._cv.wait(0.5)
                    job = self._pop()
                if self._stop:
                    return
            self._do(job)

    def wait_idle(self, timeout: float = 10.0) -> bool:
        import time

        end = time.monotonic() + timeout
        with self._cv:
            while self._pending and time.monotonic() < end:
                self._cv.wait(0.05)
            return not self._pending

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        if self._worker is not None:
            self._worker.join(timeout=2.0)


def budget_for_engine(engine, limits: Limits) -> RunBudget:
    """Account a loaded generation engine against per-run limits: its weights, its paged KV cache and its
    attention scratch, on the tier its device stands for.  Raises :class:`MemoryBudgetExceeded` (whose message is
    the denial line) when a limit is crossed, the way the reference refuses a run before it starts
    (zig/pkg/inference/src/runtime/tier/memory.zig:160 ``reserveEstimate``)."""
    tier = Tier.BACKEND if engine.device.type == "cuda" else Tier.HOST
    b = RunBudget(limits)
    b.reserve("weight", tier, int(engine.model.weight_bytes()))
    kv = engine.cache.k.numel() * engine.cache.k.element_size() + engine.cache.v.numel() * engine.cache.v.element_size()
    b.reserve("kv", tier, int(kv))
    m = engine.model
    scratch = 8 * engine.max_batch * m.Hq * (m.D + 1) * 4        # split-KV partial outputs + log-sum-exps, fp32
    b.reserve("scratch", tier, int(scratch))
    return b
