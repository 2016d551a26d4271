"""Mixture-of-experts runtime: route batching per expert, next-step expert prediction from co-activation statistics,
and a residency manager for expert weights that do not all fit on the device.

Mirrors the reference's MoE runtime (zig/pkg/inference/src/runtime/moe/runtime.zig:89-170 route batches and
per-layer predictions, runtime/moe/shared.zig:43-120 the cross-request co-activation cache, runtime/moe/
residency.zig:59-140 the touch-count / recency eviction order).  What is different by design:

* route batching is one stable sort of the [tokens x top-k] routing table on the device (no per-route appends), so
  every active expert gets one contiguous slice of token rows and weights;
* with 180 GB of HBM most MoE checkpoints are fully resident and the residency manager is a no-op; when a
  capacity is set, absent experts are copied from pinned host memory on a side stream, and the predicted experts
  of the next step are prefetched while the current step computes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import torch


@dataclass
class ExpertBatches:
    """Tokens grouped by expert: expert ``active[i]`` owns entries ``offsets[i]:offsets[i + 1]`` of ``rows`` (token
    index), ``slots`` (which of the token's top-k choices) and ``weights`` (routing weight)."""
    active: List[int]
    offsets: List[int]
    rows: torch.Tensor
    slots: torch.Tensor
    weights: torch.Tensor

    def __iter__(self):
        for i, e in enumerate(self.active):
            lo, hi = self.offsets[i], self.offsets[i + 1]
            yield e, self.rows[lo:hi], self.weights[lo:hi]


def route_batches(topk_idx: torch.Tensor, topk_w: torch.Tensor, num_experts: int) -> ExpertBatches:
    """topk_idx / topk_w [T, k] -> per-expert batches.  Token order inside an expert's batch is ascending (stable
    sort), which keeps results deterministic."""
    T, k = topk_idx.shape
    flat = topk_idx.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    counts_l = counts.tolist()                      # the one host read: expert batch sizes drive GEMM launches
    active = [e for e, c in enumerate(counts_l) if c]
    offsets = [0]
    for e in active:
        offsets.append(offsets[-1] + counts_l[e])
    return ExpertBatches(active, offsets, order // k, order % k, topk_w.reshape(-1)[order])


class CoactivationPredictor:
    """Which experts is a layer likely to need next?  Per layer: how often each expert was active and how often
    each pair was active together.  A candidate's score is its co-activation count with the currently active
    experts plus its own activity count; the best-scoring inactive experts are predicted (ties to the lowest
    index; candidates scoring zero are never predicted)."""

    def __init__(self):
        self.touch: Dict[int, torch.Tensor] = {}
        self.coact: Dict[int, torch.Tensor] = {}

    def note(self, layer: int, num_experts: int, active: Sequence[int]) -> None:
        if layer not in self.touch or self.touch[layer].numel() != num_experts:
            self.touch[layer] = torch.zeros(num_experts, dtype=torch.int64)
            self.coact[layer] = torch.zeros((num_experts, num_experts), dtype=torch.int64)
        a = torch.tensor(list(active), dtype=torch.long)
        self.touch[layer][a] += 1
        if a.numel() > 1:
            m = self.coact[layer]
            m[a[:, None], a[None, :]] += 1
            m[a, a] -= 1

    def predict(self, layer: int, active: Sequence[int], max_predicted: int) -> Tuple[List[int], List[int]]:
        if layer not in self.touch or not active or max_predicted <= 0:
            return [], []
        a = torch.tensor(list(active), dtype=torch.long)
        score = self.coact[layer][a].sum(0) + self.touch[layer]
        score[a] = -1
        out, scores = [], []
        for _ in range(max_predicted):
            best = int(torch.argmax(score))          # first maximum = lowest index among ties
            if score[best] <= 0:
                break
            out.append(best)
            scores.append(int(score[best]))
            score[best] = -1
        return out, scores


class ExpertResidency:
    """Bounded set of expert weights on the device, per layer.

    ``loader(layer, expert)`` returns the expert's weights on the device (typically a copy from pinned host
    memory); ``max_resident_per_layer`` 0 means everything stays resident.  Eviction order: fewest touches first,
    then least recently touched, then lowest expert index; experts needed by the current step are never evicted.
    """

    def __init__(self, loader: Callable[[int, int], object], max_resident_per_layer: int = 0,
                 prefetch_stream: Optional["torch.cuda.Stream"] = None):
        self.loader, self.cap, self.stream = loader, max_resident_per_layer, prefetch_stream
        self.resident: Dict[Tuple[int, int], object] = {}
        self.touches: Dict[Tuple[int, int], int] = {}
        self.last: Dict[Tuple[int, int], int] = {}
        self.step = 0
        self.stats = {"hits": 0, "misses": 0, "prefetched": 0, "prefetch_hits": 0, "evictions": 0}
        self._prefetched: set = set()

    def resident_count(self, layer: int) -> int:
        return sum(1 for (l, _e) in self.resident if l == layer)

    def _evict(self, layer: int, protect: set) -> None:
        if self.cap <= 0:
            return
        while self.resident_count(layer) > self.cap:
            cands = [(self.touches.get(k, 0), self.last.get(k, 0), k[1], k) for k in self.resident
                     if k[0] == layer and k not in protect]
            if not cands:
                return
            victim = min(cands)[3]
            del self.resident[victim]
            self._prefetched.discard(victim)
            self.stats["evictions"] += 1

    def ensure(self, layer: int, experts: Sequence[int]) -> Dict[int, object]:
        """Weights of the experts this step needs (loading the absent ones), and touch accounting."""
        self.step += 1
        need = {(layer, int(e)) for e in experts}
        if self.stream is not None and any(k in self._prefetched for k in need):
            torch.cuda.current_stream().wait_stream(self.stream)    # prefetched copies must have landed
        out = {}
        for k in sorted(need):
            self.touches[k] = self.touches.get(k, 0) + 1
            self.last[k] = self.step
            if k in self.resident:
                self.stats["hits"] += 1
                if k in self._prefetched:
                    self.stats["prefetch_hits"] += 1
                    self._prefetched.discard(k)
            else:
                self.stats["misses"] += 1
                self.resident[k] = self.loader(*k)
            out[k[1]] = self.resident[k]
        self._evict(layer, need)
        return out

    def prefetch(self, layer: int, experts: Sequence[int], protect: Sequence[int] = ()) -> int:
        """Start loading predicted experts (on the side stream when there is one); returns how many were started.
        Never evicts ``protect`` (the experts in use) and never exceeds the capacity."""
        started = 0
        keep = {(layer, int(e)) for e in protect}
        for e in experts:
            k = (layer, int(e))
            if k in self.resident:
                continue
            if self.cap > 0 and self.resident_count(layer) >= self.cap:
                evictable = [x for x in self.resident if x[0] == layer and x not in keep and x not in self._prefetched]
                if not evictable:
                    break
                victim = min(evictable, key=lambda x: (self.touches.get(x, 0), self.last.get(x, 0), x[1]))
                del self.resident[victim]
                self.stats["evictions"] += 1
            if self.stream is not None:
                with torch.cuda.stream(self.stream):
                    self.resident[k] = self.loader(*k)
            else:
                self.resident[k] = self.loader(*k)
            self._prefetched.add(k)
            self.stats["prefetched"] += 1
            started += 1
        return started


class HostExpertStore:
    """Expert weights parked in (pinned) host memory; ``load`` copies one expert to the device.  Works for plain
    tensors and for block-fp8 weights (anything with ``.to(device)``)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.host: Dict[Hashable, object] = {}

    def put(self, layer: int, expert: int, weights: Dict[str, object]) -> None:
        def park(v):
            v = v.to("cpu")
            if self.device.type == "cuda" and isinstance(v, torch.Tensor):
                v = v.pin_memory()
            return v

        self.host[(layer, expert)] = {n: park(v) for n, v in weights.items()}

    def load(self, layer: int, expert: int) -> Dict[str, object]:
        return {n: (v.to(self.device, non_blocking=True) if isinstance(v, torch.Tensor) else v.to(self.device))
                for n, v in self.host[(layer, expert)].items()}

    def bytes(self) -> int:
        tot = 0
        for ws in self.host.values():
            for v in ws.values():
                ts = [v] if isinstance(v, torch.Tensor) else [getattr(v, "q", None), getattr(v, "scales", None)]
                tot += sum(t.numel() * t.element_size() for t in ts if isinstance(t, torch.Tensor))
        return tot


class DiskExpertStore:
    """Expert weights whose home is a file on disk (NVMe): ``put`` collects them, ``seal`` writes one safetensors
    file and reopens it memory-mapped, ``load`` brings one expert to the device through a bounded pinned-host
    cache (:class:`antfly_b200.runtime.tiering.TieredStore`: least recently used experts leave the host tier when
    its budget is full, and come back from the file on their next use).  The third tier under
    :class:`HostExpertStore` for checkpoints whose experts exceed host memory too."""

    def __init__(self, device, path: str, host_budget_bytes: int = 0):
        self.device, self.path, self.host_budget = torch.device(device), path, int(host_budget_bytes)
        self._staged: Dict[str, torch.Tensor] = {}
        self._flags: Dict[Hashable, Dict[str, bool]] = {}
        self.store = None

    def put(self, layer: int, expert: int, weights: Dict[str, object]) -> None:
        if self.store is not None:
            raise RuntimeError("the store is sealed")
        self._flags[(layer, expert)] = {}
        for n, v in weights.items():
            key = f"l{layer}.e{expert}.{n}"
            if isinstance(v, torch.Tensor):
                self._staged[key] = v.to("cpu")
            else:                                       # block-fp8 weight: codes (as bytes) + scales
                q = v.q.to("cpu")
                self._staged[key + "::q"] = q.view(torch.uint8) if q.dtype != torch.uint8 else q
                self._staged[key + "::scales"] = v.scales.to("cpu")
                self._flags[(layer, expert)][n] = bool(v.interleaved_swiglu)

    def seal(self) -> None:
        from ..formats.safetensors_io import save_file
        from .tiering import Limits, RunBudget, SafetensorsSource, TieredStore

        save_file(self._staged, self.path)
        self._names = {k for k in self._staged}
        self._staged = {}
        self.store = TieredStore(SafetensorsSource(self.path), self.device, RunBudget(Limits(host=self.host_budget)),
                                 start_worker=False)

    def load(self, layer: int, expert: int) -> Dict[str, object]:
        from ..ops.quant import Fp8Weight
        from .tiering import Tier

        if self.store is None:
            self.seal()
        out: Dict[str, object] = {}
        pre = f"l{layer}.e{expert}."
        host = lambda k: self.store.get(k, Tier.HOST).to(self.device, non_blocking=True)
        for n, swiglu in self._flags[(layer, expert)].items():
            out[n] = Fp8Weight(host(pre + n + "::q").view(torch.float8_e4m3fn), host(pre + n + "::scales"), swiglu)
        for k in self._names:
            if k.startswith(pre) and "::" not in k:
                out[k[len(pre):]] = host(k)
        return out

    def bytes(self) -> int:
        return self.store.budget.host_total if self.store is not None else 0
