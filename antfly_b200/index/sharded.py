"""Sharded vector search across GPUs: one index shard per rank, per-rank top-k, cross-GPU merge.

Each rank searches its shard with global ids (``id_offset`` = first row of the shard).  The merge is fused into
the two select launches that exist anyway:

* push: the select that finishes a shard's local search (the tail of the score GEMM's candidate stream) stores
  each query's k best, plus a flag "a candidate buffer of this shard overflowed", into EVERY rank's merge buffer
  through peer pointers and bumps every rank's arrival counter (``red.release.sys``), one bump per query CTA;
* merge: one select per rank waits -- bounded, a status word on expiry -- for its own counter to reach the
  cumulative number of query rows pushed so far, then picks the k best of world * k candidates that now sit in
  local memory.

There is no barrier and no separate gather: two merge buffers alternate between consecutive searches and the
counters only grow, so a rank can overwrite a buffer only after the search in between, which every peer enters
after it has finished reading.  If any shard overflowed a candidate buffer (adversarially ordered data), every
rank learns it from the pushed flags and all of them repeat the search on the safe path together.

All ranks must call ``search`` in the same order with the same number of queries and the same k.  Over gloo /
CPU the same merge runs through ``all_gather`` for the host-logic tests.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops import index_ops as IX
from ..parallel.dp_embed import GatherSchedule
from .flat import FlatIndex, SearchResult


class MergeWorkspace:
    """Symmetric merge buffers of one rank: for each of two parities, world slots of [max_queries, max_k] values
    and ids and [max_queries] flags, plus one arrival counter per parity.  Shared by the flat and IVF shards."""

    def __init__(self, rank: int, world: int, device, max_queries: int, max_k: int, group=None):
        import torch.distributed._symmetric_memory as symm

        self.rank, self.world, self.device = rank, world, device
        self.max_queries, self.max_k = max_queries, max_k
        self.slot = max_queries * max_k
        self.per_par = world * (2 * self.slot + max_queries)  # words per parity
        words = 2 * self.per_par + 64
        self.buf = symm.empty(words, dtype=torch.int32, device=device)
        self.hdl = symm.rendezvous(self.buf, group or dist.group.WORLD)
        self.buf.zero_()
        torch.cuda.synchronize()
        dist.barrier(group)  # host-side: counters are zero everywhere before the first push
        self.bases = [int(p) for p in self.hdl.buffer_ptrs]
        self.sched = GatherSchedule(world)

    # word offsets inside one rank's buffer
    def _val(self, par: int, src: int) -> int:
        return par * self.per_par + src * self.slot

    def _idx(self, par: int, src: int) -> int:
        return par * self.per_par + self.world * self.slot + src * self.slot

    def _flag(self, par: int, src: int) -> int:
        return par * self.per_par + 2 * self.world * self.slot + src * self.max_queries

    def _ready(self, par: int) -> int:
        return 2 * self.per_par + par

    def push_targets(self, par: int):
        """Peer addresses of this rank's slot in every rank's buffer: (vals, ids, flags, counters)."""
        P = ctypes.c_void_p * self.world
        r = self.rank
        return (P(*[b + 4 * self._val(par, r) for b in self.bases]), P(*[b + 4 * self._idx(par, r) for b in self.bases]),
                P(*[b + 4 * self._flag(par, r) for b in self.bases]), P(*[b + 4 * self._ready(par) for b in self.bases]))

    def merge(self, par: int, target: int, nq: int, k: int):
        """Select the k best over the world slots of parity `par` once `target` query rows have arrived."""
        srcs, flags = [], []
        for s in range(self.world):
            v = self.buf[self._val(par, s): self._val(par, s) + nq * k].view(torch.float32).view(nq, k)
            i = self.buf[self._idx(par, s): self._idx(par, s) + nq * k].view(nq, k)
            srcs.append((v, i, None, k))
            flags.append(self.buf[self._flag(par, s): self._flag(par, s) + nq])
        ready = self.buf[self._ready(par): self._ready(par) + 1]
        return IX.topk_select(srcs, nq, k, self.world * k, want_threshold=False, wait=(ready, target),
                              src_flags=flags)


class ShardedFlatIndex:
    def __init__(self, local_vectors: torch.Tensor, metric: str, rank: int, world: int, rows_per_rank: int,
                 storage: str = "bf16", max_queries: int = 1024, max_k: int = 128, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.local = FlatIndex(local_vectors, metric=metric, storage=storage, id_offset=rank * rows_per_rank)
        self.device = self.local.device
        self.max_queries, self.max_k = max_queries, max_k
        self.ws: Optional[MergeWorkspace] = None
        if world > 1 and self.device.type == "cuda":
            self.ws = MergeWorkspace(rank, world, self.device, max_queries, max_k, group)

    def search(self, queries: torch.Tensor, k: int) -> SearchResult:
        if self.world == 1:
            return self.local.search(queries, k)
        if self.ws is None:
            res = self.local.search(queries, k)
            return merge_over_group(res, k, self.world, self.group)
        nq = queries.shape[0]
        assert nq <= self.max_queries and k <= self.max_k
        ws = self.ws
        par, target = ws.sched.next(nq)
        self.local._search(queries, k, push=ws.push_targets(par))
        tv, ti, _, ovf = ws.merge(par, target, nq, k)
        if int(ovf):  # some shard overflowed a candidate buffer: every rank sees the flag, all take the safe path
            par, target = ws.sched.next(nq)
            self.local._search(queries, k, push=ws.push_targets(par), safe=True)
            tv, ti, _, _ = ws.merge(par, target, nq, k)
        return SearchResult(tv, ti)


def merge_over_group(res: SearchResult, k: int, world: int, group=None) -> SearchResult:
    """Host-logic twin of the device merge (gloo / CPU ranks): all-gather the per-rank lists, select the k best."""
    nq = res.distances.shape[0]
    vals = [torch.empty_like(res.distances) for _ in range(world)]
    ids = [torch.empty_like(res.ids) for _ in range(world)]
    dist.all_gather(vals, res.distances.contiguous(), group=group)
    dist.all_gather(ids, res.ids.contiguous(), group=group)
    srcs = [(v, i, None, k) for v, i in zip(vals, ids)]
    tv, ti, _, _ = IX.topk_select(srcs, nq, k, world * k)
    return SearchResult(tv, ti)


class ShardedIVFIndex:
    """IVF over a database split across ranks: the k-means centroids are trained jointly (the update's sums and
    counts are all-reduced, so every rank holds the same centroids and probes the same lists); every rank keeps the
    members of all lists that fall into its shard, searches them with the fixed launch sequence of
    :class:`IVFIndex`, and the final select pushes into every rank's merge buffer."""

    def __init__(self, local_vectors: torch.Tensor, n_lists: int, metric: str, rank: int, world: int,
                 rows_per_rank: int, max_queries: int = 1024, max_k: int = 128, group=None, train_sample: int = 0,
                 max_iter: int = 16):
        from .ivf import IVFIndex

        self.rank, self.world, self.group = rank, world, group
        all_reduce = None
        if world > 1:
            def all_reduce(t):
                dist.all_reduce(t, group=group)
                return t
        init = None
        if world > 1:
            # one seed set for everybody: rank 0 draws n_lists of its rows, all ranks start Lloyd from them
            dev = local_vectors.device
            g = torch.Generator(device=dev).manual_seed(0)
            pick = torch.randperm(local_vectors.shape[0], generator=g, device=dev)[:n_lists]
            init = local_vectors[pick].float().contiguous()
            if init.shape[0] < n_lists:
                init = torch.cat([init, torch.randn(n_lists - init.shape[0], init.shape[1], device=dev)], 0)
            dist.broadcast(init, src=0, group=group)
        self.local = IVFIndex(local_vectors, n_lists, metric=metric, max_iter=max_iter, train_sample=train_sample,
                              id_offset=rank * rows_per_rank, all_reduce=all_reduce, init_centroids=init)
        self.device = self.local.x.device
        self.max_queries, self.max_k = max_queries, max_k
        self.ws: Optional[MergeWorkspace] = None
        if world > 1 and self.device.type == "cuda":
            self.ws = MergeWorkspace(rank, world, self.device, max_queries, max_k, group)

    def search(self, queries: torch.Tensor, k: int, nprobe: int = 64) -> SearchResult:
        if self.world == 1:
            return self.local.search(queries, k, nprobe)
        if self.ws is None:
            return merge_over_group(self.local.search(queries, k, nprobe), k, self.world, self.group)
        nq = queries.shape[0]
        assert nq <= self.max_queries and k <= self.max_k
        ws = self.ws
        par, target = ws.sched.next(nq)
        # pushed ids must be global: map sorted rows to ids before the push select
        res = self.local.search(queries, k, nprobe, check=False)
        ovf_local = res.overflow
        IX.topk_select([(res.distances.contiguous(), res.ids.contiguous(), None, k)], nq, k, k,
                       overflow=ovf_local, push=ws.push_targets(par))
        tv, ti, _, ovf = ws.merge(par, target, nq, k)
        if int(ovf):  # every rank sees the same flags: all repeat on the safe path together
            par, target = ws.sched.next(nq)
            safe = self.local._search_host(queries, k, nprobe)
            IX.topk_select([(safe.distances.contiguous(), safe.ids.contiguous(), None, k)], nq, k, k,
                           push=ws.push_targets(par))
            tv, ti, _, _ = ws.merge(par, target, nq, k)
        return SearchResult(tv, ti)
