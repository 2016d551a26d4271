"""Sharded vector search across GPUs: one index shard per rank, per-rank top-k, cross-GPU merge.

Each rank searches its shard with global ids (``id_offset`` = first row of the shard).  The merge is the select
kernel reading every rank's (distance, id) list straight out of peer memory: the lists live in a symmetric buffer,
a rank publishes its list, ranks meet at a barrier on the stream, and every rank (or only rank 0) selects the k
best of world * k candidates.  No host hop, no NCCL all-gather of candidates.  Over gloo / CPU the same merge runs
through ``all_gather`` for the host-logic tests.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import index_ops as IX
from .flat import FlatIndex, SearchResult


class ShardedFlatIndex:
    def __init__(self, local_vectors: torch.Tensor, metric: str, rank: int, world: int, rows_per_rank: int,
                 storage: str = "bf16", max_queries: int = 1024, max_k: int = 128, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.local = FlatIndex(local_vectors, metric=metric, storage=storage, id_offset=rank * rows_per_rank)
        self.device = self.local.device
        self.max_queries, self.max_k = max_queries, max_k
        self._symm = None
        if world > 1 and self.device.type == "cuda":
            import torch.distributed._symmetric_memory as symm

            n = max_queries * max_k
            self._buf = symm.empty(2 * n, dtype=torch.float32, device=self.device)  # values then ids (int32 bits)
            self._hdl = symm.rendezvous(self._buf, group or dist.group.WORLD)
            self._symm = symm

    def search(self, queries: torch.Tensor, k: int) -> SearchResult:
        res = self.local.search(queries, k)
        if self.world == 1:
            return res
        nq = res.distances.shape[0]
        if self._symm is None:
            vals = [torch.empty_like(res.distances) for _ in range(self.world)]
            ids = [torch.empty_like(res.ids) for _ in range(self.world)]
            dist.all_gather(vals, res.distances.contiguous(), group=self.group)
            dist.all_gather(ids, res.ids.contiguous(), group=self.group)
            srcs = [(v, i, None, k) for v, i in zip(vals, ids)]
            tv, ti, _, _ = IX.topk_select(srcs, nq, k, self.world * k)
            return SearchResult(tv, ti)
        assert nq <= self.max_queries and k <= self.max_k
        n = self.max_queries * self.max_k
        my_v = self._buf[: nq * k].view(nq, k)
        my_i = self._buf[n: n + nq * k].view(torch.int32).view(nq, k)
        my_v.copy_(res.distances)
        my_i.copy_(res.ids)
        self._hdl.barrier()  # every rank's list is published before anyone reads
        srcs = []
        for r in range(self.world):
            pb = self._hdl.get_buffer(r, (2 * n,), torch.float32)
            srcs.append((pb[: nq * k].view(nq, k), pb[n: n + nq * k].view(torch.int32).view(nq, k), None, k))
        tv, ti, _, _ = IX.topk_select(srcs, nq, k, self.world * k)
        self._hdl.barrier()  # nobody overwrites its list while a peer still reads it
        return SearchResult(tv, ti)
