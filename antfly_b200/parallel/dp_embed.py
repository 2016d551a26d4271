"""Data-parallel embedding with the gather fused into the producer kernel.

Every rank embeds its slice of a global batch; the pooling kernel that produces the final [B_local, H] rows also
stores them into every rank's gathered buffer through peer pointers and bumps an arrival counter there, so after
the step each rank holds the embeddings of the whole batch without a separate all-gather.  (The reference defines
a ``data_parallel`` mode that nothing consumes: zig/pkg/inference/src/runtime/distributed.zig:18-63.)
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..models.bert import BertModel, PackedBatch
from ..ops.dense import POOL_MODES
from .fused import _ptr_array


class DpEmbedder:
    def __init__(self, model: BertModel, rank: int, world: int, max_local_batch: int = 512, group=None):
        self.model, self.rank, self.world, self.group = model, rank, world, group
        self.H = model.cfg.hidden_size
        self.max_local = max_local_batch
        self.device = model.device
        self._symm = None
        if world > 1 and self.device.type == "cuda":
            import torch.distributed._symmetric_memory as symm

            n = world * max_local_batch * self.H
            self._buf = symm.empty(n + 64, dtype=torch.float32, device=self.device)
            self._hdl = symm.rendezvous(self._buf, group or dist.group.WORLD)
            self._buf.zero_()
            torch.cuda.synchronize()
            dist.barrier(group)
            bases = [int(p) for p in self._hdl.buffer_ptrs]
            self._peer_out = _ptr_array(bases)
            self._peer_ready = _ptr_array([b + 4 * n for b in bases])
            self._n = n
            self._symm = symm

    def embed(self, local: PackedBatch, pooling: str = "mean", normalize: bool = True) -> torch.Tensor:
        """Embeds this rank's batch; returns the gathered fp32 [world * B_local, H] (every rank gets all rows).
        All ranks must pass the same local batch size."""
        h = self.model.encode(local)
        B = local.batch
        if self.world == 1:
            from ..ops import dense as Dn

            return Dn.pool(h, local.starts, local.lens, mode=pooling, normalize=normalize)
        if self._symm is None:  # CPU / gloo path
            from ..ops import dense as Dn

            mine = Dn.pool(h, local.starts, local.lens, mode=pooling, normalize=normalize)
            outs = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(outs, mine, group=self.group)
            return torch.cat(outs, 0)
        assert B <= self.max_local
        out = torch.empty((B, self.H), dtype=torch.float32, device=self.device)
        rc = N.cuda().afb_pool_gather(
            N.ptr(h), N.ptr(local.starts), N.ptr(local.lens), None, N.ptr(out), ctypes.c_int(B), ctypes.c_int(self.H),
            ctypes.c_int(POOL_MODES[pooling]), ctypes.c_int(1 if normalize else 0), self._peer_out, self._peer_ready,
            ctypes.c_int(self.world), ctypes.c_int(self.rank * B), N.stream_ptr())
        N.check(rc, "afb_pool_gather")
        N.count_launch()
        # Rows from every rank have landed once the counter reads world * B; the symmetric-memory barrier on the
        # stream orders that for the consumer and doubles as the "safe to overwrite next step" fence.
        self._hdl.barrier()
        gathered = self._buf[: self.world * B * self.H].view(self.world * B, self.H)
        ready = self._buf[self._n: self._n + 1].view(torch.int32)
        self.last_ready_count = ready.clone()
        ready.zero_()
        self._hdl.barrier()
        return gathered
