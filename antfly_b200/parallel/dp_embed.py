"""Data-parallel embedding with the gather fused into the producer kernel.

Every rank embeds its slice of a global batch; the pooling kernel that produces the final [B_local, H] rows also
stores them into every rank's gathered buffer through peer pointers and bumps an arrival counter there, so after
the step each rank holds the embeddings of the whole batch without a separate all-gather.  (The reference defines
a ``data_parallel`` mode that nothing consumes: zig/pkg/inference/src/runtime/distributed.zig:18-63.)

Hand-off protocol (no barrier anywhere, every wait bounded):

* Two gathered buffers alternate between consecutive steps, each with its own arrival counter.  Counters only
  ever grow; the consumer waits for the cumulative number of rows pushed into that buffer so far, so nothing is
  reset and no reset can race with a fast peer.
* The consumer is a one-warp kernel on the same stream (``afb_peer_counter_wait``): it polls the counter with
  ``ld.acquire.sys`` for at most the cross-GPU wait limit, then records a timeout in the status word and returns.
  Whatever is launched after it on the stream sees the gathered rows.
* A rank can push into a buffer again only after it has finished the wait of the step in between, which needs
  every peer to have run that step's pooling kernel -- and a peer launches that kernel after everything it
  enqueued for the older step.  So rows returned by ``embed`` stay intact for work enqueued on the stream before
  the next ``embed`` call; copy them if they must live longer.
* All ranks must call ``embed`` the same number of times with the same local batch size.  After a timeout the
  counters of the ranks disagree: read the status word, tear the group down and build a new ``DpEmbedder``.
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


class GatherSchedule:
    """Host-side bookkeeping of the double-buffered gather: which buffer a step uses and the cumulative arrival
    count its consumer waits for.  Pure arithmetic, shared with the CPU protocol model in the tests."""

    def __init__(self, world: int):
        self.world = world
        self.step = 0
        self.pushed = [0, 0]  # rows pushed into buffer 0 / 1 so far, by all ranks together

    def next(self, local_rows: int):
        """-> (buffer parity, arrival target of this step's consumer)."""
        par = self.step & 1
        self.pushed[par] += self.world * local_rows
        self.step += 1
        return par, _wrap_i32(self.pushed[par])


def _wrap_i32(v: int) -> int:
    v &= 0xFFFFFFFF
    return v - (1 << 32) if v >= (1 << 31) else v


class DpEmbedder:
    def __init__(self, model: BertModel, rank: int, world: int, max_local_batch: int = 512, group=None):
        self.model, self.rank, self.world, self.group = model, rank, world, group
        self.H = model.cfg.hidden_size
        self.max_local = max_local_batch
        self.device = model.device
        self._symm = None
        self.sched = GatherSchedule(world)
        if world > 1 and self.device.type == "cuda":
            import torch.distributed._symmetric_memory as symm

            n = world * max_local_batch * self.H  # floats per gathered buffer
            self._buf = symm.empty(2 * n + 64, dtype=torch.float32, device=self.device)
            self._hdl = symm.rendezvous(self._buf, group or dist.group.WORLD)
            self._buf.zero_()
            torch.cuda.synchronize()
            dist.barrier(group)  # host-side: nobody pushes before every rank's counters are zero
            bases = [int(p) for p in self._hdl.buffer_ptrs]
            self._peer_out = [_ptr_array([b + 4 * n * par for b in bases]) for par in (0, 1)]
            self._peer_ready = [_ptr_array([b + 4 * (2 * n + par) for b in bases]) for par in (0, 1)]
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
        par, target = self.sched.next(B)
        out = torch.empty((B, self.H), dtype=torch.float32, device=self.device)
        lib = N.cuda()
        rc = lib.afb_pool_gather(
            N.ptr(h), N.ptr(local.starts), N.ptr(local.lens), None, N.ptr(out), ctypes.c_int(B), ctypes.c_int(self.H),
            ctypes.c_int(POOL_MODES[pooling]), ctypes.c_int(1 if normalize else 0), self._peer_out[par],
            self._peer_ready[par], ctypes.c_int(self.world), ctypes.c_int(self.rank * B), N.stream_ptr())
        N.check(rc, "afb_pool_gather")
        ready = self._buf[2 * self._n + par: 2 * self._n + par + 1]
        rc = lib.afb_peer_counter_wait(N.ptr(ready), ctypes.c_int(target), N.stream_ptr())
        N.check(rc, "afb_peer_counter_wait")
        N.count_launch(2)
        base = par * self._n
        return self._buf[base: base + self.world * B * self.H].view(self.world * B, self.H)
