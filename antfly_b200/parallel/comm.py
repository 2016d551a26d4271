"""Process-group bootstrap and the baseline (NCCL-only) tensor-parallel communicator.

Environment contract (replaces the reference's TERMITE_MLX_* / MLX_* variables,
zig/pkg/inference/src/runtime/distributed.zig:18-63): ``RANK``, ``WORLD_SIZE``, ``LOCAL_RANK``, ``MASTER_ADDR``
(default 127.0.0.1), ``MASTER_PORT``; optional ``ANTFLY_B200_DISTRIBUTED_MODE`` = ``none | tensor_parallel |
data_parallel``.  One process per GPU.  ``TpComm`` is the path that only calls NCCL -- the baseline the fused
peer-memory kernels are compared against; it also works over gloo on CPU ranks for the host-logic tests.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistributedConfig:
    mode: str = "none"
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0

    @classmethod
    def from_env(cls, env=None) -> "DistributedConfig":
        e = env if env is not None else os.environ
        world = int(e.get("WORLD_SIZE", "1"))
        mode = e.get("ANTFLY_B200_DISTRIBUTED_MODE", "tensor_parallel" if world > 1 else "none")
        if mode not in ("none", "tensor_parallel", "data_parallel"):
            raise ValueError(f"unknown distributed mode {mode!r}")
        return cls(mode, int(e.get("RANK", "0")), world, int(e.get("LOCAL_RANK", e.get("RANK", "0"))))


def init_process_group(cfg: Optional[DistributedConfig] = None, backend: Optional[str] = None,
                       timeout_s: float = 600.0) -> DistributedConfig:
    cfg = cfg or DistributedConfig.from_env()
    if cfg.world_size <= 1 or dist.is_initialized():
        return cfg
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    use_cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if use_cuda else "gloo")
    kw = {}
    if backend == "nccl":
        torch.cuda.set_device(cfg.local_rank)
        kw["device_id"] = torch.device("cuda", cfg.local_rank)
    dist.init_process_group(backend, rank=cfg.rank, world_size=cfg.world_size,
                            timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return cfg


class TpComm:
    """Baseline collectives for tensor parallelism: all-reduce of row-parallel partial outputs and the merge of
    vocabulary-sharded arg-max results."""

    def __init__(self, rank: int, world: int, device, hidden: int = 0, max_tokens: int = 0, group=None):
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self.bytes_reduced = 0

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        self.bytes_reduced += t.numel() * t.element_size()
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        flat = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(flat, t, group=self.group)
        return flat.view((self.world,) + tuple(t.shape))

    def argmax_merge(self, idx: torch.Tensor, val: torch.Tensor) -> torch.Tensor:
        """Each rank holds the best (value, global index) of its vocabulary shard; returns the global arg-max
        (lowest index on ties), identical on every rank."""
        vals = self.all_gather(val.float())          # [W, R]
        idxs = self.all_gather(idx.int())            # [W, R]
        best = vals.max(0).values
        cand = torch.where(vals == best[None], idxs, torch.full_like(idxs, 2 ** 31 - 1))
        return cand.min(0).values.int()

    def barrier(self) -> None:
        dist.barrier(group=self.group)
