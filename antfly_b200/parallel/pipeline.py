"""Pipeline parallelism over decoder layers: the execution side of the planner's ``pipeline`` strategy.

Each rank holds a contiguous range of layers (and the KV cache of those layers only, which is what lets a model
that does not fit one GPU run at all); hidden states travel rank to rank with point-to-point sends, and the last
stage's logits are broadcast so that every rank samples the same token and keeps its scheduler and block tables in
step with the others -- all ranks run the same engine loop on the same requests, as with tensor parallelism.  The
reference cuts its graph at attention boundaries and walks the partitions in order, moving tensors through host
memory (zig/pkg/inference/src/graph/parallel_strategy.zig:181-320, graph/multi_executor.zig); here the transfers
are ``torch.distributed`` point-to-point calls (NCCL over NVLink between GPUs, gloo between CPU ranks).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .strategy import ParallelPlan


class PipelineStage:
    def __init__(self, rank: int, world: int, group=None, dtype=torch.bfloat16):
        self.rank, self.world, self.group, self.dtype = rank, world, group, dtype
        self.sent_bytes = self.received_bytes = 0

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world - 1

    def recv_hidden(self, tokens: int, hidden: int, device) -> torch.Tensor:
        buf = torch.empty((tokens, hidden), dtype=self.dtype, device=device)
        dist.recv(buf, src=self.rank - 1, group=self.group)
        self.received_bytes += buf.numel() * buf.element_size()
        return buf

    def send_hidden(self, x: torch.Tensor) -> None:
        x = x.to(self.dtype).contiguous()
        dist.send(x, dst=self.rank + 1, group=self.group)
        self.sent_bytes += x.numel() * x.element_size()

    def share_logits(self, logits: Optional[torch.Tensor], rows: int, width: int, device) -> torch.Tensor:
        """Broadcast the last stage's output rows to every stage."""
        buf = logits.to(self.dtype).contiguous() if self.is_last else torch.empty((rows, width), dtype=self.dtype,
                                                                                  device=device)
        dist.broadcast(buf, src=self.world - 1, group=self.group)
        return buf


def build_stage(cfg, sd, plan: ParallelPlan, rank: int, device="cuda", group=None):
    """Load rank ``rank``'s layers of a pipeline plan and wire the stage transport."""
    from ..models.llama import LlamaModel

    if plan.strategy != "pipeline":
        raise ValueError(f"not a pipeline plan: {plan.strategy}")
    first, last = plan.ranks[rank].layers
    model = LlamaModel.from_state_dict(cfg, sd, device=device, layers=(first, last))
    model.set_pipeline(PipelineStage(rank, plan.world, group), first, last)
    return model
