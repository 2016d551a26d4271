"""Tensor-parallel weight sharding rules.

Same split as the reference's gpt_tensor_parallel_rules (zig/pkg/inference/src/graph/sharding.zig:28-130):
q/k/v/gate/up projections are split by output rows (column-parallel), o/down by input columns (row-parallel),
everything else is replicated.  Block-scaled fp8 weights shard on 32-element K blocks, so a column split must
land on a multiple of 32.
"""
from __future__ import annotations

import re
from typing import Dict

import torch

COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "query", "key", "value",
                   "intermediate.dense")
ROW_PARALLEL = ("o_proj", "down_proj", "attention.output.dense", "output.dense")


def shard_dim(name: str) -> int:
    """0: split output rows, 1: split input columns, -1: replicate."""
    if name.endswith(".bias"):
        base = name[: -len(".bias")]
        return 0 if any(base.endswith(k) for k in COLUMN_PARALLEL) else -1
    base = name[: -len(".weight")] if name.endswith(".weight") else name
    # "attention.output.dense" must be tested before the generic "output.dense".
    if any(base.endswith(k) for k in COLUMN_PARALLEL):
        return 0
    if any(base.endswith(k) for k in ROW_PARALLEL):
        return 1
    return -1


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    if world == 1:
        return w
    n = w.shape[0]
    assert n % world == 0, f"cannot split {n} rows over {world} ranks"
    s = n // world
    return w[rank * s:(rank + 1) * s].contiguous()


def shard_cols(w: torch.Tensor, rank: int, world: int, block: int = 32) -> torch.Tensor:
    if world == 1:
        return w
    k = w.shape[1]
    assert k % (world * block) == 0, f"cannot split {k} columns over {world} ranks on {block}-element blocks"
    s = k // world
    return w[:, rank * s:(rank + 1) * s].contiguous()


def shard_state_dict(sd: Dict[str, torch.Tensor], rank: int, world: int) -> Dict[str, torch.Tensor]:
    out = {}
    for name, t in sd.items():
        d = shard_dim(name)
        if d == 0:
            out[name] = shard_rows(t, rank, world)
        elif d == 1 and t.dim() == 2:
            out[name] = shard_cols(t, rank, world, block=1 if t.shape[1] % (world * 32) else 32)
        else:
            out[name] = t
    return out
