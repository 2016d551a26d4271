"""Parallel-strategy planner: single device, tensor parallel, or pipeline parallel.

The reference plans a graph partition (zig/pkg/inference/src/graph/parallel_strategy.zig:60-323): ``single``;
``pipeline`` = cut the layer stack at attention boundaries into contiguous stages, one per device; ``tensor`` =
replicate the graph and shard the weights by the Megatron rules.  The plan here is the same decision expressed on
decoder layers: which layers a rank runs (pipeline) or which slice of every layer it holds (tensor), checked against
the divisibility the kernels need.  ``tensor`` plans run through the fused tensor-parallel kernels; ``pipeline``
plans through :mod:`antfly_b200.parallel.pipeline` (layer ranges per rank, hidden states sent rank to rank).
Mixture-of-experts checkpoints can additionally split their routed experts across ranks
(``LlamaModel.set_expert_parallel``: replicated routing, local experts, one all-reduce per MoE layer).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple


@dataclass
class RankPlan:
    rank: int
    layers: Tuple[int, int]            # [first, last) decoder layers this rank executes
    tp_rank: int = 0
    tp_size: int = 1
    holds_embedding: bool = True
    holds_lm_head: bool = True


@dataclass
class ParallelPlan:
    strategy: str                       # single | tensor | pipeline
    world: int
    ranks: List[RankPlan] = field(default_factory=list)
    notes: List[str] = field(default_factory=list)


def plan_parallel(cfg, world: int, strategy: Optional[str] = None, hbm_bytes: Optional[int] = None) -> ParallelPlan:
    """Choose / validate a strategy for ``world`` GPUs.  ``strategy`` None picks tensor parallelism when the head
    counts divide (it shortens every step), else pipeline, else single."""
    L = cfg.num_hidden_layers
    hq, hkv, F = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    if world <= 1:
        return ParallelPlan("single", 1, [RankPlan(0, (0, L))])
    tp_ok = hq % world == 0 and (hkv % world == 0 or world % hkv == 0) and (F // world) % 128 == 0 and \
        cfg.vocab_size % world == 0
    if strategy is None:
        strategy = "tensor" if tp_ok else ("pipeline" if L >= world else "single")
    if strategy == "tensor":
        if not tp_ok:
            raise ValueError(f"tensor parallel over {world} GPUs needs heads ({hq}/{hkv}), FFN ({F}) and vocabulary "
                             f"({cfg.vocab_size}) to split evenly (FFN shard a multiple of 128)")
        plan = ParallelPlan("tensor", world, [RankPlan(r, (0, L), r, world) for r in range(world)])
        if hkv < world:
            plan.notes.append(f"{hkv} KV heads over {world} ranks: KV heads are replicated {world // hkv}x")
        return plan
    if strategy == "pipeline":
        if L < world:
            raise ValueError(f"pipeline parallel needs at least one layer per stage ({L} layers, {world} stages)")
        base, extra = divmod(L, world)
        ranks, first = [], 0
        for r in range(world):
            n = base + (1 if r < extra else 0)
            ranks.append(RankPlan(r, (first, first + n), holds_embedding=r == 0, holds_lm_head=r == world - 1))
            first += n
        return ParallelPlan("pipeline", world, ranks, ["stage boundaries fall between decoder layers; activations "
                                                       "cross stages once per boundary per step"])
    if strategy == "single":
        return ParallelPlan("single", world, [RankPlan(0, (0, L))], ["extra GPUs idle (or serve replicas)"])
    raise ValueError(f"unknown strategy {strategy!r}")
