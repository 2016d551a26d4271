"""HBM budgeting for a generation deployment: how many bytes the weights, the paged KV cache and the step
activations take, and how many KV blocks fit next to the weights on one GPU.

The reference plans residency over GPU / RAM / NVMe tiers (zig/pkg/inference/src/runtime/tier/memory.zig:455,
``estimateGptGeneration``); a B200 holds 180 GB of HBM3e, so the planner here is the single-tier version: fit the
weights, reserve the activation and workspace peak, give the rest to KV blocks, and refuse a configuration that
cannot hold even one full-length sequence.
"""
from __future__ import annotations

from dataclasses import dataclass

HBM_BYTES_B200 = 180 * 10 ** 9


@dataclass
class MemoryEstimate:
    weight_bytes: int
    kv_bytes_per_token: int
    kv_bytes_per_block: int
    activation_bytes: int
    workspace_bytes: int

    def total(self, num_blocks: int) -> int:
        return self.weight_bytes + self.activation_bytes + self.workspace_bytes + num_blocks * self.kv_bytes_per_block


def estimate_generation(cfg, tp_size: int = 1, page: int = 16, kv_dtype_bytes: float = 2.0,
                        weight_bits: float = 8.25, max_step_tokens: int = 8192) -> MemoryEstimate:
    """Per-GPU bytes for a Llama-style decoder config under tensor parallelism.  ``weight_bits`` 8.25 = block-fp8
    (8 bits + one e8m0 scale byte per 32 values); the embedding table stays bf16 and is replicated."""
    H, L, F, V = cfg.hidden_size, cfg.num_hidden_layers, cfg.intermediate_size, cfg.vocab_size
    D = cfg.head_dim
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    hkv_local = max(hkv // tp_size, 1)
    per_layer = (hq * D * H + 2 * hkv * D * H) + hq * D * H + 3 * H * F  # qkv, o, gate/up/down
    linear_params = L * per_layer / tp_size + V * H / tp_size               # + vocabulary-sharded LM head
    weight_bytes = int(linear_params * weight_bits / 8) + V * H * 2 + (2 * L + 1) * H * 2
    kv_tok = int(2 * L * hkv_local * D * kv_dtype_bytes)
    # step activations: residual + normed + qkv + context + gate/up + a few fp32 split-K slices, per token
    act_tok = 2 * (2 * H + (hq + 2 * hkv) * D // tp_size + hq * D // tp_size + 3 * F // tp_size) + 8 * 4 * H
    logits = max_step_tokens and min(max_step_tokens, 256) * (V // tp_size) * 2
    return MemoryEstimate(weight_bytes, kv_tok, kv_tok * page, act_tok * max_step_tokens + logits, 512 << 20)


def plan_kv_blocks(cfg, hbm_bytes: int = HBM_BYTES_B200, tp_size: int = 1, page: int = 16,
                   kv_dtype_bytes: float = 2.0, max_seq_len: int = 8192, utilization: float = 0.92,
                   **kw) -> int:
    """Number of KV blocks that fit beside the weights; raises if not even one ``max_seq_len`` sequence fits."""
    est = estimate_generation(cfg, tp_size, page, kv_dtype_bytes, **kw)
    free = int(hbm_bytes * utilization) - est.weight_bytes - est.activation_bytes - est.workspace_bytes
    blocks = free // est.kv_bytes_per_block if free > 0 else 0
    need = (max_seq_len + page - 1) // page
    if blocks < need:
        raise MemoryError(f"model needs {est.weight_bytes / 1e9:.1f} GB of weights and {need} KV blocks for one "
                          f"sequence of {max_seq_len} tokens; only {max(blocks, 0)} blocks fit in "
                          f"{hbm_bytes / 1e9:.0f} GB at tp={tp_size}")
    return int(blocks)
