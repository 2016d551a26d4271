"""LayerNorm-based decoder family: GPT-2, GPT-Neo, GPT-NeoX / Pythia, OPT, GPT-J, Phi (1 / 1.5 / 2) and Falcon, on the same
paged-KV engine interface as :class:`antfly_b200.models.llama.LlamaModel`.

What differs from the Llama family and how it maps onto the existing kernels (the reference covers these under one
``ModelFamily`` switch, zig/pkg/inference/src/models/gpt.zig:28-233, zig/pkg/inference/src/architectures/gpt.zig):

* LayerNorm with bias instead of RMSNorm: the same norm kernel (``rms=False``, beta), fused with the residual add.
* biased linears with a GELU (erf or tanh form) / ReLU MLP: the bf16 tcgen05 GEMM with its bias + activation +
  residual epilogues; weights stay bf16 (these are small models).
* learned absolute positions (GPT-2, OPT with its offset of 2): added to the token embedding; the RoPE + KV-write
  kernel is then run with all positions zero, which rotates by the identity and only writes K / V into the cache.
* partial rotary embedding and the parallel residual of GPT-NeoX (``x + attn(ln1 x) + mlp(ln2 x)``).
* the single-norm parallel block of GPT-J and Phi (``x + attn(ln x) + mlp(ln x)``), GPT-J's interleaved
  ("consecutive pairs") rotary embedding, and the biased LM head both of them carry.
* fused QKV layouts: GPT-2's ``c_attn`` is a transposed ``Conv1D`` [in, 3 * out]; GPT-NeoX interleaves q, k, v per
  head; both are re-packed at load time into the [q heads | k heads | v heads] rows the kernels expect.
* GPT-Neo: unscaled attention scores (softmax scale 1) and layers that alternate between global attention and a
  256-token sliding window.
* Falcon: multi-query (one shared K / V head) or grouped K / V heads, rotary positions, bias-free linears, the
  parallel block with one shared LayerNorm (7B) or two (``new_decoder_architecture``), whose fused QKV rows are
  grouped per K / V head and are regrouped at load time.  ALiBi variants are not supported.
* BLOOM: a LayerNorm on the token embeddings, no position embeddings at all -- attention scores get the ALiBi bias
  ``slope_h * (key - query)`` instead.  The paged flash kernel has no bias input, so this family's attention runs
  through the tensor-op reference path on either device (correct, not a tuned path).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..ops import attention as A
from ..ops import dense as Dn
from ..ops import reference as R
from ..ops import sampling as S
from .llama import StepBatch


@dataclass
class GptConfig:
    family: str = "gpt2"              # gpt2 | gpt_neo | gpt_neox | opt | gptj | phi | falcon | bloom
    vocab_size: int = 50257
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 1024
    layer_norm_eps: float = 1e-5
    activation: str = "gelu_tanh"     # gelu | gelu_tanh | relu
    rope_theta: float = 10000.0
    rotary_pct: float = 0.0           # 0: learned absolute positions
    parallel_residual: bool = False
    position_offset: int = 0          # OPT: 2
    tie_word_embeddings: bool = True
    sliding_window: int = 0
    shared_norm: bool = False         # GPT-J / Phi: one LayerNorm feeds both the attention and the MLP branch
    rope_half_split: bool = True      # False: GPT-J pairs (2i, 2i + 1) instead of (i, i + rot/2)
    num_kv_heads: int = 0             # 0: one K / V head per query head; Falcon: 1 (multi-query) or a group count
    attn_scale: float = 0.0           # 0: 1 / sqrt(head_dim); GPT-Neo: 1
    layer_windows: Optional[List[int]] = None   # per-layer sliding window (0 = global); GPT-Neo's local layers
    alibi: bool = False               # BLOOM: linear position bias on the scores, no position embeddings

    # Names the engine reads from every decoder config.
    @property
    def num_key_value_heads(self) -> int:
        return self.num_kv_heads or self.num_attention_heads

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def from_hf(cls, d: dict) -> "GptConfig":
        mt = d.get("model_type", "gpt2")
        act = {"gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh", "gelu": "gelu",
               "relu": "relu"}
        if mt == "gpt2":
            H = d.get("n_embd", d.get("hidden_size", 768))
            return cls("gpt2", d["vocab_size"], H, d.get("n_layer", d.get("num_hidden_layers", 12)),
                       d.get("n_head", d.get("num_attention_heads", 12)), d.get("n_inner") or 4 * H,
                       d.get("n_positions", d.get("max_position_embeddings", 1024)),
                       d.get("layer_norm_epsilon", 1e-5), act[d.get("activation_function", "gelu_new")],
                       tie_word_embeddings=d.get("tie_word_embeddings", True))
        if mt == "gpt_neox":
            rp = d.get("rope_parameters") or d.get("rope_scaling") or {}
            theta = d.get("rope_theta") or d.get("rotary_emb_base") or rp.get("rope_theta") or 10000.0
            pct = d.get("rotary_pct") or rp.get("partial_rotary_factor") or d.get("partial_rotary_factor") or 1.0
            return cls("gpt_neox", d["vocab_size"], d["hidden_size"], d["num_hidden_layers"],
                       d["num_attention_heads"], d["intermediate_size"], d.get("max_position_embeddings", 2048),
                       d.get("layer_norm_eps", 1e-5), act[d.get("hidden_act", "gelu")], float(theta), float(pct),
                       bool(d.get("use_parallel_residual", True)),
                       tie_word_embeddings=d.get("tie_word_embeddings", False))
        if mt == "opt":
            assert d.get("do_layer_norm_before", True), "post-LayerNorm OPT variants (350m) are not supported"
            assert d.get("word_embed_proj_dim", d["hidden_size"]) == d["hidden_size"]
            return cls("opt", d["vocab_size"], d["hidden_size"], d["num_hidden_layers"], d["num_attention_heads"],
                       d["ffn_dim"], d.get("max_position_embeddings", 2048), 1e-5,
                       act[d.get("activation_function", "relu")], position_offset=2,
                       tie_word_embeddings=d.get("tie_word_embeddings", True))
        if mt == "gptj":
            H, nh = d["n_embd"], d["n_head"]
            rot = d.get("rotary_dim") or (H // nh)
            return cls("gptj", d["vocab_size"], H, d["n_layer"], nh, d.get("n_inner") or 4 * H,
                       d.get("n_positions", 2048), d.get("layer_norm_epsilon", 1e-5),
                       act[d.get("activation_function", "gelu_new")], 10000.0, rot / (H // nh), True,
                       tie_word_embeddings=False, shared_norm=True, rope_half_split=False)
        if mt == "phi":
            rp = d.get("rope_parameters") or d.get("rope_scaling") or {}
            theta = d.get("rope_theta") or rp.get("rope_theta") or 10000.0
            pct = d.get("partial_rotary_factor") or rp.get("partial_rotary_factor") or 0.5
            return cls("phi", d["vocab_size"], d["hidden_size"], d["num_hidden_layers"], d["num_attention_heads"],
                       d["intermediate_size"], d.get("max_position_embeddings", 2048), d.get("layer_norm_eps", 1e-5),
                       act[d.get("hidden_act", "gelu_new")], float(theta), float(pct), True,
                       tie_word_embeddings=False, shared_norm=True)
        if mt == "gpt_neo":
            H, L = d["hidden_size"], d.get("num_layers", d.get("num_hidden_layers"))
            kinds = d.get("attention_layers")
            if not kinds:
                kinds = [k for pat, rep in d.get("attention_types", [[["global"], L]]) for _ in range(rep) for k in pat]
            win = int(d.get("window_size", 256))
            return cls("gpt_neo", d["vocab_size"], H, L, d.get("num_heads", d.get("num_attention_heads")),
                       d.get("intermediate_size") or 4 * H, d.get("max_position_embeddings", 2048),
                       d.get("layer_norm_epsilon", 1e-5), act[d.get("activation_function", "gelu_new")],
                       tie_word_embeddings=d.get("tie_word_embeddings", True), attn_scale=1.0,
                       layer_windows=[win if k == "local" else 0 for k in kinds[:L]])
        if mt == "bloom":
            H = d.get("hidden_size", d.get("n_embed"))
            return cls("bloom", d["vocab_size"], H, d.get("n_layer", d.get("num_hidden_layers")),
                       d.get("n_head", d.get("num_attention_heads")), 4 * H, 1 << 20,
                       d.get("layer_norm_epsilon", 1e-5), "gelu_tanh",
                       tie_word_embeddings=d.get("tie_word_embeddings", True), alibi=True)
        if mt == "falcon":
            if d.get("alibi"):
                raise ValueError("Falcon checkpoints with ALiBi positions are not supported")
            H, nh = d["hidden_size"], d["num_attention_heads"]
            new = bool(d.get("new_decoder_architecture", False))
            par = bool(d.get("parallel_attn", True)) or new
            nkv = d.get("num_kv_heads") or nh if new else (1 if d.get("multi_query", True) else nh)
            n_ln = d.get("num_ln_in_parallel_attn") or (2 if new else 1)
            rp = d.get("rope_parameters") or {}
            return cls("falcon", d["vocab_size"], H, d["num_hidden_layers"], nh, d.get("ffn_hidden_size") or 4 * H,
                       d.get("max_position_embeddings", 2048), d.get("layer_norm_epsilon", 1e-5),
                       act[d.get("activation", "gelu")], float(d.get("rope_theta") or rp.get("rope_theta") or 10000.0),
                       1.0, par, tie_word_embeddings=d.get("tie_word_embeddings", True),
                       shared_norm=par and n_ln == 1, num_kv_heads=int(nkv))
        raise ValueError(f"unsupported model_type {mt!r}")


_ACT = {"gelu": "gelu", "gelu_tanh": "gelu_tanh", "relu": "relu"}


class GptModel:
    """Same call surface as LlamaModel (``forward(StepBatch, k_cache, v_cache)``, ``greedy_tokens``, ``Hq``,
    ``Hkv``, ``D``, ``n_layers``) so the engine, the scheduler and speculative decoding work unchanged."""

    tp_rank, tp_size, comm, fused = 0, 1, None, None

    def __init__(self, cfg: GptConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["embed"].device
        self.Hq, self.Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.D = cfg.head_dim
        self.n_layers = cfg.num_hidden_layers
        self.rope_dim = int(round(self.D * cfg.rotary_pct)) if cfg.rotary_pct > 0 else 0
        self.vocab_local, self.vocab_offset = weights["lm_head"].shape[0], 0
        self._zero_pos: Optional[torch.Tensor] = None
        self._alibi: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------------------------------------------
    @classmethod
    def from_state_dict(cls, cfg: GptConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "GptModel":
        H, nh, D = cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}
        if cfg.family == "gpt2":
            pre = "transformer." if any(k.startswith("transformer.") for k in sd) else ""
            w["embed"], w["pos"] = t(sd[pre + "wte.weight"]), t(sd[pre + "wpe.weight"])
            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}h.{l}.", f"l{l}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "ln_1.weight"]), t(sd[s + "ln_1.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "ln_2.weight"]), t(sd[s + "ln_2.bias"])
                # Conv1D stores [in, out]; the kernels want nn.Linear's [out, in]
                w[p + "qkv.w"], w[p + "qkv.b"] = t(sd[s + "attn.c_attn.weight"].t()), t(sd[s + "attn.c_attn.bias"])
                w[p + "o.w"], w[p + "o.b"] = t(sd[s + "attn.c_proj.weight"].t()), t(sd[s + "attn.c_proj.bias"])
                w[p + "fc.w"], w[p + "fc.b"] = t(sd[s + "mlp.c_fc.weight"].t()), t(sd[s + "mlp.c_fc.bias"])
                w[p + "proj.w"], w[p + "proj.b"] = t(sd[s + "mlp.c_proj.weight"].t()), t(sd[s + "mlp.c_proj.bias"])
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "ln_f.weight"]), t(sd[pre + "ln_f.bias"])
            w["lm_head"] = t(sd["lm_head.weight"]) if "lm_head.weight" in sd and not cfg.tie_word_embeddings else \
                w["embed"]
        elif cfg.family == "gpt_neox":
            pre = "gpt_neox." if any(k.startswith("gpt_neox.") for k in sd) else ""
            w["embed"] = t(sd[pre + "embed_in.weight"])
            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}layers.{l}.", f"l{l}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "input_layernorm.weight"]), t(sd[s + "input_layernorm.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "post_attention_layernorm.weight"]), t(
                    sd[s + "post_attention_layernorm.bias"])
                # rows are [head][q | k | v][D]; regroup to [q heads | k heads | v heads]
                qkv_w = sd[s + "attention.query_key_value.weight"].view(nh, 3, D, H).permute(1, 0, 2, 3).reshape(
                    3 * H, H)
                qkv_b = sd[s + "attention.query_key_value.bias"].view(nh, 3, D).permute(1, 0, 2).reshape(3 * H)
                w[p + "qkv.w"], w[p + "qkv.b"] = t(qkv_w), t(qkv_b)
                w[p + "o.w"], w[p + "o.b"] = t(sd[s + "attention.dense.weight"]), t(sd[s + "attention.dense.bias"])
                w[p + "fc.w"], w[p + "fc.b"] = t(sd[s + "mlp.dense_h_to_4h.weight"]), t(sd[s + "mlp.dense_h_to_4h.bias"])
                w[p + "proj.w"], w[p + "proj.b"] = t(sd[s + "mlp.dense_4h_to_h.weight"]), t(
                    sd[s + "mlp.dense_4h_to_h.bias"])
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "final_layer_norm.weight"]), t(sd[pre + "final_layer_norm.bias"])
            w["lm_head"] = t(sd["embed_out.weight"]) if "embed_out.weight" in sd else w["embed"]
        elif cfg.family == "opt":
            pre = "model.decoder." if any(k.startswith("model.decoder.") for k in sd) else "decoder."
            w["embed"], w["pos"] = t(sd[pre + "embed_tokens.weight"]), t(sd[pre + "embed_positions.weight"])
            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}layers.{l}.", f"l{l}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "self_attn_layer_norm.weight"]), t(
                    sd[s + "self_attn_layer_norm.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "final_layer_norm.weight"]), t(sd[s + "final_layer_norm.bias"])
                w[p + "qkv.w"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.weight"] for n in ("q", "k", "v")], 0))
                w[p + "qkv.b"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.bias"] for n in ("q", "k", "v")], 0))
                w[p + "o.w"], w[p + "o.b"] = t(sd[s + "self_attn.out_proj.weight"]), t(sd[s + "self_attn.out_proj.bias"])
                w[p + "fc.w"], w[p + "fc.b"] = t(sd[s + "fc1.weight"]), t(sd[s + "fc1.bias"])
                w[p + "proj.w"], w[p + "proj.b"] = t(sd[s + "fc2.weight"]), t(sd[s + "fc2.bias"])
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "final_layer_norm.weight"]), t(sd[pre + "final_layer_norm.bias"])
            w["lm_head"] = t(sd["lm_head.weight"]) if "lm_head.weight" in sd and not cfg.tie_word_embeddings else \
                w["embed"]
        elif cfg.family == "gptj":
            pre = "transformer." if any(k.startswith("transformer.") for k in sd) else ""
            w["embed"] = t(sd[pre + "wte.weight"])
            zeros = lambda n: torch.zeros(n, dtype=dtype, device=device)
            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}h.{l}.", f"l{l}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "ln_1.weight"]), t(sd[s + "ln_1.bias"])
                w[p + "qkv.w"] = t(torch.cat([sd[s + f"attn.{n}_proj.weight"] for n in ("q", "k", "v")], 0))
                w[p + "qkv.b"] = zeros(3 * H)
                w[p + "o.w"], w[p + "o.b"] = t(sd[s + "attn.out_proj.weight"]), zeros(H)
                w[p + "fc.w"], w[p + "fc.b"] = t(sd[s + "mlp.fc_in.weight"]), t(sd[s + "mlp.fc_in.bias"])
                w[p + "proj.w"], w[p + "proj.b"] = t(sd[s + "mlp.fc_out.weight"]), t(sd[s + "mlp.fc_out.bias"])
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "ln_f.weight"]), t(sd[pre + "ln_f.bias"])
            w["lm_head"], w["lm_head.b"] = t(sd["lm_head.weight"]), t(sd["lm_head.bias"])
        elif cfg.family == "phi":
            pre = "model." if any(k.startswith("model.") for k in sd) else ""
            w["embed"] = t(sd[pre + "embed_tokens.weight"])
            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}layers.{l}.", f"l{l}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "input_layernorm.weight"]), t(sd[s + "input_layernorm.bias"])
                w[p + "qkv.w"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.weight"] for n in ("q", "k", "v")], 0))
                w[p + "qkv.b"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.bias"] for n in ("q", "k", "v")], 0))
                w[p + "o.w"], w[p + "o.b"] = t(sd[s + "self_attn.dense.weight"]), t(sd[s + "self_attn.dense.bias"])
                w[p + "fc.w"], w[p + "fc.b"] = t(sd[s + "mlp.fc1.weight"]), t(sd[s + "mlp.fc1.bias"])
                w[p + "proj.w"], w[p + "proj.b"] = t(sd[s + "mlp.fc2.weight"]), t(sd[s + "mlp.fc2.bias"])
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "final_layernorm.weight"]), t(sd[pre + "final_layernorm.bias"])
            w["lm_head"], w["lm_head.b"] = t(sd["lm_head.weight"]), t(sd["lm_head.bias"])
        elif cfg.family == "bloom":
            pre = "transformer." if any(k.startswith("transformer.") for k in sd) else ""
            w["embed"] = t(sd[pre + "word_embeddings.weight"])
            w["embed.ln.g"] = t(sd[pre + "word_embeddings_layernorm.weight"])
            w["embed.ln.b"] = t(sd[pre + "word_embeddings_layernorm.bias"])
            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}h.{l}.", f"l{l}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "input_layernorm.weight"]), t(sd[s + "input_layernorm.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "post_attention_layernorm.weight"]), t(
                    sd[s + "post_attention_layernorm.bias"])
                a = s + "self_attention."
                # rows are [head][q | k | v][D], as in GPT-NeoX
                w[p + "qkv.w"] = t(sd[a + "query_key_value.weight"].view(nh, 3, D, H).permute(1, 0, 2, 3).reshape(
                    3 * H, H))
                w[p + "qkv.b"] = t(sd[a + "query_key_value.bias"].view(nh, 3, D).permute(1, 0, 2).reshape(3 * H))
                w[p + "o.w"], w[p + "o.b"] = t(sd[a + "dense.weight"]), t(sd[a + "dense.bias"])
                w[p + "fc.w"], w[p + "fc.b"] = t(sd[s + "mlp.dense_h_to_4h.weight"]), t(sd[s + "mlp.dense_h_to_4h.bias"])
                w[p + "proj.w"], w[p + "proj.b"] = t(sd[s + "mlp.dense_4h_to_h.weight"]), t(
                    sd[s + "mlp.dense_4h_to_h.bias"])
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "ln_f.weight"]), t(sd[pre + "ln_f.bias"])
            w["lm_head"] = t(sd["lm_head.weight"]) if "lm_head.weight" in sd and not cfg.tie_word_embeddings else \
                w["embed"]
        elif cfg.family == "gpt_neo":
            pre = "transformer." if any(k.startswith("transformer.") for k in sd) else ""
            w["embed"], w["pos"] = t(sd[pre + "wte.weight"]), t(sd[pre + "wpe.weight"])
            zeros = lambda n: torch.zeros(n, dtype=dtype, device=device)
            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}h.{l}.", f"l{l}."
                a = s + "attn.attention."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "ln_1.weight"]), t(sd[s + "ln_1.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "ln_2.weight"]), t(sd[s + "ln_2.bias"])
                w[p + "qkv.w"] = t(torch.cat([sd[a + f"{n}_proj.weight"] for n in ("q", "k", "v")], 0))
                w[p + "qkv.b"] = zeros(3 * H)
                w[p + "o.w"], w[p + "o.b"] = t(sd[a + "out_proj.weight"]), t(sd[a + "out_proj.bias"])
                w[p + "fc.w"], w[p + "fc.b"] = t(sd[s + "mlp.c_fc.weight"]), t(sd[s + "mlp.c_fc.bias"])
                w[p + "proj.w"], w[p + "proj.b"] = t(sd[s + "mlp.c_proj.weight"]), t(sd[s + "mlp.c_proj.bias"])
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "ln_f.weight"]), t(sd[pre + "ln_f.bias"])
            w["lm_head"] = t(sd["lm_head.weight"]) if "lm_head.weight" in sd and not cfg.tie_word_embeddings else \
                w["embed"]
        elif cfg.family == "falcon":
            pre = "transformer." if any(k.startswith("transformer.") for k in sd) else ""
            nkv = cfg.num_key_value_heads
            w["embed"] = t(sd[pre + "word_embeddings.weight"])
            zeros = lambda n: torch.zeros(n, dtype=dtype, device=device)

            def regroup(x: torch.Tensor) -> torch.Tensor:
                """Fused QKV rows (or bias entries) -> [q heads | k heads | v heads]."""
                tail = x.shape[1:]
                if grouped:      # per K / V head: its query heads, then k, then v
                    g = x.view(nkv, nh // nkv + 2, D, *tail)
                    return torch.cat([g[:, :-2].reshape(nh * D, *tail), g[:, -2].reshape(nkv * D, *tail),
                                      g[:, -1].reshape(nkv * D, *tail)], 0)
                if nkv == 1:     # multi-query: already [q heads | k | v]
                    return x
                g = x.view(nh, 3, D, *tail)   # per head: q, k, v
                return g.permute(1, 0, 2, *range(3, 3 + len(tail))).reshape(3 * nh * D, *tail)

            for l in range(cfg.num_hidden_layers):
                s, p = f"{pre}h.{l}.", f"l{l}."
                two_ln = s + "ln_attn.weight" in sd
                grouped = two_ln or (nkv not in (1, nh))
                if two_ln:
                    w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "ln_attn.weight"]), t(sd[s + "ln_attn.bias"])
                    w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "ln_mlp.weight"]), t(sd[s + "ln_mlp.bias"])
                else:
                    w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "input_layernorm.weight"]), t(sd[s + "input_layernorm.bias"])
                    if s + "post_attention_layernorm.weight" in sd:
                        w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "post_attention_layernorm.weight"]), t(
                            sd[s + "post_attention_layernorm.bias"])
                a = s + "self_attention."
                w[p + "qkv.w"] = t(regroup(sd[a + "query_key_value.weight"]))
                w[p + "qkv.b"] = t(regroup(sd[a + "query_key_value.bias"])) if a + "query_key_value.bias" in sd else \
                    zeros((nh + 2 * nkv) * D)
                w[p + "o.w"] = t(sd[a + "dense.weight"])
                w[p + "o.b"] = t(sd[a + "dense.bias"]) if a + "dense.bias" in sd else zeros(H)
                for ours, theirs, n in (("fc", "dense_h_to_4h", cfg.intermediate_size), ("proj", "dense_4h_to_h", H)):
                    w[p + ours + ".w"] = t(sd[s + f"mlp.{theirs}.weight"])
                    w[p + ours + ".b"] = t(sd[s + f"mlp.{theirs}.bias"]) if s + f"mlp.{theirs}.bias" in sd else zeros(n)
            w["lnf.g"], w["lnf.b"] = t(sd[pre + "ln_f.weight"]), t(sd[pre + "ln_f.bias"])
            w["lm_head"] = t(sd["lm_head.weight"]) if "lm_head.weight" in sd and not cfg.tie_word_embeddings else \
                w["embed"]
        else:
            raise ValueError(cfg.family)
        return cls(cfg, w)

    @classmethod
    def random_init(cls, cfg: GptConfig, device="cuda", seed: int = 0, dtype=torch.bfloat16) -> "GptModel":
        g = torch.Generator().manual_seed(seed)
        H, F = cfg.hidden_size, cfg.intermediate_size
        rnd = lambda *s, std=0.02: (torch.randn(*s, generator=g) * std).to(dtype).to(device)
        w: Dict[str, torch.Tensor] = {"embed": rnd(cfg.vocab_size, H)}
        if cfg.rotary_pct <= 0:
            w["pos"] = rnd(cfg.max_position_embeddings + cfg.position_offset, H)
        for l in range(cfg.num_hidden_layers):
            p = f"l{l}."
            for n in ("ln1", "ln2"):
                w[p + n + ".g"], w[p + n + ".b"] = torch.ones(H, dtype=dtype, device=device), rnd(H)
            nq = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
            w[p + "qkv.w"], w[p + "qkv.b"] = rnd(nq, H), rnd(nq)
            w[p + "o.w"], w[p + "o.b"] = rnd(H, H), rnd(H)
            w[p + "fc.w"], w[p + "fc.b"] = rnd(F, H), rnd(F)
            w[p + "proj.w"], w[p + "proj.b"] = rnd(H, F), rnd(H)
        w["lnf.g"], w["lnf.b"] = torch.ones(H, dtype=dtype, device=device), rnd(H)
        w["lm_head"] = w["embed"] if cfg.tie_word_embeddings else rnd(cfg.vocab_size, H)
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def forward(self, b: StepBatch, k_cache: torch.Tensor, v_cache: torch.Tensor,
                attn_scratch: Optional[A.PagedAttnScratch] = None) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        Hq, Hkv, D, eps = self.Hq, self.Hkv, self.D, cfg.layer_norm_eps
        scale = cfg.attn_scale or None
        T = b.ids.numel()
        act = _ACT[cfg.activation]
        x = Dn.embed_gather(b.ids, w["embed"])
        if "embed.ln.g" in w:
            x = Dn.norm(x, w["embed.ln.g"], w["embed.ln.b"], eps=eps, rms=False)
        if "pos" in w or cfg.alibi:
            if "pos" in w:
                x = x + w["pos"].index_select(0, (b.positions + cfg.position_offset).long())
            if self._zero_pos is None or self._zero_pos.numel() < T:
                self._zero_pos = torch.zeros(max(T, 1024), dtype=torch.int32, device=x.device)
            rope_pos, rope_dim = self._zero_pos[:T], D  # identity rotation: the kernel only writes K / V
        else:
            rope_pos, rope_dim = b.positions, self.rope_dim
        for l in range(self.n_layers):
            p = f"l{l}."
            h = Dn.norm(x, w[p + "ln1.g"], w[p + "ln1.b"], eps=eps, rms=False)
            qkv = Dn.gemm_bf16(h, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            q = A.rope_kv_write(qkv, rope_pos, b.slots, k_cache[l], v_cache[l], Hq, Hkv, D, cfg.rope_theta,
                                rope_dim=rope_dim, half_split=cfg.rope_half_split)
            window = cfg.layer_windows[l] if cfg.layer_windows else cfg.sliding_window
            if cfg.alibi:
                if self._alibi is None:
                    self._alibi = R.alibi_slopes(Hq).to(q.device)
                # the position bias changes the scores, so the kernel that carries per-score terms serves it
                ctx = A.paged_attention_sink(q, k_cache[l], v_cache[l], b.block_tables, b.q_starts, b.q_lens,
                                             b.kv_lens, scale=scale, window=window, alibi=self._alibi).to(q.dtype)
            else:
                ctx = A.paged_attention(q, k_cache[l], v_cache[l], b.block_tables, b.q_starts, b.q_lens, b.kv_lens,
                                        b.max_q_len, max_kv=b.max_kv, scale=scale, window=window, num_splits=b.attn_splits,
                                        scratch=attn_scratch)
            if cfg.parallel_residual:
                # x + attn(ln1 x) + mlp(ln2 x): both branches read the same x
                a_out = Dn.gemm_bf16(ctx.view(T, Hq * D), w[p + "o.w"], bias=w[p + "o.b"], residual=x)
                h2 = h if cfg.shared_norm else Dn.norm(x, w[p + "ln2.g"], w[p + "ln2.b"], eps=eps, rms=False)
                m = Dn.gemm_bf16(h2, w[p + "fc.w"], bias=w[p + "fc.b"], act=act)
                x = Dn.gemm_bf16(m, w[p + "proj.w"], bias=w[p + "proj.b"], residual=a_out)
            else:
                x = Dn.gemm_bf16(ctx.view(T, Hq * D), w[p + "o.w"], bias=w[p + "o.b"], residual=x)
                h2 = Dn.norm(x, w[p + "ln2.g"], w[p + "ln2.b"], eps=eps, rms=False)
                m = Dn.gemm_bf16(h2, w[p + "fc.w"], bias=w[p + "fc.b"], act=act)
                x = Dn.gemm_bf16(m, w[p + "proj.w"], bias=w[p + "proj.b"], residual=x)
        rows = x if b.logit_rows.numel() == T else x.index_select(0, b.logit_rows.long())
        hl = Dn.norm(rows, w["lnf.g"], w["lnf.b"], eps=eps, rms=False)
        return Dn.gemm_bf16(hl, w["lm_head"], bias=w.get("lm_head.b"))

    @property
    def graph_safe(self) -> bool:
        """Every step is a fixed launch sequence with no read-back to the host (the ALiBi family included: its
        position bias is applied inside the attention kernel), so decode buckets can be captured as CUDA graphs."""
        return True

    def greedy_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        return S.argmax(logits)

    def draft_view(self, n_layers: int) -> "GptModel":
        m = GptModel(self.cfg, self.w)
        m.n_layers = n_layers
        return m

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        for v in self.w.values():
            if v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                n += v.numel() * v.element_size()
        return n
