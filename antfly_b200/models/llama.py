"""Llama-family decoder (Llama / Mistral / Qwen2 / Qwen3 style: RMSNorm, GQA, RoPE, SwiGLU) over a paged KV cache.

What the layer computes follows the reference's decoderBlock (zig/pkg/inference/src/architectures/gpt.zig:3044:
norm -> QKV -> RoPE -> paged attention -> o_proj -> +residual -> norm -> SwiGLU FFN -> +residual) and its
Megatron sharding rules (zig/pkg/inference/src/graph/sharding.zig:74-82: q/k/v/gate/up split by output rows,
o/down split by input columns).  How it is executed is B200-first:

* weights are block-scaled fp8 (e4m3 + e8m0 per 32) streamed by the W8A16 tcgen05 GEMM; activations bf16;
* a step is one packed batch of tokens (decode tokens and prefill chunks mixed), one launch per op;
* skinny decode GEMMs run split-K and hand fp32 partial sums to the next kernel, which fuses the reduction with
  what it had to do anyway: residual add + RMSNorm, or RoPE + KV-cache write;
* SwiGLU is the epilogue of the fused gate/up GEMM (rows interleaved at load time);
* a decode step with a fixed batch is captured once in a CUDA graph and replayed.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import attention as A
from ..ops import dense as Dn
from ..ops.gguf_ops import DEVICE_TYPES as GGUF_DEVICE_TYPES, GgufWeight
from ..ops import quant as Q
from ..ops import sampling as S
from ..runtime.moe import CoactivationPredictor, ExpertResidency, HostExpertStore, route_batches


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    intermediate_size: int = 14336
    head_dim: int = 0
    rope_theta: float = 500000.0
    rope_dim: int = 0
    rope_half_split: bool = True
    rope_freq_scale: float = 1.0
    # frequency-dependent context extension (llama3, yarn, longrope): a table of rope_dim / 2 frequencies and the
    # factor that multiplies cos / sin; None: the closed-form frequencies
    rope_inv_freq: Optional[List[float]] = None
    rope_mscale: float = 1.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    qkv_bias: bool = False        # Qwen2
    qk_norm: bool = False         # Qwen3 per-head RMS norm on Q and K
    sliding_window: int = 0       # Mistral
    max_position_embeddings: int = 131072
    norm_plus_one: bool = False   # Gemma: RMSNorm scales by (1 + gamma)
    embed_scale: float = 1.0      # Gemma: token embeddings multiplied by sqrt(hidden)
    gate_act: str = "silu"        # gated-MLP activation: silu (SwiGLU), gelu_tanh (GeGLU, Gemma), relu2 (BitNet)
    # BitNet b1.58: ternary weights with one scale per matrix, activations rounded to 8 bits per token before
    # every projection, an extra RMS norm before the attention-output and the down projections
    mrope_sections: Optional[List[int]] = None   # Qwen2-VL: rotary pairs split between time / row / column streams
    # Gemma-3: a norm after attention and after the MLP as well as before them, a fixed softmax scale, and layers
    # that alternate between a sliding window with its own rotary base and global attention
    post_norms: bool = False
    attn_scale: float = 0.0                       # 0: 1 / sqrt(head_dim)
    layer_windows: Optional[List[int]] = None     # per layer: window length, 0 = global
    layer_rope: Optional[List[List[float]]] = None  # per layer: [theta, frequency scale]
    bitnet: bool = False
    bitnet_scale_divides: bool = False   # packed checkpoints of the "bitlinear" kind store 1 / scale
    # Mixture of experts (Mixtral, Qwen2-MoE, Qwen3-MoE): 0 experts = dense MLP
    num_experts: int = 0
    num_experts_per_tok: int = 2
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True   # renormalise the selected experts' weights to sum to one
    shared_expert_intermediate_size: int = 0
    # Gemma-2: scaled attention scores and final logits pass through cap * tanh(x / cap)
    attn_logit_softcapping: float = 0.0
    final_logit_softcapping: float = 0.0
    # a learned per-head sink logit in the attention softmax (checkpoints that carry ``self_attn.sinks``)
    attn_sinks: bool = False

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if not self.rope_dim:
            self.rope_dim = self.head_dim

    @classmethod
    def from_hf(cls, d: dict) -> "LlamaConfig":
        keys = {f for f in cls.__dataclass_fields__}
        cfg = cls(**{k: v for k, v in d.items() if k in keys and v is not None})
        # RoPE settings: top-level ``rope_theta`` (older config.json files) or the ``rope_parameters`` /
        # ``rope_scaling`` dictionary (newer ones); linear position scaling is a scalar, the frequency-dependent
        # schemes (llama3, yarn, longrope) become a frequency table once head_dim / rope_dim are settled below.
        rp = d.get("rope_parameters") or d.get("rope_scaling") or {}
        if d.get("rope_theta") is None and rp.get("rope_theta") is not None:
            cfg.rope_theta = float(rp["rope_theta"])
        if rp.get("rope_type", rp.get("type")) == "linear" and rp.get("factor"):
            cfg.rope_freq_scale = 1.0 / float(rp["factor"])
        prf = d.get("partial_rotary_factor") or rp.get("partial_rotary_factor")
        if prf:
            cfg.rope_dim = int(cfg.head_dim * float(prf))
        if d.get("use_sliding_window") is False:
            cfg.sliding_window = 0
        mt = d.get("model_type", "")
        if mt in ("qwen2", "qwen2_vl", "qwen2_vl_text"):
            cfg.qkv_bias = True
        if rp.get("mrope_section"):
            cfg.mrope_sections = [int(v) for v in rp["mrope_section"]]
        if mt == "qwen3":
            cfg.qk_norm = True
        if mt in ("mixtral", "qwen2_moe", "qwen3_moe"):
            cfg.num_experts = int(d.get("num_local_experts") or d.get("num_experts") or 0)
            cfg.num_experts_per_tok = int(d.get("num_experts_per_tok", 2))
            cfg.moe_intermediate_size = int(d.get("moe_intermediate_size") or d.get("intermediate_size"))
            cfg.norm_topk_prob = True if mt == "mixtral" else bool(d.get("norm_topk_prob", False))
            cfg.shared_expert_intermediate_size = int(d.get("shared_expert_intermediate_size") or 0) \
                if mt == "qwen2_moe" else 0
            if d.get("mlp_only_layers") or int(d.get("decoder_sparse_step", 1) or 1) != 1:
                raise ValueError("models that mix dense and sparse MLP layers are not supported")
            cfg.qkv_bias = mt == "qwen2_moe"
            cfg.qk_norm = mt == "qwen3_moe"
        if mt == "bitnet":
            cfg.bitnet = True
            cfg.gate_act = "relu2"
            cfg.tie_word_embeddings = d.get("tie_word_embeddings", True)
            cfg.bitnet_scale_divides = (d.get("quantization_config") or {}).get("linear_class") == "bitlinear"
        if mt in ("gemma3_text", "gemma3"):
            cfg.norm_plus_one, cfg.qk_norm, cfg.post_norms = True, True, True
            cfg.embed_scale = float(cfg.hidden_size) ** 0.5
            cfg.gate_act = "gelu_tanh"
            cfg.tie_word_embeddings = d.get("tie_word_embeddings", True)
            cfg.attn_scale = float(d.get("query_pre_attn_scalar") or cfg.head_dim) ** -0.5
            kinds = d.get("layer_types") or [
                "full_attention" if (i + 1) % int(d.get("sliding_window_pattern", 6) or 6) == 0 else "sliding_attention"
                for i in range(cfg.num_hidden_layers)]
            win = int(d.get("sliding_window") or 0)
            per = {k: v for k, v in rp.items() if isinstance(v, dict)}        # newer files: one entry per layer kind
            g_par, l_par = per.get("full_attention", rp), per.get("sliding_attention", {})
            g_theta = float(g_par.get("rope_theta") or d.get("rope_theta") or 1000000.0)
            g_scale = 1.0 / float(g_par["factor"]) if g_par.get("rope_type", g_par.get("type")) == "linear" and \
                g_par.get("factor") else 1.0
            l_theta = float(l_par.get("rope_theta") or d.get("rope_local_base_freq") or 10000.0)
            cfg.layer_windows = [win if k == "sliding_attention" else 0 for k in kinds]
            cfg.layer_rope = [[l_theta, 1.0] if k == "sliding_attention" else [g_theta, g_scale] for k in kinds]
            cfg.sliding_window, cfg.rope_theta, cfg.rope_freq_scale = 0, g_theta, g_scale
        if mt == "gemma2":
            cfg.norm_plus_one, cfg.post_norms = True, True
            cfg.embed_scale = float(cfg.hidden_size) ** 0.5
            cfg.gate_act = "gelu_tanh"
            cfg.tie_word_embeddings = d.get("tie_word_embeddings", True)
            cfg.attn_scale = float(d.get("query_pre_attn_scalar") or cfg.head_dim) ** -0.5
            cfg.attn_logit_softcapping = float(d.get("attn_logit_softcapping") or 0.0)
            cfg.final_logit_softcapping = float(d.get("final_logit_softcapping") or 0.0)
            kinds = d.get("layer_types") or ["sliding_attention" if i % 2 == 0 else "full_attention"
                                             for i in range(cfg.num_hidden_layers)]
            win = int(d.get("sliding_window") or 0)
            cfg.layer_windows = [win if k == "sliding_attention" else 0 for k in kinds]
            cfg.sliding_window = 0
        if mt == "gemma":
            cfg.norm_plus_one = True
            cfg.embed_scale = float(cfg.hidden_size) ** 0.5
            cfg.gate_act = "gelu_tanh"
            cfg.tie_word_embeddings = d.get("tie_word_embeddings", True)
        if not cfg.layer_rope and not cfg.mrope_sections:
            from .rope_scaling import rope_frequencies

            rope = dict(rp)
            if "original_max_position_embeddings" not in rope and d.get("original_max_position_embeddings"):
                rope["original_max_position_embeddings"] = d["original_max_position_embeddings"]   # Phi-3 long
            cfg.rope_inv_freq, cfg.rope_mscale = rope_frequencies(
                rope, cfg.rope_theta, cfg.rope_dim or cfg.head_dim, int(d.get("max_position_embeddings") or 0))
        return cfg

    @classmethod
    def llama3_8b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def llama3_70b(cls) -> "LlamaConfig":
        return cls(hidden_size=8192, num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                   intermediate_size=28672)

    @classmethod
    def tiny(cls, **kw) -> "LlamaConfig":
        base = dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, intermediate_size=512, head_dim=64, rope_theta=10000.0)
        base.update(kw)
        return cls(**base)


@dataclass
class StepBatch:
    """One forward pass worth of packed tokens (all int32 tensors on the model's device)."""
    ids: torch.Tensor           # [T]
    positions: torch.Tensor     # [T]
    slots: torch.Tensor         # [T] KV-cache slot of each token
    q_starts: torch.Tensor      # [B]
    q_lens: torch.Tensor        # [B]
    kv_lens: torch.Tensor       # [B] sequence length including this step's tokens
    block_tables: torch.Tensor  # [B, max_blocks]
    logit_rows: torch.Tensor    # [R] token rows whose logits are wanted
    max_q_len: int = 1
    attn_splits: int = 1
    max_kv: int = 0             # largest kv_lens entry when the host knows it (0: unknown); bounds page expansion
    # multimodal prompts: rows of this step whose embedding is a given vector instead of a table row, and three
    # rotary position streams [3, T] (time / row / column) in place of ``positions``
    embed_rows: Optional[torch.Tensor] = None
    embed_vals: Optional[torch.Tensor] = None
    pos3: Optional[torch.Tensor] = None
    # runs of rows (image tokens) that attend to one another in both directions: (q_starts, q_lens, kv_lens,
    # block_tables, longest run, row indices), each run described like a sequence of its own whose keys end where
    # the run ends
    bidir: Optional[tuple] = None


def pick_split_k(n_out: int, k_in: int, m_tokens: int, sm_count: int = 148) -> int:
    """Split K so a skinny GEMM still puts about one CTA on every SM."""
    bt = 16 if m_tokens <= 16 else 32 if m_tokens <= 32 else 64 if m_tokens <= 64 else 128 if m_tokens <= 128 else 256
    tiles = ((n_out + 127) // 128) * ((m_tokens + bt - 1) // bt)
    if tiles >= sm_count:
        return 1
    num_kb = (k_in + 127) // 128
    # Aim for about one CTA per SM, keep at least 4 K-chunks per CTA and at most 8 partial slices for the
    # consumer to sum (every slice is read back by the kernel that follows).
    s = max(1, min((sm_count + tiles - 1) // tiles, num_kb // 4, 8))
    return s


@dataclass
class MoeRuntimeState:
    store: HostExpertStore
    residency: ExpertResidency
    predictor: CoactivationPredictor
    max_predicted: int = 2


def bitnet_ternary(weight: torch.Tensor, weight_scale: Optional[torch.Tensor], scale_divides: bool):
    """One BitNet projection -> (ternary matrix with entries -1 / 0 / +1 as fp32, the scalar that multiplies it).

    Full-precision weights are ternarised on load (``round(w / mean|w|)`` clipped to [-1, 1], scalar ``mean|w|``).
    Packed checkpoints hold four 2-bit codes per byte -- byte row ``r`` carries output rows ``r``, ``r + R``,
    ``r + 2R``, ``r + 3R`` (``R`` = packed rows) in bits 0-1, 2-3, 4-5, 6-7, each code being the value plus one --
    and the scalar beside them."""
    if weight.dtype == torch.uint8:
        R_ = weight.shape[0]
        t = torch.cat([((weight >> (2 * i)) & 3) for i in range(4)], 0).float() - 1.0
        assert t.shape[0] == 4 * R_
        sc = float(weight_scale.float().flatten()[0]) if weight_scale is not None else 1.0
        return t, (1.0 / sc if scale_divides else sc)
    wf = weight.float()
    top = float(wf.abs().max())
    if top > 0 and bool(((wf.abs() == top) | (wf == 0)).all()):
        return torch.sign(wf), top           # already ternary times one scalar (decoded from a 2-bit file format)
    m = float(wf.abs().mean().clamp(min=1e-5))
    return (wf / m).round().clamp(-1, 1), m


class LlamaModel:
    def __init__(self, cfg: LlamaConfig, weights: Dict[str, object], tp_rank: int = 0, tp_size: int = 1,
                 comm=None):
        self.cfg, self.w = cfg, weights
        self.tp_rank, self.tp_size, self.comm = tp_rank, tp_size, comm
        self.device = weights["embed"].device
        self.Hq = cfg.num_attention_heads // tp_size
        self.Hkv = max(cfg.num_key_value_heads // tp_size, 1)
        self.D = cfg.head_dim
        self.n_layers = cfg.num_hidden_layers
        self.vocab_local = weights["lm_head"].out_features \
            if isinstance(weights["lm_head"], (Q.Fp8Weight, GgufWeight)) else weights["lm_head"].shape[0]
        self.vocab_offset = tp_rank * self.vocab_local if tp_size > 1 else 0
        self._scratch: Dict[tuple, torch.Tensor] = {}
        self.moe_runtime = None   # set by offload_experts(): expert weights live in host memory
        self.ep = None            # set by set_expert_parallel(): (rank, size, process group)
        self.pp = None            # set by set_pipeline(): this model is one stage of a layer pipeline
        self.layer_lo = 0
        # rotary frequency table of a context-extension scheme, on the model's device (None: closed form)
        self.rope_table = torch.tensor(cfg.rope_inv_freq, dtype=torch.float32, device=self.device) \
            if cfg.rope_inv_freq else None

    # --------------------------------------------------------------------------------------------------
    @classmethod
    def random_init(cls, cfg: LlamaConfig, device="cuda", seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                    comm=None, fast_init: Optional[bool] = None, n_layers: Optional[int] = None) -> "LlamaModel":
        """Random block-fp8 weights of this rank's shard.  ``fast_init`` draws directly in the quantised domain
        (no fp32 master), which is what the full-size benchmark models use; small test models quantise real
        Gaussian weights so the fp32 oracle has something to compare with."""
        H, F, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        Hq, Hkv = cfg.num_attention_heads // tp_size, max(cfg.num_key_value_heads // tp_size, 1)
        if fast_init is None:
            fast_init = H >= 2048
        L = n_layers or cfg.num_hidden_layers
        g = torch.Generator().manual_seed(seed)
        dev = device

        def dense(n, k, s):
            return (torch.randn(n, k, generator=g) * (k ** -0.5)).to(torch.bfloat16)

        def fp8(n, k, s, swiglu=False):
            if fast_init:
                return Q.random_fp8(n, k, dev, seed=s, interleaved_swiglu=swiglu)
            w = dense(n, k, s).to(dev)
            p = Q.pack_fp8(w)
            p.interleaved_swiglu = swiglu
            return p

        w: Dict[str, object] = {}
        V = cfg.vocab_size
        if fast_init:
            ge = torch.Generator(device=dev).manual_seed(seed + 1)
            w["embed"] = (torch.randn(V, H, generator=ge, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        else:
            w["embed"] = (torch.randn(V, H, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=dev)
        for l in range(L):
            p = f"l{l}."
            s0 = seed * 1000003 + l * 16 + tp_rank * 7919
            w[p + "ln1"], w[p + "ln2"] = ones(H), ones(H)
            w[p + "qkv"] = fp8((Hq + 2 * Hkv) * D, H, s0 + 1)
            if cfg.qkv_bias:
                w[p + "qkv.b"] = (torch.randn((Hq + 2 * Hkv) * D, generator=g) * 0.02).to(torch.bfloat16).to(dev)
            if cfg.qk_norm:
                w[p + "qn"], w[p + "kn"] = ones(D), ones(D)
            w[p + "o"] = fp8(H, Hq * D, s0 + 2)
            w[p + "gu"] = fp8(2 * (F // tp_size), H, s0 + 3, swiglu=True)
            w[p + "down"] = fp8(H, F // tp_size, s0 + 4)
        w["norm"] = ones(H)
        vl = V // tp_size if tp_size > 1 else V
        if cfg.tie_word_embeddings and tp_size == 1:
            w["lm_head"] = Q.pack_fp8(w["embed"]) if not fast_init else fp8(vl, H, seed + 99)
        else:
            w["lm_head"] = fp8(vl, H, seed + 99 + tp_rank)
        m = cls(cfg, w, tp_rank, tp_size, comm)
        m.n_layers = L
        return m

    @classmethod
    def from_state_dict(cls, cfg: LlamaConfig, sd: Dict[str, torch.Tensor], device="cuda", tp_rank: int = 0,
                        tp_size: int = 1, comm=None, layers: Optional[tuple] = None,
                        experts: Optional[tuple] = None) -> "LlamaModel":
        """HF names (model.layers.N.self_attn.{q,k,v,o}_proj, mlp.{gate,up,down}_proj, ...) -> fused, sharded,
        block-fp8 packed layout.  ``layers`` = (first, last) loads only that range of decoder layers (a pipeline
        stage); the stage is then wired with :meth:`set_pipeline`.  ``experts`` = (rank, size) loads only the routed
        experts ``e`` with ``e % size == rank`` (expert parallelism, wired with :meth:`set_expert_parallel`)."""
        from ..parallel.sharding import shard_rows, shard_cols

        D = cfg.head_dim
        pre = "model." if any(k.startswith("model.") for k in sd) else ""
        w: Dict[str, object] = {}
        emb = sd[pre + "embed_tokens.weight"].to(torch.bfloat16)
        w["embed"] = emb.to(device)
        for l in range(*(layers or (0, cfg.num_hidden_layers))):
            s, p = f"{pre}layers.{l}.", f"l{l}."
            if cfg.bitnet:
                assert tp_size == 1, "BitNet models run on one GPU"
                sd = dict(sd)
                ws = {}
                for name in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                             "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"):
                    sd[s + name + ".weight"], ws[name] = bitnet_ternary(
                        sd[s + name + ".weight"], sd.get(s + name + ".weight_scale"), cfg.bitnet_scale_divides)
                rows = lambda name: torch.full((sd[s + name + ".weight"].shape[0],), ws[name])
                w[p + "qkv.ws"] = torch.cat([rows("self_attn." + n + "_proj") for n in "qkv"]).to(device)
                w[p + "o.ws"] = rows("self_attn.o_proj").to(device)
                w[p + "gu.ws"] = torch.stack([rows("mlp.gate_proj"), rows("mlp.up_proj")], 1).flatten().to(device)
                w[p + "down.ws"] = rows("mlp.down_proj").to(device)
                w[p + "attn_sub"] = sd[s + "self_attn.attn_sub_norm.weight"].to(torch.bfloat16).to(device)
                w[p + "ffn_sub"] = sd[s + "mlp.ffn_sub_norm.weight"].to(torch.bfloat16).to(device)
            w[p + "ln1"] = sd[s + "input_layernorm.weight"].to(torch.bfloat16).to(device)
            if cfg.post_norms:     # four norms per layer; "post_attention" here is the one on the attention output
                w[p + "ln2"] = sd[s + "pre_feedforward_layernorm.weight"].to(torch.bfloat16).to(device)
                w[p + "post_attn"] = sd[s + "post_attention_layernorm.weight"].to(torch.bfloat16).to(device)
                w[p + "post_ffn"] = sd[s + "post_feedforward_layernorm.weight"].to(torch.bfloat16).to(device)
            else:
                w[p + "ln2"] = sd[s + "post_attention_layernorm.weight"].to(torch.bfloat16).to(device)
            if s + "self_attn.qkv_proj.weight" in sd:  # Phi-3: fused [q | k | v] rows
                nq, nk = cfg.num_attention_heads * D, cfg.num_key_value_heads * D
                fused = sd[s + "self_attn.qkv_proj.weight"]
                sd[s + "self_attn.q_proj.weight"], sd[s + "self_attn.k_proj.weight"] = fused[:nq], fused[nq:nq + nk]
                sd[s + "self_attn.v_proj.weight"] = fused[nq + nk:]
            if s + "mlp.gate_up_proj.weight" in sd:    # Phi-3: fused [gate ; up] rows
                gu_f = sd[s + "mlp.gate_up_proj.weight"]
                sd[s + "mlp.gate_proj.weight"], sd[s + "mlp.up_proj.weight"] = gu_f[: gu_f.shape[0] // 2], gu_f[
                    gu_f.shape[0] // 2:]
            q = shard_rows(sd[s + "self_attn.q_proj.weight"], tp_rank, tp_size)
            k = shard_rows(sd[s + "self_attn.k_proj.weight"], tp_rank, tp_size)
            v = shard_rows(sd[s + "self_attn.v_proj.weight"], tp_rank, tp_size)
            w[p + "qkv"] = Q.pack_fp8(torch.cat([q, k, v], 0).to(device))
            if s + "self_attn.q_proj.bias" in sd:
                w[p + "qkv.b"] = torch.cat([shard_rows(sd[s + f"self_attn.{n}_proj.bias"], tp_rank, tp_size)
                                            for n in ("q", "k", "v")]).to(torch.bfloat16).to(device)
            if s + "self_attn.q_norm.weight" in sd:
                w[p + "qn"] = sd[s + "self_attn.q_norm.weight"].to(torch.bfloat16).to(device)
                w[p + "kn"] = sd[s + "self_attn.k_norm.weight"].to(torch.bfloat16).to(device)
            w[p + "o"] = Q.pack_fp8(shard_cols(sd[s + "self_attn.o_proj.weight"], tp_rank, tp_size).to(device))
            if s + "self_attn.sinks" in sd:                     # one sink logit per query head (this rank's heads)
                cfg.attn_sinks = True
                w[p + "sinks"] = shard_rows(sd[s + "self_attn.sinks"].float().reshape(-1, 1), tp_rank,
                                            tp_size).flatten().to(device)
            if cfg.num_experts > 0:
                assert tp_size == 1, "mixture-of-experts models run on one GPU"
                moe = s + ("block_sparse_moe." if s + "block_sparse_moe.gate.weight" in sd else "mlp.")
                w[p + "router"] = sd[moe + "gate.weight"].to(torch.bfloat16).to(device)
                Fm = cfg.moe_intermediate_size
                for e in range(cfg.num_experts):
                    if experts is not None and e % experts[1] != experts[0]:
                        continue
                    if moe + "experts.gate_up_proj" in sd:      # fused [E, 2F, H] (gate rows, then up rows) / [E, H, F]
                        gu = sd[moe + "experts.gate_up_proj"][e]
                        g_e, u_e, d_e = gu[:Fm], gu[Fm:], sd[moe + "experts.down_proj"][e]
                    elif moe + f"experts.{e}.w1.weight" in sd:  # Mixtral checkpoints: w1 gate, w3 up, w2 down
                        g_e, u_e = sd[moe + f"experts.{e}.w1.weight"], sd[moe + f"experts.{e}.w3.weight"]
                        d_e = sd[moe + f"experts.{e}.w2.weight"]
                    else:
                        g_e, u_e = sd[moe + f"experts.{e}.gate_proj.weight"], sd[moe + f"experts.{e}.up_proj.weight"]
                        d_e = sd[moe + f"experts.{e}.down_proj.weight"]
                    w[p + f"e{e}.gu"] = Q.pack_fp8_swiglu(g_e.to(device), u_e.to(device))
                    w[p + f"e{e}.down"] = Q.pack_fp8(d_e.to(device))
                if cfg.shared_expert_intermediate_size:
                    w[p + "shared.gu"] = Q.pack_fp8_swiglu(sd[moe + "shared_expert.gate_proj.weight"].to(device),
                                                           sd[moe + "shared_expert.up_proj.weight"].to(device))
                    w[p + "shared.down"] = Q.pack_fp8(sd[moe + "shared_expert.down_proj.weight"].to(device))
                    w[p + "shared.gate"] = sd[moe + "shared_expert_gate.weight"].to(torch.bfloat16).to(device)
                continue
            gate = shard_rows(sd[s + "mlp.gate_proj.weight"], tp_rank, tp_size).to(device)
            up = shard_rows(sd[s + "mlp.up_proj.weight"], tp_rank, tp_size).to(device)
            w[p + "gu"] = Q.pack_fp8_swiglu(gate, up)
            w[p + "down"] = Q.pack_fp8(shard_cols(sd[s + "mlp.down_proj.weight"], tp_rank, tp_size).to(device))
        w["norm"] = sd[pre + "norm.weight"].to(torch.bfloat16).to(device)
        head = emb if cfg.tie_word_embeddings else sd.get("lm_head.weight", emb)
        w["lm_head"] = Q.pack_fp8(shard_rows(head, tp_rank, tp_size).to(device) if tp_size > 1 else head.to(device))
        return cls(cfg, w, tp_rank, tp_size, comm)

    def draft_view(self, n_layers: int) -> "LlamaModel":
        """A shallower model that shares this model's first ``n_layers`` layers, embedding, final norm and LM
        head (self-speculative draft).  It needs its own KV cache of n_layers layers."""
        m = LlamaModel(self.cfg, self.w, self.tp_rank, self.tp_size, self.comm)
        m.n_layers = n_layers
        m.fused = self.fused
        return m

    def weight_bytes(self) -> int:
        n = 0
        for l in range(self.n_layers):
            for nm in ("qkv", "o", "gu", "down"):
                n += self.w[f"l{l}.{nm}"].nbytes()
        n += self.w["lm_head"].nbytes() if isinstance(self.w["lm_head"], Q.Fp8Weight) else 0
        return n

    # --------------------------------------------------------------------------------------------------
    # Skinny batches (decode, speculative verify) take the native MX path: activations are quantised to MX fp8
    # (two terms ~ bf16 accuracy) and the tensor core applies both block scales; large prefill batches keep
    # bf16 activations and dequantise the weights in the GEMM (W8A16).  The MX kernel tiles any number of tokens
    # (128 per CTA), so the boundary is a tuning knob: ANTFLY_B200_MX_MAX_TOKENS moves it (e.g. to route prefill
    # chunks through the block-scaled tensor-core path as well).
    mx_max_tokens: int = int(os.environ.get("ANTFLY_B200_MX_MAX_TOKENS", "128"))
    act_terms: int = 2

    def _use_mx(self, T: int) -> bool:
        c = self.cfg
        return (T <= self.mx_max_tokens and self.act_terms > 0 and c.hidden_size % 128 == 0
                and (c.intermediate_size // self.tp_size) % 128 == 0 and (self.Hq * self.D) % 128 == 0)

    @classmethod
    def from_gguf_native(cls, cfg: LlamaConfig, gguf_file, device="cuda") -> "LlamaModel":
        """A dense Llama-family GGUF checkpoint served from its own block formats: every projection stored as Q8_0,
        Q4_0, MXFP4, Q4_K, Q5_K or Q6_K stays in those bytes on the device (a fused projection keeps one segment per
        part, so mixed-format files work) and is expanded inside the kernels; other tensors (norms, embeddings,
        F16 / F32 projections) load as usual.  Decode batches then move 4.25 - 8.5 bits per weight instead of the
        re-packed 8.25.  The counterpart of the reference running GGUF tensors directly through its quantised
        matmuls (zig/pkg/inference/src/graph/quant_matmul.zig:17-60)."""
        from ..formats import gguf as GG

        if cfg.num_experts > 0 or cfg.bitnet:
            raise NotImplementedError("native GGUF serving covers dense, non-ternary decoders")
        f = gguf_file
        names = {GG.hf_name(n): n for n in f.tensors}

        def native(hf: str):
            info = f.tensors[names[hf]]
            return info.type in GGUF_DEVICE_TYPES and len(info.shape) == 2 and info.shape[1] % 32 == 0

        def seg(hf: str):
            info = f.tensors[names[hf]]
            return torch.from_numpy(f.raw(names[hf]).copy()).to(device), info.type, int(info.shape[0])

        def weight(parts, interleave=False):
            """GgufWeight when every part is in a device format, else a re-packed fp8 weight of the parts."""
            K = int(f.tensors[names[parts[0]]].shape[1])
            if all(native(h) for h in parts):
                return GgufWeight([seg(h) for h in parts], K, interleave)
            mats = [f.tensor(names[h]).to(torch.bfloat16) for h in parts]
            if interleave:
                return Q.pack_fp8(torch.stack(mats, 1).reshape(-1, K).to(device))
            return Q.pack_fp8(torch.cat(mats, 0).to(device))

        w: Dict[str, object] = {}
        emb = f.tensor(names["model.embed_tokens.weight"]).to(torch.bfloat16)
        w["embed"] = emb.to(device)
        for l in range(cfg.num_hidden_layers):
            s_, p = f"model.layers.{l}.", f"l{l}."
            w[p + "ln1"] = f.tensor(names[s_ + "input_layernorm.weight"]).to(torch.bfloat16).to(device)
            w[p + "ln2"] = f.tensor(names[s_ + "post_attention_layernorm.weight"]).to(torch.bfloat16).to(device)
            w[p + "qkv"] = weight([s_ + f"self_attn.{n}_proj.weight" for n in "qkv"])
            if s_ + "self_attn.q_proj.bias" in names:
                w[p + "qkv.b"] = torch.cat([f.tensor(names[s_ + f"self_attn.{n}_proj.bias"]) for n in "qkv"]).to(
                    torch.bfloat16).to(device)
            if cfg.qk_norm:
                w[p + "qn"] = f.tensor(names[s_ + "self_attn.q_norm.weight"]).to(torch.bfloat16).to(device)
                w[p + "kn"] = f.tensor(names[s_ + "self_attn.k_norm.weight"]).to(torch.bfloat16).to(device)
            w[p + "o"] = weight([s_ + "self_attn.o_proj.weight"])
            w[p + "gu"] = weight([s_ + "mlp.gate_proj.weight", s_ + "mlp.up_proj.weight"], interleave=True)
            w[p + "down"] = weight([s_ + "mlp.down_proj.weight"])
        w["norm"] = f.tensor(names["model.norm.weight"]).to(torch.bfloat16).to(device)
        if "lm_head.weight" in names and not cfg.tie_word_embeddings:
            w["lm_head"] = weight(["lm_head.weight"])
        else:
            w["lm_head"] = w["embed"]
        m = cls(cfg, w)
        m.native_gguf = True
        return m

    def _linear(self, h, w: "Q.Fp8Weight", T: int, **kw) -> torch.Tensor:
        """h is bf16 [T, K] or already-quantised MX activations."""
        if isinstance(w, GgufWeight):               # weights served from their GGUF block bytes
            y = w(h)
            res = kw.get("residual")
            return (y.float() + res.float()).to(torch.bfloat16) if res is not None else y
        if isinstance(h, Q.MxAct):
            return Q.gemm_mxfp8(h, w, **kw)
        if self._use_mx(T) and h.shape[1] % 128 == 0:
            return Q.gemm_mxfp8(Q.quantize_mx(h, terms=self.act_terms), w, **kw)
        return Q.gemm_w8a16(h, w, **kw)

    def _reduce(self, parts: torch.Tensor) -> torch.Tensor:
        """Tensor-parallel sum of row-parallel partial outputs (baseline path: NCCL all-reduce)."""
        if self.tp_size == 1 or self.comm is None:
            return parts
        y = parts.sum(0, keepdim=True) if parts.shape[0] > 1 else parts
        self.comm.all_reduce(y)
        return y

    fused = None  # antfly_b200.parallel.fused.FusedTp when the peer-memory path is enabled
    native_gguf = False  # True: projections are GgufWeight objects (quantised bytes expanded inside the kernels)
    return_hidden = False  # True: forward returns the final-norm hidden states of the wanted rows, not logits

    @property
    def graph_safe(self) -> bool:
        """False when a step's launch sequence depends on the data (expert routing): no CUDA-graph capture."""
        return self.cfg.num_experts == 0

    def _forward_fused(self, b: StepBatch, k_cache, v_cache, attn_scratch) -> torch.Tensor:
        """Tensor-parallel step with the collectives fused into the GEMM and norm kernels (skinny batches)."""
        cfg, w, fz = self.cfg, self.w, self.fused
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        T = b.ids.numel()
        tl = fz.tokens_per_rank(T)
        x_full = Dn.embed_gather(b.ids, w["embed"])
        h = Dn.norm(x_full, w["l0.ln1"], eps=cfg.rms_norm_eps, rms=True, mx_terms=self.act_terms)
        x = x_full[self.tp_rank * tl:(self.tp_rank + 1) * tl].contiguous()
        for l in range(self.n_layers):
            p = f"l{l}."
            qkv_w: Q.Fp8Weight = w[p + "qkv"]
            sk = pick_split_k(qkv_w.out_features, qkv_w.in_features, T)
            if l == 0:
                parts = Q.gemm_mxfp8(h, qkv_w, partials=True, split_k=sk)
            else:
                parts = fz.gemm_gathered(qkv_w, T, split_k=sk, partials=True)
            q = A.rope_kv_write(None, b.positions, b.slots, k_cache[l], v_cache[l], Hq, Hkv, D, cfg.rope_theta,
                                partials=parts, bias=w.get(p + "qkv.b"), rope_dim=cfg.rope_dim,
                                half_split=cfg.rope_half_split, freq_scale=cfg.rope_freq_scale,
                                q_norm_w=w.get(p + "qn"), k_norm_w=w.get(p + "kn"), norm_eps=cfg.rms_norm_eps,
                                inv_freq=self.rope_table, rope_mscale=cfg.rope_mscale)
            ctx = A.paged_attention(q, k_cache[l], v_cache[l], b.block_tables, b.q_starts, b.q_lens, b.kv_lens,
                                    b.max_q_len, max_kv=b.max_kv, window=cfg.sliding_window, num_splits=b.attn_splits,
                                    scratch=attn_scratch, mx_terms=self.act_terms)
            o_w: Q.Fp8Weight = w[p + "o"]
            S = fz.gemm_push(ctx, o_w, T, pick_split_k(o_w.out_features, o_w.in_features, T))
            x = fz.norm_reduce_gather(w[p + "ln2"], x, T, S, o_w.out_features, cfg.rms_norm_eps)
            gu_w: Q.Fp8Weight = w[p + "gu"]
            sk = pick_split_k(gu_w.out_features, gu_w.in_features, T)
            if sk > 1:
                act = Q.swiglu_quantize_mx(fz.gemm_gathered(gu_w, T, split_k=sk, partials=True),
                                           terms=self.act_terms)
            else:
                act = Q.quantize_mx(fz.gemm_gathered(gu_w, T, swiglu=True), terms=self.act_terms)
            d_w: Q.Fp8Weight = w[p + "down"]
            S = fz.gemm_push(act, d_w, T, pick_split_k(d_w.out_features, d_w.in_features, T))
            nw = w["norm"] if l + 1 == self.n_layers else w[f"l{l + 1}.ln1"]
            x = fz.norm_reduce_gather(nw, x, T, S, d_w.out_features, cfg.rms_norm_eps)
        return fz.gemm_gathered(w["lm_head"], T)

    def _forward_one_shot(self, b: StepBatch, k_cache, v_cache, attn_scratch) -> torch.Tensor:
        """Tensor-parallel step whose two collectives per layer are one-shot all-reduces fused into the
        row-parallel GEMMs (push) and the norms (wait + sum): one NVLink hop each, replicated residual stream."""
        cfg, w, fz = self.cfg, self.w, self.fused
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        T = b.ids.numel()
        mxt = self.act_terms
        x = Dn.embed_gather(b.ids, w["embed"])
        h = Dn.norm(x, w["l0.ln1"], eps=cfg.rms_norm_eps, rms=True, mx_terms=mxt)
        for l in range(self.n_layers):
            p = f"l{l}."
            qkv_w: Q.Fp8Weight = w[p + "qkv"]
            parts = Q.gemm_mxfp8(h, qkv_w, partials=True,
                                 split_k=pick_split_k(qkv_w.out_features, qkv_w.in_features, T))
            q = A.rope_kv_write(None, b.positions, b.slots, k_cache[l], v_cache[l], Hq, Hkv, D, cfg.rope_theta,
                                partials=parts, bias=w.get(p + "qkv.b"), rope_dim=cfg.rope_dim,
                                half_split=cfg.rope_half_split, freq_scale=cfg.rope_freq_scale,
                                q_norm_w=w.get(p + "qn"), k_norm_w=w.get(p + "kn"), norm_eps=cfg.rms_norm_eps,
                                inv_freq=self.rope_table, rope_mscale=cfg.rope_mscale)
            ctx = A.paged_attention(q, k_cache[l], v_cache[l], b.block_tables, b.q_starts, b.q_lens, b.kv_lens,
                                    b.max_q_len, max_kv=b.max_kv, window=cfg.sliding_window, num_splits=b.attn_splits,
                                    scratch=attn_scratch, mx_terms=mxt)
            o_w: Q.Fp8Weight = w[p + "o"]
            fz.gemm_bcast(ctx, o_w, T, pick_split_k(o_w.out_features, o_w.in_features, T), 0)
            x, h = fz.norm_bcast(w[p + "ln2"], x, T, cfg.rms_norm_eps, 0)
            gu_w: Q.Fp8Weight = w[p + "gu"]
            sk = pick_split_k(gu_w.out_features, gu_w.in_features, T)
            if sk > 1:
                act = Q.swiglu_quantize_mx(Q.gemm_mxfp8(h, gu_w, partials=True, split_k=sk), terms=mxt)
            else:
                act = Q.quantize_mx(Q.gemm_mxfp8(h, gu_w, swiglu=True), terms=mxt)
            d_w: Q.Fp8Weight = w[p + "down"]
            fz.gemm_bcast(act, d_w, T, pick_split_k(d_w.out_features, d_w.in_features, T), 1)
            nw = w["norm"] if l + 1 == self.n_layers else w[f"l{l + 1}.ln1"]
            x, h = fz.norm_bcast(nw, x, T, cfg.rms_norm_eps, 1)
        return Q.gemm_mxfp8(h, w["lm_head"])

    # -- compiled artifacts: the in-memory layout (fused, interleaved, block-fp8 packed) saved as it is ------------
    ARTIFACT_FORMAT = "antfly_b200.llama.packed.v1"

    def save_artifact(self, path: str) -> None:
        """Write this model's weights exactly as the kernels consume them (fused QKV, interleaved gate / up, block
        fp8 codes + scales) so that a later start only reads and uploads: no fusing, no re-quantising.  The
        reference's counterpart is its compiled artifact (zig/pkg/inference/src/compiled_artifact.zig,
        native_run_artifact.zig)."""
        import dataclasses
        import json

        from ..formats import safetensors_io as ST

        tensors, swiglu = {}, []
        for name, v in self.w.items():
            if isinstance(v, Q.Fp8Weight):
                tensors[name + "::q"] = v.q.view(torch.uint8) if v.q.dtype != torch.uint8 else v.q
                tensors[name + "::scales"] = v.scales
                if v.interleaved_swiglu:
                    swiglu.append(name)
            elif isinstance(v, torch.Tensor):
                if not (name == "lm_head" and v.data_ptr() == self.w["embed"].data_ptr()):
                    tensors[name] = v
        ST.save_file(tensors, path, {"format": self.ARTIFACT_FORMAT, "config": json.dumps(dataclasses.asdict(self.cfg)),
                                     "swiglu": json.dumps(swiglu), "tp_rank": self.tp_rank, "tp_size": self.tp_size})

    @classmethod
    def from_artifact(cls, path: str, device="cuda", comm=None) -> "LlamaModel":
        import json

        from ..formats import safetensors_io as ST

        meta = ST.read_metadata(path)
        if meta.get("format") != cls.ARTIFACT_FORMAT:
            raise ValueError(f"{path}: not a packed model artifact (format {meta.get('format')!r})")
        cfg = LlamaConfig(**json.loads(meta["config"]))
        swiglu = set(json.loads(meta.get("swiglu", "[]")))
        raw = ST.load_file(path)
        w: Dict[str, object] = {}
        for name, t in raw.items():
            if name.endswith("::q"):
                base = name[:-3]
                w[base] = Q.Fp8Weight(t.view(torch.float8_e4m3fn).to(device), raw[base + "::scales"].to(device),
                                      base in swiglu)
            elif not name.endswith("::scales"):
                w[name] = t.to(device)
        if "lm_head" not in w:
            w["lm_head"] = w["embed"]
        return cls(cfg, w, int(meta.get("tp_rank", 0)), int(meta.get("tp_size", 1)), comm)

    def set_expert_parallel(self, rank: int, size: int, group=None) -> None:
        """Expert parallelism for mixture-of-experts layers: every rank runs the attention and the router on the
        same tokens (so the routing is identical everywhere), computes only the experts it holds
        (``e % size == rank``) and the partial outputs are summed across ranks with one all-reduce per MoE layer.
        Expert weights, the bulk of a MoE checkpoint, are thereby split ``size`` ways with no token exchange; the
        shared expert, if any, is computed on every rank after the reduction."""
        self.ep = (rank, size, group)

    def set_pipeline(self, stage, first_layer: int, last_layer: int) -> None:
        """Make this model one stage of a pipeline over decoder layers [first_layer, last_layer): the first stage
        embeds the tokens, every stage runs its layers on the hidden states it receives and passes them on, the
        last stage applies the final norm and the LM head, and the logits are shared with every stage so that all
        ranks sample the same tokens and keep their schedulers in step.  ``stage`` provides the transport
        (:class:`antfly_b200.parallel.pipeline.PipelineStage`)."""
        self.pp, self.layer_lo = stage, first_layer
        self.n_layers = last_layer - first_layer

    def offload_experts(self, max_resident_per_layer: int, max_predicted: int = 2, spill_path: Optional[str] = None,
                        host_budget_bytes: int = 0) -> "MoeRuntimeState":
        """Move the routed experts' weights to (pinned) host memory and keep at most ``max_resident_per_layer`` of
        each layer's experts on the device; absent experts are copied in when a step routes to them and the experts
        predicted for the next step are prefetched on a side stream.  For checkpoints whose experts exceed HBM.
        With ``spill_path`` the experts' home is that file instead, and at most ``host_budget_bytes`` of them are
        cached in host memory (for checkpoints whose experts exceed host memory as well)."""
        if spill_path is not None:
            from ..runtime.moe import DiskExpertStore

            store = DiskExpertStore(self.device, spill_path, host_budget_bytes)
        else:
            store = HostExpertStore(self.device)
        for l in range(self.n_layers):
            for e in range(self.cfg.num_experts):
                gu, down = self.w.pop(f"l{l}.e{e}.gu", None), self.w.pop(f"l{l}.e{e}.down", None)
                if gu is not None:
                    store.put(l, e, {"gu": gu, "down": down})
        if spill_path is not None:
            store.seal()
        stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.moe_runtime = MoeRuntimeState(store, ExpertResidency(store.load, max_resident_per_layer, stream),
                                           CoactivationPredictor(), max_predicted)
        return self.moe_runtime

    def _moe_mlp(self, h: torch.Tensor, l: int, T: int) -> torch.Tensor:
        """Sparse mixture-of-experts MLP: soft-max router, top-k experts per token (weights optionally renormalised),
        each expert a SwiGLU MLP on the block-fp8 GEMMs, outputs combined with the routing weights in fp32; plus the
        sigmoid-gated shared expert of Qwen2-MoE.  Tokens are gathered per expert, so every expert's weights are
        read once per step whatever the batch.  Returns fp32 [T, H]."""
        cfg, w, p = self.cfg, self.w, f"l{l}."
        logits = Dn.gemm_bf16(h, w[p + "router"], out_dtype=torch.float32).float()
        probs = torch.softmax(logits, -1)
        topv, topi = probs.topk(cfg.num_experts_per_tok, -1)
        if cfg.norm_topk_prob:
            topv = topv / topv.sum(-1, keepdim=True)
        out = torch.zeros((T, h.shape[1]), dtype=torch.float32, device=h.device)
        batches = route_batches(topi, topv, cfg.num_experts)
        rt = self.moe_runtime
        mine = (lambda e: True) if self.ep is None else (lambda e: e % self.ep[1] == self.ep[0])
        if rt is not None:  # offloaded experts: load what this step needs, prefetch what the next is likely to
            active = [e for e in batches.active if mine(e)]
            ws = rt.residency.ensure(l, active)
            rt.predictor.note(l, cfg.num_experts, batches.active)
            rt.residency.prefetch(l, [e for e in rt.predictor.predict(l, batches.active, rt.max_predicted)[0]
                                      if mine(e)], protect=active)
        for e, rows, wts in batches:
            if not mine(e):
                continue                       # another rank's expert
            gu, down = (ws[e]["gu"], ws[e]["down"]) if rt is not None else (w[p + f"e{e}.gu"], w[p + f"e{e}.down"])
            xe = h.index_select(0, rows)
            act = self._linear(xe, gu, rows.numel(), swiglu=True)
            ye = self._linear(act, down, rows.numel()).float()
            out.index_add_(0, rows, ye * wts[:, None])
        if self.ep is not None:
            import torch.distributed as dist

            dist.all_reduce(out, group=self.ep[2])
        if p + "shared.gu" in w:
            act = self._linear(h, w[p + "shared.gu"], T, swiglu=True)
            ys = self._linear(act, w[p + "shared.down"], T).float()
            gate = torch.sigmoid(Dn.gemm_bf16(h, w[p + "shared.gate"], out_dtype=torch.float32).float())
            out = out + gate * ys
        return out

    def _forward_general(self, b: StepBatch, k_cache, v_cache, attn_scratch) -> torch.Tensor:
        """Variants the fused decode path does not special-case (Gemma: (1 + gamma) norms, scaled embeddings,
        GeGLU): same kernels, with the gated activation applied between the gate/up and down GEMMs instead of in
        an epilogue.  Single GPU."""
        assert self.tp_size == 1, "this model variant runs on one GPU"
        cfg, w = self.cfg, self.w
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        T = b.ids.numel()
        gp1, eps = cfg.norm_plus_one, cfg.rms_norm_eps
        pp, lo = self.pp, self.layer_lo
        hi = lo + self.n_layers
        if pp is None or pp.is_first:
            x = Dn.embed_gather(b.ids, w["embed"], scale=cfg.embed_scale)
            if b.embed_rows is not None:         # soft tokens (image patches) replace their placeholders' rows
                x.index_copy_(0, b.embed_rows.long(), b.embed_vals.to(x.dtype))
        else:
            x = pp.recv_hidden(T, cfg.hidden_size, w[f"l{lo}.ln1"].device)
        zero_pos = torch.zeros_like(b.positions) if b.pos3 is not None else None
        h = Dn.norm(x, w[f"l{lo}.ln1"], eps=eps, rms=True, gamma_plus_one=gp1)

        def lin(a, key, residual=None):
            if not cfg.bitnet:
                return self._linear(a, w[key], T, residual=residual) if residual is not None else \
                    self._linear(a, w[key], T)
            # 8-bit activations are whole numbers up to 128 in magnitude and the weights are -1 / 0 / +1: both are
            # exact in the GEMM's input formats and the fp32 accumulation is exact integer arithmetic
            af = a.float()
            amax = af.abs().amax(-1, keepdim=True).clamp(min=1e-5)
            aq = (af * (127.0 / amax)).round().clamp(-128, 127).to(torch.bfloat16)
            y = Q.gemm_w8a16(aq, w[key], partials=True).sum(0) * (amax / 127.0) * w[key + ".ws"]
            return (y + residual.float()).to(torch.bfloat16) if residual is not None else y.to(torch.bfloat16)

        for l in range(lo, hi):
            p = f"l{l}."
            k_cache_l, v_cache_l = k_cache[l - lo], v_cache[l - lo]
            qkv = lin(h, p + "qkv")
            qkv_bias, rope_pos = w.get(p + "qkv.b"), b.positions
            if b.pos3 is not None:
                # three-stream rotation done here on the fused buffer; the cache-write kernel then rotates by
                # position zero, which is the identity
                from .qwen2vl import mrope_rotate

                assert cfg.mrope_sections is not None and not cfg.qk_norm and cfg.rope_dim == D
                if qkv_bias is not None:
                    qkv = (qkv.float() + qkv_bias.float()).to(qkv.dtype)
                nqk = (Hq + Hkv) * D
                qkv[:, :nqk] = mrope_rotate(qkv[:, :nqk].view(T, Hq + Hkv, D), b.pos3, cfg.rope_theta,
                                            cfg.mrope_sections).view(T, nqk)
                qkv_bias, rope_pos = None, zero_pos
            theta, fscale = cfg.layer_rope[l] if cfg.layer_rope else (cfg.rope_theta, cfg.rope_freq_scale)
            window = cfg.layer_windows[l] if cfg.layer_windows else cfg.sliding_window
            q = A.rope_kv_write(qkv, rope_pos, b.slots, k_cache_l, v_cache_l, Hq, Hkv, D, theta,
                                bias=qkv_bias, rope_dim=cfg.rope_dim, half_split=cfg.rope_half_split,
                                freq_scale=fscale, q_norm_w=w.get(p + "qn"), k_norm_w=w.get(p + "kn"),
                                norm_eps=eps, norm_plus_one=gp1, inv_freq=self.rope_table,
                                rope_mscale=cfg.rope_mscale)
            if cfg.attn_sinks or cfg.attn_logit_softcapping:
                # a softmax with an extra term: the kernel that carries it (bf16 caches)
                ctx = A.paged_attention_sink(q, k_cache_l, v_cache_l, b.block_tables, b.q_starts, b.q_lens, b.kv_lens,
                                             scale=cfg.attn_scale or None, window=window, sinks=w.get(p + "sinks"),
                                             softcap=cfg.attn_logit_softcapping)
            else:
                ctx = A.paged_attention(q, k_cache_l, v_cache_l, b.block_tables, b.q_starts, b.q_lens, b.kv_lens,
                                        b.max_q_len, max_kv=b.max_kv, scale=cfg.attn_scale or None, window=window,
                                        num_splits=b.attn_splits, scratch=attn_scratch)
            if b.bidir is not None:
                # second pass over the image runs without the causal mask (their keys are already in the cache);
                # its rows replace the causal ones
                bs, bl, bk, bt, bmax, brow = b.bidir
                both = A.paged_attention(q, k_cache_l, v_cache_l, bt, bs, bl, bk, bmax, max_kv=b.max_kv, scale=cfg.attn_scale or None,
                                         window=window, causal=False, decode=False)
                ctx.index_copy_(0, brow, both.index_select(0, brow))
            ctx = ctx.view(T, Hq * D)
            if cfg.bitnet:
                ctx = Dn.norm(ctx.contiguous(), w[p + "attn_sub"], eps=eps, rms=True)
            if cfg.post_norms:
                a_out = Dn.norm(lin(ctx, p + "o"), w[p + "post_attn"], eps=eps, rms=True, gamma_plus_one=gp1)
                x = (x.float() + a_out.float()).to(torch.bfloat16)
            else:
                x = lin(ctx, p + "o", residual=x)
            h = Dn.norm(x, w[p + "ln2"], eps=eps, rms=True, gamma_plus_one=gp1)
            if cfg.num_experts > 0:
                x = (x.float() + self._moe_mlp(h, l, T)).to(torch.bfloat16)
                if l + 1 < hi:
                    h = Dn.norm(x, w[f"l{l + 1}.ln1"], eps=eps, rms=True, gamma_plus_one=gp1)
                continue
            # columns alternate gate_i, up_i; activation and product in one elementwise kernel
            act = Dn.gated_act(lin(h, p + "gu"), cfg.gate_act, interleaved=True).to(torch.bfloat16)
            if cfg.bitnet:
                act = Dn.norm(act.contiguous(), w[p + "ffn_sub"], eps=eps, rms=True)
            if cfg.post_norms:
                m_out = Dn.norm(lin(act, p + "down"), w[p + "post_ffn"], eps=eps, rms=True, gamma_plus_one=gp1)
                x = (x.float() + m_out.float()).to(torch.bfloat16)
            else:
                x = lin(act, p + "down", residual=x)
            if l + 1 < hi:
                h = Dn.norm(x, w[f"l{l + 1}.ln1"], eps=eps, rms=True, gamma_plus_one=gp1)
        n_rows = T if b.logit_rows.numel() == T else b.logit_rows.numel()
        if pp is not None and not pp.is_last:
            pp.send_hidden(x)
            return pp.share_logits(None, n_rows, cfg.hidden_size if self.return_hidden else self.vocab_local,
                                   x.device)
        rows = x if b.logit_rows.numel() == T else x.index_select(0, b.logit_rows.long())
        hl = Dn.norm(rows, w["norm"], eps=eps, rms=True, gamma_plus_one=gp1)
        if not self.return_hidden:
            head = w["lm_head"]
            hl = self._linear(hl, head, rows.shape[0]) if isinstance(head, (Q.Fp8Weight, GgufWeight)) else \
                Dn.gemm_bf16(hl, head)
            if cfg.final_logit_softcapping:
                cap = cfg.final_logit_softcapping
                hl = (torch.tanh(hl.float() / cap) * cap).to(hl.dtype)
        return hl if pp is None else pp.share_logits(hl, n_rows, hl.shape[1], hl.device)

    def forward(self, b: StepBatch, k_cache: torch.Tensor, v_cache: torch.Tensor,
                attn_scratch: Optional[A.PagedAttnScratch] = None) -> torch.Tensor:
        """Runs the stack on one step batch; K/V of the step's tokens are written into
        k_cache / v_cache [L, num_blocks, page, Hkv, D].  Returns bf16 logits [R, vocab_local]."""
        cfg, w = self.cfg, self.w
        if cfg.norm_plus_one or cfg.embed_scale != 1.0 or cfg.gate_act != "silu" or cfg.num_experts > 0 or \
                self.pp is not None or b.embed_rows is not None or b.pos3 is not None or cfg.post_norms or \
                b.bidir is not None or cfg.attn_sinks or cfg.attn_logit_softcapping or cfg.final_logit_softcapping or \
                self.native_gguf:
            return self._forward_general(b, k_cache, v_cache, attn_scratch)
        if (self.fused is not None and self._use_mx(b.ids.numel())
                and b.logit_rows.numel() == b.ids.numel() and isinstance(w["lm_head"], Q.Fp8Weight)
                and b.ids.numel() <= self.fused.ws.max_tokens):
            if self.fused.one_shot:
                return self._forward_one_shot(b, k_cache, v_cache, attn_scratch)
            if b.ids.numel() % self.tp_size == 0:
                return self._forward_fused(b, k_cache, v_cache, attn_scratch)
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        T = b.ids.numel()
        mxt = self.act_terms if self._use_mx(T) else 0
        x = Dn.embed_gather(b.ids, w["embed"])
        h = Dn.norm(x, w["l0.ln1"], eps=cfg.rms_norm_eps, rms=True, mx_terms=mxt)
        for l in range(self.n_layers):
            p = f"l{l}."
            qkv_w: Q.Fp8Weight = w[p + "qkv"]
            parts = self._linear(h, qkv_w, T, partials=True,
                                 split_k=pick_split_k(qkv_w.out_features, qkv_w.in_features, T))
            q = A.rope_kv_write(None, b.positions, b.slots, k_cache[l], v_cache[l], Hq, Hkv, D, cfg.rope_theta,
                                partials=parts, bias=w.get(p + "qkv.b"), rope_dim=cfg.rope_dim,
                                half_split=cfg.rope_half_split, freq_scale=cfg.rope_freq_scale,
                                q_norm_w=w.get(p + "qn"), k_norm_w=w.get(p + "kn"), norm_eps=cfg.rms_norm_eps,
                                inv_freq=self.rope_table, rope_mscale=cfg.rope_mscale)
            ctx = A.paged_attention(q, k_cache[l], v_cache[l], b.block_tables, b.q_starts, b.q_lens, b.kv_lens,
                                    b.max_q_len, max_kv=b.max_kv, window=cfg.sliding_window, num_splits=b.attn_splits,
                                    scratch=attn_scratch, mx_terms=mxt)
            o_w: Q.Fp8Weight = w[p + "o"]
            parts = self._reduce(self._linear(ctx if mxt else ctx.view(T, Hq * D), o_w, T, partials=True,
                                              split_k=pick_split_k(o_w.out_features, o_w.in_features, T)))
            x, h = Dn.norm(None, w[p + "ln2"], eps=cfg.rms_norm_eps, rms=True, residual=x, partials=parts,
                           want_sum=True, mx_terms=mxt)
            gu_w: Q.Fp8Weight = w[p + "gu"]
            sk = pick_split_k(gu_w.out_features, gu_w.in_features, T) if mxt else 1
            if sk > 1:
                # Too few weight tiles to fill the SMs: split K and let the quantiser apply SwiGLU to the summed slices.
                act = Q.swiglu_quantize_mx(self._linear(h, gu_w, T, partials=True, split_k=sk), terms=mxt)
            else:
                act = self._linear(h, gu_w, T, swiglu=True)
            d_w: Q.Fp8Weight = w[p + "down"]
            parts = self._reduce(self._linear(act, d_w, T, partials=True,
                                              split_k=pick_split_k(d_w.out_features, d_w.in_features, T)))
            last = l + 1 == self.n_layers
            nw = w["norm"] if last else w[f"l{l + 1}.ln1"]
            if last:
                # Only the rows whose logits are wanted go through the final norm and the LM head.
                x = Dn.norm(None, nw, eps=cfg.rms_norm_eps, rms=True, residual=x, partials=parts, want_sum=True,
                            want_norm=False)
            else:
                x, h = Dn.norm(None, nw, eps=cfg.rms_norm_eps, rms=True, residual=x, partials=parts, want_sum=True,
                               mx_terms=mxt)
        rows = x if b.logit_rows.numel() == T else x.index_select(0, b.logit_rows.long())
        if self.return_hidden:
            return Dn.norm(rows, w["norm"], eps=cfg.rms_norm_eps, rms=True)
        hl = Dn.norm(rows, w["norm"], eps=cfg.rms_norm_eps, rms=True,
                     mx_terms=self.act_terms if self._use_mx(rows.shape[0]) else 0)
        head = w["lm_head"]
        if isinstance(head, Q.Fp8Weight):
            return self._linear(hl, head, rows.shape[0])
        return Dn.gemm_bf16(hl, head)

    def greedy_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        """Arg-max over the (possibly vocabulary-sharded) logits -> global token ids, int32 [R]."""
        if self.tp_size == 1 or self.comm is None:
            return S.argmax(logits)
        if self.fused is not None and logits.shape[0] <= self.fused.ws.ARGMAX_ROWS:
            return self.fused.argmax(logits, self.vocab_offset)
        idx, val = S.argmax(logits, vocab_offset=self.vocab_offset, want_val=True)
        return self.comm.argmax_merge(idx, val)
