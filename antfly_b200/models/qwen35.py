"""Qwen3.5 hybrid decoder: gated delta-rule (linear attention) layers interleaved with gated full-attention layers.

Every ``full_attention_interval``-th layer is softmax attention with an output gate -- the query projection is twice
as wide, its second half is a per-channel sigmoid gate on the attention output --, partial rotary embedding
(``partial_rotary_factor`` of each head, half-split pairs) and per-head RMS norms on Q and K with (1 + w) weights;
all other layers are :class:`GatedDeltaNetLayer`.  All norms are RMS with (1 + w).  A sequence's state is a KV
cache for the attention layers and (convolution tail, matrix state) for the recurrent ones, so memory does not
grow with context in three layers out of four.

The reference builds the same decoder around its delta-rule op
(zig/pkg/inference/src/architectures/gpt.zig:4462-4775, family qwen3.5 in models/gpt.zig:28).  Here projections run
on the bf16 GEMM and the attention layers on the packed flash kernel (prefill) or tensor ops over the cached keys
(decode); the model keeps its own per-sequence state (it is not served through the paged-KV engine, whose block
tables have no place for recurrent state).  Checked against ``transformers`` Qwen3_5ForCausalLM on CPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import dense as Dn
from ..ops import reference as R
from .deltanet import DeltaNetConfig, GatedDeltaNetLayer


@dataclass
class Qwen35Config:
    vocab_size: int = 151936
    hidden_size: int = 2048
    intermediate_size: int = 6144
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    num_key_value_heads: int = 2
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000000.0
    partial_rotary_factor: float = 0.25
    layer_types: List[str] = field(default_factory=list)
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    tie_word_embeddings: bool = False

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen35Config":
        d = dict(d.get("text_config") or d)
        rp = d.get("rope_parameters") or {}
        kw = {k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None}
        kw.setdefault("rope_theta", rp.get("rope_theta", d.get("rope_theta", 10000000.0)))
        kw.setdefault("partial_rotary_factor", rp.get("partial_rotary_factor", d.get("partial_rotary_factor", 0.25)))
        cfg = cls(**kw)
        if not cfg.layer_types:
            interval = int(d.get("full_attention_interval", 4))
            cfg.layer_types = ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
                               for i in range(cfg.num_hidden_layers)]
        return cfg


def _rms1p(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm with (1 + w) weights, fp32 arithmetic."""
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())


@dataclass
class Qwen35State:
    """One sequence's decoding state: per layer either (K, V) [Hkv, t, D] or (conv tail, S)."""
    layers: List[Optional[tuple]]
    length: int = 0


class Qwen35Model:
    def __init__(self, cfg: Qwen35Config, weights: Dict[str, torch.Tensor], linear: Dict[int, GatedDeltaNetLayer]):
        self.cfg, self.w, self.linear = cfg, weights, linear
        self.device = weights["embed"].device
        self.dtype = weights["embed"].dtype

    @classmethod
    def from_state_dict(cls, cfg: Qwen35Config, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "Qwen35Model":
        pre = "model.language_model." if any(k.startswith("model.language_model.") for k in sd) else "model."
        t = lambda x: x.to(dtype).to(device).contiguous()
        f = lambda x: x.float().to(device).contiguous()
        w = {"embed": t(sd[pre + "embed_tokens.weight"]), "norm": f(sd[pre + "norm.weight"])}
        w["lm_head"] = w["embed"] if cfg.tie_word_embeddings or "lm_head.weight" not in sd else t(sd["lm_head.weight"])
        dcfg = DeltaNetConfig(cfg.hidden_size, cfg.linear_num_key_heads, cfg.linear_num_value_heads,
                              cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.linear_conv_kernel_dim,
                              cfg.rms_norm_eps)
        linear = {}
        for l, kind in enumerate(cfg.layer_types):
            s, p = f"{pre}layers.{l}.", f"l{l}."
            w[p + "ln1"], w[p + "ln2"] = f(sd[s + "input_layernorm.weight"]), f(sd[s + "post_attention_layernorm.weight"])
            w[p + "gu"] = t(torch.cat([sd[s + "mlp.gate_proj.weight"], sd[s + "mlp.up_proj.weight"]], 0))
            w[p + "down"] = t(sd[s + "mlp.down_proj.weight"])
            if kind == "linear_attention":
                linear[l] = GatedDeltaNetLayer.from_state_dict(dcfg, sd, prefix=s + "linear_attn.", device=device,
                                                               dtype=dtype)
            else:
                a = s + "self_attn."
                w[p + "qkv"] = t(torch.cat([sd[a + "q_proj.weight"], sd[a + "k_proj.weight"], sd[a + "v_proj.weight"]], 0))
                w[p + "o"] = t(sd[a + "o_proj.weight"])
                w[p + "qn"], w[p + "kn"] = f(sd[a + "q_norm.weight"]), f(sd[a + "k_norm.weight"])
        return cls(cfg, w, linear)

    # ------------------------------------------------------------------------------------------------------------
    def new_state(self) -> Qwen35State:
        return Qwen35State([None] * self.cfg.num_hidden_layers, 0)

    def _attention(self, l: int, x: torch.Tensor, st: Qwen35State) -> torch.Tensor:
        c, w = self.cfg, self.w
        T = x.shape[0]
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        p = f"l{l}."
        proj = Dn.gemm_bf16(x, w[p + "qkv"], out_dtype=torch.float32).float()
        qg = proj[:, : 2 * Hq * D].view(T, Hq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(T, Hq * D)
        k = proj[:, 2 * Hq * D: 2 * Hq * D + Hkv * D].view(T, Hkv, D)
        v = proj[:, 2 * Hq * D + Hkv * D:].view(T, Hkv, D)
        q, k = _rms1p(q, w[p + "qn"], c.rms_norm_eps), _rms1p(k, w[p + "kn"], c.rms_norm_eps)
        pos = torch.arange(st.length, st.length + T, device=x.device, dtype=torch.int32)
        rd = int(D * c.partial_rotary_factor)
        q, k = R.rope(q, pos, c.rope_theta, rd, True, 1.0), R.rope(k, pos, c.rope_theta, rd, True, 1.0)
        prev = st.layers[l]
        kk = k.transpose(0, 1) if prev is None else torch.cat([prev[0], k.transpose(0, 1)], 1)   # [Hkv, t, D]
        vv = v.transpose(0, 1) if prev is None else torch.cat([prev[1], v.transpose(0, 1)], 1)
        st.layers[l] = (kk, vv)
        g = Hq // Hkv
        sc = torch.einsum("thd,hsd->hts", q.float(), kk.repeat_interleave(g, 0).float()) * D ** -0.5
        n_keys = kk.shape[1]
        qpos = torch.arange(n_keys - T, n_keys, device=x.device)[:, None]
        sc = sc.masked_fill(torch.arange(n_keys, device=x.device)[None, :] > qpos, float("-inf"))
        ctx = torch.einsum("hts,hsd->thd", sc.softmax(-1), vv.repeat_interleave(g, 0).float()).reshape(T, Hq * D)
        ctx = ctx * torch.sigmoid(gate)
        return Dn.gemm_bf16(ctx.to(self.dtype).contiguous(), w[p + "o"], out_dtype=torch.float32).float()

    def forward(self, ids: torch.Tensor, state: Optional[Qwen35State] = None) -> Tuple[torch.Tensor, Qwen35State]:
        """ids [T] (the next tokens of one sequence, in order) -> (logits [T, vocab] fp32, state)."""
        c, w = self.cfg, self.w
        st = state if state is not None else self.new_state()
        x = w["embed"][ids.long()].float()
        T = x.shape[0]
        for l, kind in enumerate(c.layer_types):
            p = f"l{l}."
            h = _rms1p(x, w[p + "ln1"], c.rms_norm_eps).to(self.dtype)
            if kind == "linear_attention":
                y, st.layers[l] = self.linear[l].forward(h, st.layers[l])
                y = y.float()
            else:
                y = self._attention(l, h.contiguous(), st)
            x = x + y
            h = _rms1p(x, w[p + "ln2"], c.rms_norm_eps).to(self.dtype).contiguous()
            gu = Dn.gemm_bf16(h, w[p + "gu"], out_dtype=torch.float32).float()
            F = gu.shape[1] // 2
            act = (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]).to(self.dtype).contiguous()
            x = x + Dn.gemm_bf16(act, w[p + "down"], out_dtype=torch.float32).float()
        st.length += T
        h = _rms1p(x, w["norm"], c.rms_norm_eps).to(self.dtype).contiguous()
        return Dn.gemm_bf16(h, w["lm_head"], out_dtype=torch.float32).float(), st

    def generate(self, prompt: Sequence[int], max_new_tokens: int, eos_token_id: Optional[int] = None) -> List[int]:
        """Greedy decoding: prefill the prompt once, then one token at a time over the carried state."""
        ids = torch.tensor(list(prompt), dtype=torch.int64, device=self.device)
        logits, st = self.forward(ids)
        out: List[int] = []
        for _ in range(max_new_tokens):
            tok = int(logits[-1].argmax())
            out.append(tok)
            if eos_token_id is not None and tok == eos_token_id:
                break
            logits, st = self.forward(torch.tensor([tok], dtype=torch.int64, device=self.device), st)
        return out
