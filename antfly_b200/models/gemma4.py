"""Gemma-4 text decoder: per-layer embeddings, layers that share another layer's keys and values, two attention
geometries, optional mixture-of-experts block, final-logit soft cap.

What distinguishes it from the Llama-style decoders of ``models/llama.py``:

* alternating ``sliding_attention`` / ``full_attention`` layers with DIFFERENT head widths (``head_dim`` vs
  ``global_head_dim``) and rotary schemes (plain RoPE, base 10k, vs "proportional" RoPE: pairs span the whole head,
  only the first ``partial_rotary_factor`` of the angles rotate); Q and K get per-head RMS norms, V an RMS norm
  without weights; the softmax scale is 1; with ``attention_k_eq_v`` the full-attention layers have no value
  projection (V = the K projection before its norm and rotation) and their own number of KV heads;
* the last ``num_kv_shared_layers`` layers compute no keys or values: each reads the cache of the last earlier
  layer of its own type (the reference's shared-KV layers, zig/pkg/inference/src/models/gpt.zig:1121);
* per-layer embeddings (zig/pkg/inference/src/models/gpt.zig:153): a second embedding table gives every token a
  small vector per layer, mixed with a projection of the main embedding, and gates a low-rank update at the end of
  each layer; every layer's output is multiplied by a stored scalar;
* four norms per layer; an optional MoE block runs in parallel with the dense MLP (router on the un-normalised
  residual, top-k weights renormalised and scaled per expert); KV-shared layers may use a double-wide MLP;
* logits are soft-capped: ``cap * tanh(logits / cap)`` (zig/pkg/inference/src/models/gpt.zig:219).

Because the layers' cache geometries differ, the model keeps its own per-sequence state (like the hybrid
Qwen3.5 decoder) and is served through ``pipelines.generation.StatefulGenerator``; projections run on the bf16
GEMM, the rest is tensor arithmetic.  Checked against ``transformers`` Gemma4ForCausalLM on CPU.  Reference:
zig/pkg/inference/src/architectures/gpt.zig (family gemma4), gemma4_runtime / gemma4_projector for the vision side.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import dense as Dn


@dataclass
class Gemma4Config:
    vocab_size: int = 262144
    hidden_size: int = 2304
    intermediate_size: int = 9216
    num_hidden_layers: int = 30
    num_attention_heads: int = 8
    num_key_value_heads: int = 4
    head_dim: int = 256
    global_head_dim: int = 512
    num_global_key_value_heads: Optional[int] = None
    attention_k_eq_v: bool = False
    rms_norm_eps: float = 1e-6
    sliding_window: int = 512
    layer_types: List[str] = field(default_factory=list)
    final_logit_softcapping: Optional[float] = None
    vocab_size_per_layer_input: int = 262144
    hidden_size_per_layer_input: int = 256
    num_kv_shared_layers: int = 0
    enable_moe_block: bool = False
    use_double_wide_mlp: bool = False
    num_experts: Optional[int] = None
    top_k_experts: Optional[int] = None
    moe_intermediate_size: Optional[int] = None
    rope_local_theta: float = 10000.0
    rope_global_theta: float = 1000000.0
    rope_global_fraction: float = 0.25
    tie_word_embeddings: bool = True

    @classmethod
    def from_hf(cls, d: dict) -> "Gemma4Config":
        d = dict(d.get("text_config") or d)
        kw = {k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None}
        rp = d.get("rope_parameters") or {}
        if "sliding_attention" in rp:
            kw["rope_local_theta"] = rp["sliding_attention"].get("rope_theta", 10000.0)
        if "full_attention" in rp:
            kw["rope_global_theta"] = rp["full_attention"].get("rope_theta", 1000000.0)
            kw["rope_global_fraction"] = rp["full_attention"].get("partial_rotary_factor", 1.0) \
                if rp["full_attention"].get("rope_type") == "proportional" else 1.0
        cfg = cls(**kw)
        if not cfg.layer_types:
            cfg.layer_types = ["sliding_attention" if (i + 1) % 6 else "full_attention"
                               for i in range(cfg.num_hidden_layers)]
            cfg.layer_types[-1] = "full_attention"
        return cfg


def _rms(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    return y * w.float() if w is not None else y


def _gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def _rope_half(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [T, H, D]; rotates pairs (j, j + D / 2) by pos * inv_freq[j] (inv_freq 0 = no rotation)."""
    ang = pos.float()[:, None] * inv_freq[None, :]                    # [T, D / 2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    h = x.shape[-1] // 2
    a, b = x[..., :h].float(), x[..., h:].float()
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)


@dataclass
class Gemma4State:
    kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)   # layer -> (K, V) [Hkv, t, D]
    length: int = 0


class Gemma4TextModel:
    def __init__(self, cfg: Gemma4Config, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device, self.dtype = weights["embed"].device, weights["embed"].dtype
        c = cfg
        L = c.num_hidden_layers
        first_shared = L - c.num_kv_shared_layers
        self.first_shared = first_shared
        prev = c.layer_types[:first_shared]
        # a shared layer reads the cache of the last non-shared layer of its own type
        self.kv_source = {l: (len(prev) - 1 - prev[::-1].index(c.layer_types[l])) if (l >= first_shared > 0) else l
                          for l in range(L)}
        dev = self.device
        d_loc, d_glb = c.head_dim, (c.global_head_dim or c.head_dim)
        self.inv_freq = {
            "sliding_attention": 1.0 / (c.rope_local_theta ** (torch.arange(0, d_loc, 2, device=dev).float() / d_loc))}
        n_rot = int(c.rope_global_fraction * d_glb // 2)
        inv = 1.0 / (c.rope_global_theta ** (torch.arange(0, 2 * n_rot, 2, device=dev).float() / d_glb))
        self.inv_freq["full_attention"] = torch.cat([inv, torch.zeros(d_glb // 2 - n_rot, device=dev)])

    # ------------------------------------------------------------------------------------------------------------
    @classmethod
    def from_state_dict(cls, cfg: Gemma4Config, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "Gemma4TextModel":
        pre = "model.language_model." if any(k.startswith("model.language_model.") for k in sd) else "model."
        t = lambda x: x.to(dtype).to(device).contiguous()
        f = lambda x: x.float().to(device).contiguous()
        w: Dict[str, torch.Tensor] = {"embed": t(sd[pre + "embed_tokens.weight"]), "norm": f(sd[pre + "norm.weight"])}
        w["lm_head"] = w["embed"] if cfg.tie_word_embeddings or "lm_head.weight" not in sd else t(sd["lm_head.weight"])
        if cfg.hidden_size_per_layer_input:
            w["ple.embed"] = t(sd[pre + "embed_tokens_per_layer.weight"])
            w["ple.proj"] = t(sd[pre + "per_layer_model_projection.weight"])
            w["ple.norm"] = f(sd[pre + "per_layer_projection_norm.weight"])
        for l in range(cfg.num_hidden_layers):
            s, p = f"{pre}layers.{l}.", f"l{l}."
            a = s + "self_attn."
            w[p + "q"], w[p + "o"] = t(sd[a + "q_proj.weight"]), t(sd[a + "o_proj.weight"])
            w[p + "qn"] = f(sd[a + "q_norm.weight"])
            if a + "k_proj.weight" in sd:
                w[p + "k"], w[p + "kn"] = t(sd[a + "k_proj.weight"]), f(sd[a + "k_norm.weight"])
            if a + "v_proj.weight" in sd:
                w[p + "v"] = t(sd[a + "v_proj.weight"])
            for n, key in (("ln1", "input_layernorm"), ("ln2", "post_attention_layernorm"),
                           ("ln3", "pre_feedforward_layernorm"), ("ln4", "post_feedforward_layernorm")):
                w[p + n] = f(sd[s + key + ".weight"])
            w[p + "gu"] = t(torch.cat([sd[s + "mlp.gate_proj.weight"], sd[s + "mlp.up_proj.weight"]], 0))
            w[p + "down"] = t(sd[s + "mlp.down_proj.weight"])
            w[p + "scalar"] = f(sd[s + "layer_scalar"]) if s + "layer_scalar" in sd else torch.ones(1, device=device)
            if cfg.hidden_size_per_layer_input:
                w[p + "ple.gate"], w[p + "ple.proj"] = t(sd[s + "per_layer_input_gate.weight"]), t(
                    sd[s + "per_layer_projection.weight"])
                w[p + "ple.norm"] = f(sd[s + "post_per_layer_input_norm.weight"])
            if cfg.enable_moe_block:
                w[p + "r.proj"], w[p + "r.scale"] = f(sd[s + "router.proj.weight"]), f(sd[s + "router.scale"])
                w[p + "r.per_expert"] = f(sd[s + "router.per_expert_scale"])
                w[p + "e.gu"], w[p + "e.down"] = t(sd[s + "experts.gate_up_proj"]), t(sd[s + "experts.down_proj"])
                for n, key in (("ln5", "post_feedforward_layernorm_1"), ("ln6", "post_feedforward_layernorm_2"),
                               ("ln7", "pre_feedforward_layernorm_2")):
                    w[p + n] = f(sd[s + key + ".weight"])
        return cls(cfg, w)

    def new_state(self) -> Gemma4State:
        return Gemma4State()

    # ------------------------------------------------------------------------------------------------------------
    def _lin(self, x: torch.Tensor, wt: torch.Tensor) -> torch.Tensor:
        return Dn.gemm_bf16(x.to(self.dtype).contiguous(), wt, out_dtype=torch.float32).float()

    def _attention(self, l: int, h: torch.Tensor, st: Gemma4State, pos: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"l{l}."
        kind = c.layer_types[l]
        sliding = kind == "sliding_attention"
        D = c.head_dim if sliding else (c.global_head_dim or c.head_dim)
        alt = c.attention_k_eq_v and not sliding
        Hq = c.num_attention_heads
        Hkv = (c.num_global_key_value_heads or c.num_key_value_heads) if alt else c.num_key_value_heads
        T = h.shape[0]
        inv = self.inv_freq[kind]
        q = _rope_half(_rms(self._lin(h, w[p + "q"]).view(T, Hq, D), w[p + "qn"], c.rms_norm_eps), pos, inv)
        src = self.kv_source[l]
        if src != l:
            kk, vv = st.kv[src]
        else:
            kraw = self._lin(h, w[p + "k"]).view(T, Hkv, D)
            vraw = self._lin(h, w[p + "v"]).view(T, Hkv, D) if (p + "v") in w else kraw
            k = _rope_half(_rms(kraw, w[p + "kn"], c.rms_norm_eps), pos, inv)
            v = _rms(vraw, None, c.rms_norm_eps)
            prev = st.kv.get(l)
            kk = k.transpose(0, 1) if prev is None else torch.cat([prev[0], k.transpose(0, 1)], 1)
            vv = v.transpose(0, 1) if prev is None else torch.cat([prev[1], v.transpose(0, 1)], 1)
            st.kv[l] = (kk, vv)
        g = Hq // kk.shape[0]
        sc = torch.einsum("thd,hsd->hts", q, kk.repeat_interleave(g, 0))           # softmax scale is 1
        n_keys = kk.shape[1]
        kpos = torch.arange(n_keys, device=h.device)[None, :]
        qpos = pos.long()[:, None]
        mask = kpos <= qpos
        if sliding:
            mask = mask & (kpos > qpos - c.sliding_window)
            grp = getattr(self, "_groups", None)
            if grp is not None and n_keys == T:           # whole prompt in one call: image tokens see their image
                gq = grp.to(h.device)
                mask = mask | ((gq[:, None] == gq[None, :]) & (gq[:, None] >= 0))
        sc = sc.masked_fill(~mask[None], float("-inf"))
        ctx = torch.einsum("hts,hsd->thd", sc.softmax(-1), vv.repeat_interleave(g, 0)).reshape(T, Hq * D)
        return self._lin(ctx, w[p + "o"])

    def _moe(self, l: int, resid: torch.Tensor) -> torch.Tensor:
        """Experts on the pre-MLP residual: router over the weight-free RMS norm of it, top-k renormalised."""
        c, w = self.cfg, self.w
        p = f"l{l}."
        r = _rms(resid, None, c.rms_norm_eps) * w[p + "r.scale"] * c.hidden_size ** -0.5
        probs = (r @ w[p + "r.proj"].t()).softmax(-1)
        tw, ti = probs.topk(c.top_k_experts, -1)
        tw = tw / tw.sum(-1, keepdim=True) * w[p + "r.per_expert"][ti]
        x = _rms(resid, w[p + "ln7"], c.rms_norm_eps)
        out = torch.zeros_like(x)
        for e in ti.unique().tolist():
            tok, slot = torch.where(ti == e)
            gu = self._lin(x[tok], w[p + "e.gu"][e])
            F = gu.shape[1] // 2
            y = self._lin(_gelu_tanh(gu[:, :F]) * gu[:, F:], w[p + "e.down"][e])
            out.index_add_(0, tok, y * tw[tok, slot][:, None])
        return out

    def forward(self, ids: torch.Tensor, state: Optional[Gemma4State] = None, soft_rows: Optional[torch.Tensor] = None,
                soft_vals: Optional[torch.Tensor] = None, pad_token_id: int = 0,
                vision_groups: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Gemma4State]:
        """ids [T] (the next tokens of one sequence) -> (logits [T, vocab] fp32, state).

        Images: ``soft_rows`` are the positions (within ``ids``) of image placeholder tokens and ``soft_vals``
        [n, hidden] their projected soft tokens (``models/gemma4v.py``); those rows take the soft token as their
        embedding and the padding token's per-layer embedding.  ``vision_groups`` [T] (image number, -1 for text)
        lets the tokens of one image attend to each other in both directions in the sliding-window layers (the
        larger checkpoints' ``use_bidirectional_attention = "vision"``); prefill such a prompt in one call."""
        c, w = self.cfg, self.w
        st = state if state is not None else self.new_state()
        T = ids.numel()
        ids = ids.long()
        if soft_rows is not None:
            ids = ids.clone()
            ids[soft_rows.long()] = pad_token_id
        self._groups = vision_groups
        pos = torch.arange(st.length, st.length + T, device=ids.device)
        scale = torch.tensor(c.hidden_size ** 0.5, dtype=self.dtype)      # the reference model rounds the scale too
        x = (w["embed"][ids] * scale.to(w["embed"].device)).float()
        x_text = x
        if soft_rows is not None:
            x = x.clone()
            x[soft_rows.long()] = soft_vals.float().to(x.device)
        ple = None
        P = c.hidden_size_per_layer_input
        if P:
            L = c.num_hidden_layers
            pscale = torch.tensor(P ** 0.5, dtype=self.dtype).to(w["embed"].device)
            tok_part = (w["ple.embed"][ids] * pscale).float().view(T, L, P)
            proj = (self._lin(x, w["ple.proj"]) * c.hidden_size ** -0.5).view(T, L, P)
            del x_text
            ple = (_rms(proj, w["ple.norm"], c.rms_norm_eps) + tok_part) * 2.0 ** -0.5
        for l in range(c.num_hidden_layers):
            p = f"l{l}."
            h = _rms(x, w[p + "ln1"], c.rms_norm_eps)
            a = self._attention(l, h, st, pos)
            x = x + _rms(a, w[p + "ln2"], c.rms_norm_eps)
            resid = x
            h = _rms(x, w[p + "ln3"], c.rms_norm_eps)
            gu = self._lin(h, w[p + "gu"])
            F = gu.shape[1] // 2
            m = self._lin(_gelu_tanh(gu[:, :F]) * gu[:, F:], w[p + "down"])
            if c.enable_moe_block:
                m = _rms(m, w[p + "ln5"], c.rms_norm_eps) + _rms(self._moe(l, resid), w[p + "ln6"], c.rms_norm_eps)
            x = resid + _rms(m, w[p + "ln4"], c.rms_norm_eps)
            if P:
                g = _gelu_tanh(self._lin(x, w[p + "ple.gate"])) * ple[:, l]
                x = x + _rms(self._lin(g, w[p + "ple.proj"]), w[p + "ple.norm"], c.rms_norm_eps)
            x = x * w[p + "scalar"]
        st.length += T
        logits = self._lin(_rms(x, w["norm"], c.rms_norm_eps), w["lm_head"])
        if c.final_logit_softcapping:
            logits = torch.tanh(logits / c.final_logit_softcapping) * c.final_logit_softcapping
        return logits, st

    def generate(self, prompt: Sequence[int], max_new_tokens: int, eos_token_id: Optional[int] = None) -> List[int]:
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
