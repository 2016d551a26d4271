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
    last_hidden: Optional[torch.Tensor] = None      # final-norm hidden row of the newest token
    groups: Optional[torch.Tensor] = None           # image number of the current call's tokens (-1 = text)


class Gemma4TextModel:
    def __init__(self, cfg: Gemma4Config, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device, self.dtype = weights["embed"].device, weights["embed"].dtype
        self.query_only = False            # an assistant body: no keys / values of its own, see Gemma4Assistant
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
        if src != l or self.query_only:
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
            grp = st.groups
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
        st.groups = vision_groups              # (kept on the sequence's state: requests may run concurrently)
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
        x = self._layers(x, ple, st, pos)
        st.length += T
        hidden = _rms(x, w["norm"], c.rms_norm_eps)
        logits = self._lin(hidden, w["lm_head"])
        if c.final_logit_softcapping:
            logits = torch.tanh(logits / c.final_logit_softcapping) * c.final_logit_softcapping
        st.last_hidden = hidden[-1]
        return logits, st

    def _layers(self, x: torch.Tensor, ple: Optional[torch.Tensor], st: Gemma4State, pos: torch.Tensor) -> torch.Tensor:
        """The decoder stack on embedded rows x [T, hidden] at positions ``pos``; appends to (or, for a query-only
        body, only reads) the caches in ``st``.  Returns the rows before the final norm."""
        c, w = self.cfg, self.w
        P = c.hidden_size_per_layer_input if ple is not None else 0
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
        return x

    @staticmethod
    def truncate(st: Gemma4State, length: int) -> None:
        """Forget everything after the first ``length`` tokens (rejected speculative tokens)."""
        for l, (k, v) in list(st.kv.items()):
            st.kv[l] = (k[:, :length], v[:, :length])
        st.length = length

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


def kv_donor_layers(cfg: Gemma4Config) -> Tuple[Optional[int], Optional[int]]:
    """(sliding, full): the last layer of each kind that owns its cache; None when the model has no KV-shared tail
    (zig/pkg/inference/src/architectures/gemma4_mtp.zig targetKvDonorLayer)."""
    if cfg.num_kv_shared_layers == 0 or cfg.num_hidden_layers <= cfg.num_kv_shared_layers:
        return None, None
    own = cfg.layer_types[: cfg.num_hidden_layers - cfg.num_kv_shared_layers]
    last = lambda kind: max((i for i, t in enumerate(own) if t == kind), default=None)
    return last("sliding_attention"), last("full_attention")


class Gemma4Assistant:
    """Gemma-4 multi-token-prediction assistant: a compact *query-only* decoder that drafts tokens for a target model.

    One draft step (gemma4_mtp.zig draftToken): concatenate the target's (scaled) embedding of the newest token with
    an activation of target width (first the target's final hidden row of that token, then the assistant's own
    projection), map it to the assistant width with ``pre_projection``, run the assistant's layers (they have no
    keys / values of their own: every layer attends to the *target's* cache of the last cache-owning layer of its
    kind, at the newest token's position), take the final-norm hidden row, read logits off the assistant's tied
    embedding, and project the row back to target width with ``post_projection`` for the next chained step.
    With ordered embeddings the argmax only looks at the tokens of the ``centroid_intermediate_top_k`` best
    vocabulary clusters (``masked_embedding.centroids`` scores clusters, ``masked_embedding.token_ordering`` lists
    each cluster's tokens)."""

    def __init__(self, body: Gemma4TextModel, target: Gemma4TextModel, extra: Dict[str, torch.Tensor],
                 num_centroids: int = 0, centroid_top_k: int = 0, ordered: bool = False):
        slide, full = kv_donor_layers(target.cfg)
        if slide is None or full is None:
            raise ValueError("the target has no KV-shared tail with a sliding and a full donor layer")
        if extra["pre"].shape[1] != 2 * target.cfg.hidden_size:
            raise ValueError("assistant backbone width does not match the target's hidden size")
        self.body, self.target, self.x = body, target, extra
        body.query_only = True
        body.kv_source = {l: slide if t == "sliding_attention" else full for l, t in enumerate(body.cfg.layer_types)}
        self.num_centroids, self.centroid_top_k, self.ordered = num_centroids, centroid_top_k, ordered
        self.drafted = self.matched = self.rounds = 0

    @classmethod
    def from_state_dict(cls, hf_config: dict, sd: Dict[str, torch.Tensor], target: Gemma4TextModel, device="cuda",
                        dtype=torch.bfloat16) -> "Gemma4Assistant":
        tc = dict(hf_config.get("text_config") or hf_config)
        tc.setdefault("num_kv_shared_layers", 0)
        cfg = Gemma4Config.from_hf(tc)
        cfg.num_kv_shared_layers = 0
        cfg.hidden_size_per_layer_input = 0
        body = Gemma4TextModel.from_state_dict(cfg, sd, device=device, dtype=dtype)
        t = lambda x: x.to(dtype).to(device).contiguous()
        extra = {"pre": t(sd["pre_projection.weight"]), "post": t(sd["post_projection.weight"])}
        if "masked_embedding.centroids.weight" in sd:
            extra["centroids"] = t(sd["masked_embedding.centroids.weight"])
            extra["ordering"] = sd["masked_embedding.token_ordering"].to(device).long()
        return cls(body, target, extra, int(hf_config.get("num_centroids", 0)),
                   int(hf_config.get("centroid_intermediate_top_k", 0)), bool(hf_config.get("use_ordered_embeddings")))

    def _pick(self, hidden: torch.Tensor, logits: torch.Tensor) -> int:
        """Argmax of the draft logits; with ordered embeddings only over the tokens of the best clusters."""
        V = logits.numel()
        nc, k = self.num_centroids, self.centroid_top_k
        if not (self.ordered and nc and k and "centroids" in self.x and V % nc == 0):
            return int(logits.argmax())
        cl = self.body._lin(hidden[None], self.x["centroids"])[0]
        top = cl.topk(min(k, nc)).indices
        size = V // nc
        cand = self.x["ordering"].view(nc, size)[top].flatten()
        cand = cand[(cand >= 0) & (cand < V)]
        if cand.numel() == 0:
            return int(logits.argmax())
        return int(cand[logits[cand].argmax()])

    def draft(self, token: int, activation: torch.Tensor, st: Gemma4State, k: int) -> List[int]:
        """``k`` chained draft tokens after ``token`` (the newest token of ``st``, whose final hidden row is
        ``activation``).  Reads the target's caches; changes nothing."""
        tgt, body = self.target, self.body
        pos = torch.tensor([st.length - 1], device=body.device)
        scale = torch.tensor(tgt.cfg.hidden_size ** 0.5, dtype=tgt.dtype).to(tgt.device)
        out: List[int] = []
        act = activation.float()
        for _ in range(k):
            emb = (tgt.w["embed"][token] * scale).float()
            x = body._lin(torch.cat([emb, act])[None], self.x["pre"])
            h = _rms(body._layers(x, None, st, pos), body.w["norm"], body.cfg.rms_norm_eps)
            logits = body._lin(h, body.w["embed"])[0]
            token = self._pick(h[0], logits)
            out.append(token)
            act = body._lin(h, self.x["post"])[0]
        return out

    @torch.no_grad()
    def stream(self, prompt: Sequence[int], max_new_tokens: int, k: int = 4, forward_kwargs: Optional[dict] = None):
        """Greedy generation of the *target*, sped up by drafting; yields tokens as they are accepted.  Every round
        drafts ``k`` tokens, the target scores them in one pass, the longest agreeing prefix is kept plus the
        target's own next token (a correction after a mismatch, a bonus after full agreement); the rejected tail is
        cut from the target's caches.  The tokens equal the target's plain greedy output.  ``forward_kwargs``:
        extra inputs of the prompt pass (image soft tokens)."""
        tgt = self.target
        dev = tgt.device
        k = max(1, min(int(k), 16))
        logits, st = tgt.forward(torch.tensor(list(prompt), dtype=torch.int64, device=dev), None,
                                 **(forward_kwargs or {}))
        last = int(logits[-1].argmax())
        n = 1
        yield last
        if n >= max_new_tokens:
            return
        nxt, st = tgt.forward(torch.tensor([last], device=dev), st)            # the cache now covers the newest token
        while n < max_new_tokens:
            kk = min(k, max_new_tokens - n)
            drafts = self.draft(last, st.last_hidden, st, kk)
            base = st.length
            ver, st = tgt.forward(torch.tensor(drafts, device=dev), st)
            want = [int(nxt[-1].argmax())] + [int(r.argmax()) for r in ver]
            m = 0
            while m < kk and drafts[m] == want[m]:
                m += 1
            self.rounds, self.drafted, self.matched = self.rounds + 1, self.drafted + kk, self.matched + m
            for tok in (drafts[:m] + [want[m]])[: max_new_tokens - n]:
                n += 1
                yield tok
            if n >= max_new_tokens:
                return
            last = want[m]
            tgt.truncate(st, base + m)
            nxt, st = tgt.forward(torch.tensor([last], device=dev), st)

    def generate(self, prompt: Sequence[int], max_new_tokens: int, k: int = 4,
                 eos_token_id: Optional[int] = None) -> List[int]:
        out: List[int] = []
        for tok in self.stream(prompt, max_new_tokens, k):
            out.append(tok)
            if eos_token_id is not None and tok == eos_token_id:
                break
        return out
