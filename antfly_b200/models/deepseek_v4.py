"""DeepSeek-V4 decoder: single-latent attention with sinks, compressed long-range attention, hyper-connections, MoE.

What the reference implements for this family (zig/pkg/inference/src/architectures/deepseek_v4.zig,
deepseek_v4_host.zig, and architectures/gpt.zig:1412-2490), restated as tensor programs:

* **Attention input**: q = q_b(rms(q_a(x))) with a weight-free RMS per head; one shared latent row per token
  kv = rms(kv_proj(x)) that is key *and* value for every head (gpt.zig:1481-1531).  RoPE (interleaved pairs) on the
  trailing ``qk_rope_head_dim`` channels of q and kv; because values carry the rotation, the attention output is
  rotated back by the query's position before the output projection (deepseek_v4_host.zig:352-405).
* **Sliding layers**: causal window attention with a learned per-head sink logit in the softmax denominator.
* **Compressed layers** (``compressed_sparse_attention`` rate r_csa, ``heavily_compressed_attention`` rate r_hca): on
  top of the local window, the query sees one *compressed row* per block of r tokens: a sigmoid-gated mean of
  ``kv_proj(x) + position_bias`` over the block, RMS-normed and rotated at the block's last position; a row is
  visible once its position <= the query's (the open block's row sits at the newest token, so only that token sees
  it) (gpt.zig:1983-2076).  Sparse layers keep only the ``index_topk`` rows with the best indexer score
  sum_h sigmoid(w_h(x)) * <q_idx_h, k_idx> / sqrt(d_idx), where k_idx is a second compressed pool
  (gpt.zig:2402-2468); heavily compressed layers keep all visible rows.
* **Output projection**: heads are split into ``o_groups`` groups, each projected to ``o_lora_rank`` by its own
  slice of o_a, concatenated, then o_b (deepseek_v4_host.zig:796-830).
* **Hyper-connections** (``hc_mult`` residual streams per token): before each sub-block the streams are reduced to one
  row, after it the update is written back into all streams; mixing weights are sigmoids of projections of the
  RMS-scaled flat stream vector, the stream-to-stream matrix goes through Sinkhorn normalisation
  (deepseek_v4_host.zig:149-350, deepseek_v4.zig:1253-1352).  A final ``hc_head`` collapses the streams.
* **MoE**: score = sqrt(softplus) | sigmoid | exp of the router logit; top-k by score + correction bias, weights from
  the unbiased scores, optionally normalised, times ``routed_scaling_factor``; hash layers take their experts from a
  token-id table instead; experts are SwiGLU with gate clamped above and up clamped both ways at ``swiglu_limit``;
  plus an always-on shared expert (deepseek_v4.zig:829-1118).  A limit of 0 means "no clamp" here (the reference
  would clamp everything to zero).

Every projection is the shared bf16 GEMM; the attention, compression and stream mixing are batched tensor ops over
[tokens, heads] with masks instead of the reference's per-row loops.  One sequence at a time with a per-sequence
state (local rows of the last window, the compressor's running inputs and rows): a request-level pipeline drives it
(``pipelines/generation.StatefulGenerator``); speculative decoding is not offered for this cache, as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import dense as Dn

SLIDING, SPARSE, HEAVY = "sliding_attention", "compressed_sparse_attention", "heavily_compressed_attention"


@dataclass
class DeepseekV4Config:
    vocab_size: int = 129280
    hidden_size: int = 4096
    num_hidden_layers: int = 4
    num_attention_heads: int = 32
    head_dim: int = 128
    q_lora_rank: int = 1024
    qk_rope_head_dim: int = 64
    o_groups: int = 1
    o_lora_rank: int = 512
    sliding_window: int = 128
    rope_theta: float = 10000.0
    compress_rope_theta: float = 0.0
    compress_rate_csa: int = 4
    compress_rate_hca: int = 128
    index_n_heads: int = 0
    index_head_dim: int = 0
    index_topk: int = 0
    hc_mult: int = 0
    hc_sinkhorn_iters: int = 0
    hc_eps: float = 0.0
    swiglu_limit: float = 0.0
    num_local_experts: int = 8
    num_experts_per_tok: int = 2
    moe_intermediate_size: int = 1024
    shared_expert_intermediate_size: int = 0
    n_shared_experts: int = 1
    scoring_func: str = "sqrtsoftplus"
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 1.0
    num_hash_layers: int = 0
    layer_types: List[str] = field(default_factory=list)
    mlp_layer_types: List[str] = field(default_factory=list)
    rms_norm_eps: float = 1e-6
    hidden_act: str = "silu"
    tie_word_embeddings: bool = False
    eos_token_id: int = 1

    @classmethod
    def from_hf(cls, d: dict) -> "DeepseekV4Config":
        d = dict(d.get("text_config") or d)
        alias = {"rope_head_dim": "qk_rope_head_dim", "score_func": "scoring_func", "route_scale": "routed_scaling_factor",
                 "n_routed_experts": "num_local_experts", "norm_eps": "rms_norm_eps",
                 "expert_intermediate_size": "moe_intermediate_size"}
        kw = {}
        for k, v in d.items():
            k = alias.get(k, k)
            if k in cls.__dataclass_fields__ and v is not None:
                kw[k] = v
        rates = d.get("compress_rates")
        if isinstance(rates, dict):
            for key, dst in (("compressed_sparse_attention", "compress_rate_csa"), ("csa", "compress_rate_csa"),
                             ("heavily_compressed_attention", "compress_rate_hca"), ("hca", "compress_rate_hca")):
                if key in rates:
                    kw[dst] = int(rates[key])
        c = cls(**kw)
        if not c.layer_types and isinstance(d.get("compress_ratios"), list):     # a per-layer list of rates
            c.layer_types = [SLIDING if r == 0 else SPARSE if r == c.compress_rate_csa else HEAVY
                             for r in d["compress_ratios"][: c.num_hidden_layers]]
        if not c.layer_types:
            c.layer_types = [SLIDING] * c.num_hidden_layers
        if isinstance(c.eos_token_id, list):
            c.eos_token_id = c.eos_token_id[0]
        return c

    def rate(self, layer: int) -> int:
        kind = self.layer_types[layer]
        return 0 if kind == SLIDING else self.compress_rate_csa if kind == SPARSE else self.compress_rate_hca

    def theta(self, layer: int) -> float:
        if self.layer_types[layer] != SLIDING and self.compress_rope_theta > 0:
            return self.compress_rope_theta
        return self.rope_theta

    def hash_routed(self, layer: int) -> bool:
        if layer < len(self.mlp_layer_types):
            return self.mlp_layer_types[layer] == "hash_moe"
        return layer < self.num_hash_layers


# ---------------------------------------------------------------------------------------------------------------
# pieces (all fp32 tensors; rows are tokens)

def rms_rows(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y * weight if weight is not None else y


def trailing_rope(x: torch.Tensor, pos: torch.Tensor, rope_dim: int, theta: float, inverse: bool = False):
    """x [T, heads, D]: rotate channel pairs (2i, 2i+1) of the last ``rope_dim`` channels by pos / theta^(2i/rope_dim)."""
    if rope_dim == 0:
        return x
    D = x.shape[-1]
    i = torch.arange(0, rope_dim, 2, device=x.device, dtype=torch.float32)
    ang = pos.float()[:, None] / torch.pow(torch.tensor(theta, device=x.device), i / rope_dim)[None]
    if inverse:
        ang = -ang
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    head, tail = x[..., : D - rope_dim], x[..., D - rope_dim:]
    x0, x1 = tail[..., 0::2], tail[..., 1::2]
    rot = torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], -1).flatten(-2)
    return torch.cat([head, rot], -1)


def route_score(logits: torch.Tensor, func: str) -> torch.Tensor:
    if func == "sqrtsoftplus":
        return torch.sqrt(torch.nn.functional.softplus(logits, threshold=20.0).clamp_min(0.0))
    if func == "sigmoid":
        return torch.sigmoid(logits)
    if func == "softmax":
        return torch.exp(logits)
    return logits


def select_routes(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, func: str, normalize: bool,
                  scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """[T, E] router logits -> (expert ids [T, k], weights [T, k]): the bias steers the choice only."""
    s = route_score(logits, func)
    pick = (s + bias if bias is not None else s).topk(min(top_k, s.shape[-1]), -1).indices
    w = s.gather(-1, pick)
    if normalize:
        tot = w.sum(-1, keepdim=True)
        w = torch.where(tot > 0, w / tot, w)
    return pick, w * scale


def clamped_swiglu(gate: torch.Tensor, up: torch.Tensor, limit: float) -> torch.Tensor:
    if limit > 0:
        gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
    return torch.nn.functional.silu(gate) * up


def sinkhorn(m: torch.Tensor, iters: int, eps: float) -> torch.Tensor:
    """[..., n, n]: alternately divide rows then columns by (their sum + eps)."""
    for _ in range(iters):
        m = m / (m.sum(-1, keepdim=True) + eps)
        m = m / (m.sum(-2, keepdim=True) + eps)
    return m


def hyper_head_weights(streams: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
                       hc_eps: float, eps: float) -> torch.Tensor:
    """streams [T, hc, H], fn [hc, hc * H] -> sigmoid(<flat, fn_s> * rsqrt(mean flat^2 + eps) * scale + base_s) + hc_eps."""
    flat = streams.flatten(1)
    r = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + eps)
    return torch.sigmoid((flat @ fn.view(fn.shape[0], -1).t()) * r * scale.flatten()[0] + base) + hc_eps


def hyper_mix(streams: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, hc_eps: float,
              eps: float, iters: int):
    """The full connection form, fn [(2 + hc) * hc, hc * H]: -> (pre [T, hc], post [T, hc], comb [T, hc, hc])."""
    T, hc, _ = streams.shape
    flat = streams.flatten(1)
    r = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + eps)
    z = (flat @ fn.view(-1, flat.shape[1]).t()) * r                                       # [T, (2 + hc) * hc]
    sc = scale.flatten()
    pre = torch.sigmoid(z[:, :hc] * sc[0] + base[:hc]) + hc_eps
    post = torch.sigmoid(z[:, hc:2 * hc] * sc[1] + base[hc:2 * hc]) + hc_eps
    comb = torch.sigmoid(z[:, 2 * hc:] * sc[2] + base[2 * hc:]).view(T, hc, hc) + hc_eps
    return pre, post, sinkhorn(comb, iters, hc_eps)


def grouped_output_projection(x: torch.Tensor, o_a: torch.Tensor, groups: int) -> torch.Tensor:
    """x [T, groups * gw], o_a [groups * rank, gw] (group-major rows) -> [T, groups * rank]."""
    T = x.shape[0]
    gw = x.shape[1] // groups
    wa = o_a.view(groups, -1, gw)
    return torch.einsum("tgi,goi->tgo", x.view(T, groups, gw), wa).reshape(T, -1)


@dataclass
class CompressorState:
    projected: torch.Tensor          # [T, row_dim] kv_proj(x) of every token so far
    gate: torch.Tensor               # [T, gate_width]
    rows: torch.Tensor               # [ceil(T / rate), row_dim] compressed rows (rotated)
    positions: torch.Tensor          # [ceil(T / rate)]


@dataclass
class DeepseekV4State:
    length: int = 0
    local: Dict[int, torch.Tensor] = field(default_factory=dict)          # layer -> latent rows of the last window
    comp: Dict[int, CompressorState] = field(default_factory=dict)
    index: Dict[int, CompressorState] = field(default_factory=dict)


class DeepseekV4Model:
    def __init__(self, cfg: DeepseekV4Config, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device, self.dtype = weights["embed"].device, weights["embed"].dtype

    # -- loading ---------------------------------------------------------------------------------------------
    @classmethod
    def from_state_dict(cls, cfg: DeepseekV4Config, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "DeepseekV4Model":
        t = lambda x: x.to(dtype).to(device).contiguous()
        f = lambda x: x.float().to(device).contiguous()
        w: Dict[str, torch.Tensor] = {"embed": t(sd["model.embed_tokens.weight"]), "norm": f(sd["model.norm.weight"])}
        w["lm_head"] = t(sd["lm_head.weight"]) if "lm_head.weight" in sd and not cfg.tie_word_embeddings else w["embed"]
        if cfg.hc_mult:
            for n in ("fn", "base", "scale"):
                w["hc_head." + n] = f(sd["model.hc_head.hc_" + n])
        E = cfg.num_local_experts
        for l in range(cfg.num_hidden_layers):
            s, p = f"model.layers.{l}.", f"l{l}."
            w[p + "ln1"], w[p + "ln2"] = f(sd[s + "input_layernorm.weight"]), f(sd[s + "post_attention_layernorm.weight"])
            a = s + "self_attn."
            for n in ("q_a_proj", "q_b_proj", "kv_proj", "o_b_proj"):
                w[p + n] = t(sd[a + n + ".weight"])
            w[p + "o_a_proj"] = f(sd[a + "o_a_proj.weight"])
            w[p + "q_a_norm"], w[p + "kv_norm"] = f(sd[a + "q_a_norm.weight"]), f(sd[a + "kv_norm.weight"])
            w[p + "sinks"] = f(sd[a + "sinks"]).flatten()
            if cfg.hc_mult:
                for hc in ("attn_hc", "ffn_hc"):
                    for n in ("fn", "base", "scale"):
                        w[p + hc + "." + n] = f(sd[s + hc + "." + n])
            kind = cfg.layer_types[l]
            pools = [] if kind == SLIDING else ["compressor"]
            if kind == SPARSE and cfg.index_n_heads and cfg.index_head_dim:
                pools.append("compressor.indexer")
                w[p + "idx.q_b"] = t(sd[a + "compressor.indexer.q_b_proj.weight"])
                w[p + "idx.w"] = t(sd[a + "compressor.indexer.weights_proj.weight"])
            for pool in pools:
                q = p + ("idx." if pool.endswith("indexer") else "cmp.")
                w[q + "kv"], w[q + "gate"] = t(sd[a + pool + ".kv_proj.weight"]), t(sd[a + pool + ".gate_proj.weight"])
                w[q + "norm"] = f(sd[a + pool + ".kv_norm.weight"])
                w[q + "bias"] = f(sd[a + pool + ".position_bias"])
            m = s + "mlp."
            w[p + "router"] = f(sd[m + "gate.weight"])
            if m + "gate.e_score_correction_bias" in sd:
                w[p + "router.bias"] = f(sd[m + "gate.e_score_correction_bias"])
            if m + "gate.tid2eid" in sd:
                w[p + "tid2eid"] = sd[m + "gate.tid2eid"].to(device).long().view(-1, cfg.num_experts_per_tok)
            if m + "experts.gate_up_proj" in sd:                                  # packed [E, 2, I, H]
                w[p + "e.gu"] = t(sd[m + "experts.gate_up_proj"].reshape(E, -1, cfg.hidden_size))
            elif m + "experts.gate_proj" in sd:                                   # packed, split
                w[p + "e.gu"] = t(torch.cat([sd[m + "experts.gate_proj"], sd[m + "experts.up_proj"]], 1))
            else:                                                                 # one tensor per expert
                def one(e: int, *names: str) -> torch.Tensor:
                    for n in names:
                        for suffix in (".weight", ""):
                            if f"{m}experts.{e}.{n}{suffix}" in sd:
                                return sd[f"{m}experts.{e}.{n}{suffix}"]
                    raise KeyError(f"{m}experts.{e}.{names[0]}")
                w[p + "e.gu"] = t(torch.stack([torch.cat([one(e, "gate_proj", "w1"), one(e, "up_proj", "w3")], 0)
                                               for e in range(E)]))
                w[p + "e.down"] = t(torch.stack([one(e, "down_proj", "w2") for e in range(E)]))
            if p + "e.down" not in w:
                w[p + "e.down"] = t(sd[m + "experts.down_proj"])
            if m + "shared_experts.gate_proj.weight" in sd:
                w[p + "sh.gu"] = t(torch.cat([sd[m + "shared_experts.gate_proj.weight"],
                                              sd[m + "shared_experts.up_proj.weight"]], 0))
                w[p + "sh.down"] = t(sd[m + "shared_experts.down_proj.weight"])
        return cls(cfg, w)

    def new_state(self) -> DeepseekV4State:
        return DeepseekV4State()

    def _lin(self, x: torch.Tensor, wt: torch.Tensor) -> torch.Tensor:
        return Dn.gemm_bf16(x.to(self.dtype).contiguous(), wt, out_dtype=torch.float32).float()

    # -- compressed pools --------------------------------------------------------------------------------------
    def _update_pool(self, st: Optional[CompressorState], h: torch.Tensor, prefix: str, rate: int, row_dim: int,
                     theta: float, start: int) -> CompressorState:
        """Append this call's tokens to a pool and recompute every block they touch: gated mean of
        (projection + position bias) over the block's tokens so far, RMS norm, rotation at the block's last
        position so far."""
        c, w = self.cfg, self.w
        proj, gate = self._lin(h, w[prefix + "kv"]), self._lin(h, w[prefix + "gate"])
        if st is not None:
            proj, gate = torch.cat([st.projected, proj]), torch.cat([st.gate, gate])
        total = proj.shape[0]
        gw = gate.shape[1]
        if gw not in (1, rate):
            raise ValueError(f"compressor gate width {gw} is neither 1 nor the rate {rate}")
        first = start // rate
        n_blocks = (total + rate - 1) // rate
        lo = first * rate
        span = (n_blocks - first) * rate
        pad = lo + span - total
        pj = torch.nn.functional.pad(proj[lo:], (0, 0, 0, pad)).view(-1, rate, row_dim)
        gt = torch.nn.functional.pad(gate[lo:], (0, 0, 0, pad)).view(-1, rate, gw)
        slot = torch.arange(rate, device=h.device)
        g = torch.sigmoid(gt[:, slot, slot] if gw == rate else gt[..., 0])                # [blocks, rate]
        live = (lo + torch.arange(span, device=h.device)).view(-1, rate) < total
        g = g * live
        bias = w[prefix + "bias"]
        bias = bias.view(rate, row_dim) if bias.numel() == rate * row_dim else bias.view(1, row_dim) \
            if bias.numel() == row_dim else torch.zeros(1, row_dim, device=h.device)
        num = (g[..., None] * (pj + bias[None])).sum(1)
        den = g.sum(1, keepdim=True)
        rows = torch.where(den > 0, num / den.clamp_min(1e-30), num)
        rows = rms_rows(rows, w[prefix + "norm"], c.rms_norm_eps)
        ends = (first + torch.arange(n_blocks - first, device=h.device) + 1) * rate - 1
        pos = ends.clamp_max(total - 1)
        rows = trailing_rope(rows[:, None, :], pos, min(c.qk_rope_head_dim, row_dim), theta)[:, 0]
        if st is not None and first > 0:
            rows, pos = torch.cat([st.rows[:first], rows]), torch.cat([st.positions[:first], pos])
        return CompressorState(proj, gate, rows, pos)

    # -- attention ---------------------------------------------------------------------------------------------
    def _attention(self, l: int, h: torch.Tensor, st: DeepseekV4State, pos: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"l{l}."
        T, H, D = h.shape[0], c.num_attention_heads, c.head_dim
        kind, theta, rope = c.layer_types[l], c.theta(l), c.qk_rope_head_dim
        q_lora = rms_rows(self._lin(h, w[p + "q_a_proj"]), w[p + "q_a_norm"], c.rms_norm_eps)
        q = rms_rows(self._lin(q_lora, w[p + "q_b_proj"]).view(T, H, D), None, c.rms_norm_eps)
        q = trailing_rope(q, pos, rope, theta)
        kv = rms_rows(self._lin(h, w[p + "kv_proj"]), w[p + "kv_norm"], c.rms_norm_eps)          # [T, D]
        kv = trailing_rope(kv[:, None, :], pos, rope, theta)[:, 0]
        prev = st.local.get(l)
        local = kv if prev is None else torch.cat([prev, kv])
        first_pos = st.length + T - local.shape[0]
        kpos = first_pos + torch.arange(local.shape[0], device=h.device)
        window = c.sliding_window if c.sliding_window > 0 else 1 << 30
        mask = (kpos[None] <= pos[:, None]) & (kpos[None] > pos[:, None] - window)               # [T, K]
        keys, vis = local, mask
        if kind != SLIDING:
            rate = c.rate(l)
            if rate <= 1:
                raise ValueError(f"layer {l}: compressed attention needs a compress rate above 1")
            st.comp[l] = pool = self._update_pool(st.comp.get(l), h, p + "cmp.", rate, D, theta, st.length)
            seen = pool.positions[None] <= pos[:, None]                                          # [T, R]
            top_k = c.index_topk if kind == SPARSE and c.index_topk > 0 else 0
            if top_k and top_k < pool.rows.shape[0]:
                if kind == SPARSE and c.index_n_heads and c.index_head_dim:
                    st.index[l] = ipool = self._update_pool(st.index.get(l), h, p + "idx.", rate, c.index_head_dim,
                                                            theta, st.length)
                    iq = self._lin(q_lora, w[p + "idx.q_b"]).view(T, c.index_n_heads, c.index_head_dim)
                    hw = torch.sigmoid(self._lin(h, w[p + "idx.w"]))                             # [T, heads]
                    score = torch.einsum("thd,rd,th->tr", iq, ipool.rows, hw) * c.index_head_dim ** -0.5
                else:
                    score = -(pos[:, None] - pool.positions[None]).float()
                score = score.masked_fill(~seen, float("-inf"))
                pick = score.topk(top_k, -1).indices
                chosen = torch.zeros_like(seen).scatter_(1, pick, True)
                seen = seen & chosen
            elif kind == SPARSE and c.index_n_heads and c.index_head_dim:
                st.index[l] = self._update_pool(st.index.get(l), h, p + "idx.", rate, c.index_head_dim, theta,
                                                st.length)
            keys, vis = torch.cat([local, pool.rows]), torch.cat([mask, seen], 1)
        logits = torch.einsum("thd,kd->htk", q, keys) * D ** -0.5
        logits = logits.masked_fill(~vis[None], float("-inf"))
        sink = w[p + "sinks"][:, None, None].expand(H, T, 1)
        prob = torch.softmax(torch.cat([sink, logits], -1), -1)[..., 1:]                         # the sink takes mass
        ctx = torch.einsum("htk,kd->thd", prob, keys)
        ctx = trailing_rope(ctx, pos, rope, theta, inverse=True)
        st.local[l] = local[-min(window, local.shape[0]):] if window < (1 << 30) else local
        mid = grouped_output_projection(ctx.reshape(T, H * D), w[p + "o_a_proj"], max(1, c.o_groups))
        return self._lin(mid, w[p + "o_b_proj"])

    # -- feed-forward ------------------------------------------------------------------------------------------
    def _ffn(self, l: int, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"l{l}."
        logits = x @ w[p + "router"].t()
        k = min(c.num_experts_per_tok, c.num_local_experts)
        if p + "tid2eid" in w and c.hash_routed(l):
            ti = w[p + "tid2eid"][ids]
            tw = route_score(logits, c.scoring_func).gather(-1, ti)
            if c.norm_topk_prob:
                tot = tw.sum(-1, keepdim=True)
                tw = torch.where(tot > 0, tw / tot, tw)
            tw = tw * c.routed_scaling_factor
        else:
            ti, tw = select_routes(logits, w.get(p + "router.bias"), k, c.scoring_func, c.norm_topk_prob,
                                   c.routed_scaling_factor)
        out = torch.zeros_like(x)
        for e in ti.unique().tolist():
            tok, slot = torch.where(ti == e)
            gu = self._lin(x[tok], w[p + "e.gu"][e])
            I = gu.shape[1] // 2
            y = self._lin(clamped_swiglu(gu[:, :I], gu[:, I:], c.swiglu_limit), w[p + "e.down"][e])
            out.index_add_(0, tok, y * tw[tok, slot][:, None])
        if p + "sh.gu" in w:
            gu = self._lin(x, w[p + "sh.gu"])
            I = gu.shape[1] // 2
            out = out + self._lin(torch.nn.functional.silu(gu[:, :I]) * gu[:, I:], w[p + "sh.down"])
        return out

    # -- hyper-connections ---------------------------------------------------------------------------------------
    def _hc_pre(self, streams: torch.Tensor, key: str) -> torch.Tensor:
        c, w = self.cfg, self.w
        fn, base, scale = w[key + ".fn"], w[key + ".base"], w[key + ".scale"]
        hc = c.hc_mult
        if fn.numel() == (2 + hc) * hc * streams[0].numel():
            pre, _, comb = hyper_mix(streams, fn, base, scale, c.hc_eps, c.rms_norm_eps, c.hc_sinkhorn_iters)
            return torch.einsum("td,tds,tsh->th", pre, comb, streams)
        wts = hyper_head_weights(streams, fn, base, scale, c.hc_eps, c.rms_norm_eps)
        return torch.einsum("ts,tsh->th", wts, streams)

    def _hc_post(self, streams: torch.Tensor, update: torch.Tensor, key: str) -> torch.Tensor:
        c, w = self.cfg, self.w
        fn, base, scale = w[key + ".fn"], w[key + ".base"], w[key + ".scale"]
        hc = c.hc_mult
        if fn.numel() == (2 + hc) * hc * streams[0].numel():
            pre, post, comb = hyper_mix(streams, fn, base, scale, c.hc_eps, c.rms_norm_eps, c.hc_sinkhorn_iters)
            mixed = torch.einsum("tds,tsh->tdh", comb, streams)
            return pre[..., None] * (mixed + post[..., None] * update[:, None, :])
        wts = hyper_head_weights(streams, fn, base, scale, c.hc_eps, c.rms_norm_eps)
        return streams + wts[..., None] * update[:, None, :]

    # -- the model -----------------------------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, state: Optional[DeepseekV4State] = None):
        """ids [T] (the next tokens of one sequence) -> (logits [T, vocab] fp32, state)."""
        c, w = self.cfg, self.w
        st = state if state is not None else self.new_state()
        ids = ids.long().to(self.device)
        T = ids.numel()
        pos = torch.arange(st.length, st.length + T, device=self.device)
        x = w["embed"][ids].float()
        hc = c.hc_mult
        streams = x[:, None, :].expand(T, hc, -1).contiguous() if hc else None
        for l in range(c.num_hidden_layers):
            p = f"l{l}."
            a_in = self._hc_pre(streams, p + "attn_hc") if hc else x
            upd = self._attention(l, rms_rows(a_in, w[p + "ln1"], c.rms_norm_eps), st, pos)
            if hc:
                streams = self._hc_post(streams, upd, p + "attn_hc")
            else:
                x = x + upd
            f_in = self._hc_pre(streams, p + "ffn_hc") if hc else x
            upd = self._ffn(l, rms_rows(f_in, w[p + "ln2"], c.rms_norm_eps), ids)
            if hc:
                streams = self._hc_post(streams, upd, p + "ffn_hc")
            else:
                x = x + upd
        if hc:
            wts = hyper_head_weights(streams, w["hc_head.fn"], w["hc_head.base"], w["hc_head.scale"], c.hc_eps,
                                     c.rms_norm_eps)
            x = torch.einsum("ts,tsh->th", wts, streams)
        x = rms_rows(x, w["norm"], c.rms_norm_eps)
        st.length += T
        return self._lin(x, w["lm_head"]), st

    @torch.no_grad()
    def generate(self, ids, max_new_tokens: int) -> List[int]:
        logits, st = self.forward(torch.as_tensor(ids))
        out: List[int] = []
        for _ in range(max_new_tokens):
            tok = int(logits[-1].argmax())
            out.append(tok)
            if tok == self.cfg.eos_token_id:
                break
            logits, st = self.forward(torch.tensor([tok]), st)
        return out
