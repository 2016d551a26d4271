"""Plain PyTorch fp32 statements of every op the CUDA kernels implement.

They serve two purposes: (1) the numerics oracle of the GPU tests (each kernel is compared against the function
of the same name here), and (2) the CPU execution path, so models, pipelines and the HTTP API run, slowly, on a
machine with no GPU.  The maths restates the reference's CPU semantics; citations are on each function.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def act_fn(x: torch.Tensor, act: Optional[str]) -> torch.Tensor:
    if act in (None, "none"):
        return x
    if act in ("gelu", "gelu_erf"):
        return F.gelu(x)
    if act in ("gelu_tanh", "gelu_new"):
        return F.gelu(x, approximate="tanh")
    if act == "relu":
        return F.relu(x)
    if act == "silu":
        return F.silu(x)
    if act == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if act == "relu2":
        return F.relu(x).square()
    raise ValueError(f"unknown activation {act}")


def linear(a, w, bias=None, act=None, residual=None, alpha: float = 1.0) -> torch.Tensor:
    """act(alpha * a @ w.T + bias) + residual in fp32."""
    y = alpha * (a.float() @ w.float().t())
    if bias is not None:
        y = y + bias.float()
    y = act_fn(y, act)
    if residual is not None:
        y = y + residual.float()
    return y


def norm(x, gamma, beta=None, eps=1e-5, rms=False, residual=None, bias=None, partials=None,
         gamma_plus_one=False, round_sum_bf16=True):
    """Returns (sum, y).  The sum is rounded to bf16 before normalising, as the kernel stores it that way."""
    h = x.float() if x is not None else 0.0
    if partials is not None:
        h = h + partials.float().sum(0)
    if bias is not None:
        h = h + bias.float()
    if residual is not None:
        h = h + residual.float()
    s = h
    if round_sum_bf16:
        s = h.to(torch.bfloat16).float()
    g = gamma.float() + (1.0 if gamma_plus_one else 0.0)
    if rms:
        y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * g
    else:
        mu = s.mean(-1, keepdim=True)
        var = (s - mu).pow(2).mean(-1, keepdim=True)
        y = (s - mu) * torch.rsqrt(var + eps) * g
    if beta is not None:
        y = y + beta.float()
    return s, y


def bert_embed_ln(ids, positions, type_ids, word, pos, typ, gamma, beta, eps=1e-12):
    """zig/pkg/inference/src/architectures/bert.zig:131-189: three lookups, add, LayerNorm."""
    ty = type_ids.long() if type_ids is not None else torch.zeros_like(ids).long()
    h = word.float()[ids.long()] + pos.float()[positions.long()] + typ.float()[ty]
    return norm(h, gamma, beta, eps=eps, round_sum_bf16=False)[1]


def pool(h, starts, lens, mode="mean", normalize=True, mask=None):
    """zig/pkg/inference/src/pipelines/embedding.zig:322-390 (+ l2Normalize)."""
    out = []
    hf = h.float()
    for s, n in zip(starts.tolist(), lens.tolist()):
        rows = hf[s:s + n]
        if mask is not None:
            m = mask[s:s + n] > 0
            rows_active = rows[m]
        else:
            rows_active = rows
        if mode == "cls":
            v = rows[0] if n > 0 else torch.zeros(hf.shape[-1], device=h.device)
        elif rows_active.shape[0] == 0:
            v = torch.zeros(hf.shape[-1], device=h.device)
        elif mode == "mean":
            v = rows_active.mean(0)
        elif mode == "max":
            v = rows_active.max(0).values
        elif mode == "last":
            v = rows_active[-1]
        else:
            raise ValueError(mode)
        if normalize:
            nrm = v.norm()
            v = v / nrm if nrm > 0 else v * 0
        out.append(v)
    return torch.stack(out)


def maxsim(q, d, starts, lens):
    """zig/pkg/inference/src/pipelines/reranking.zig:354-383: sum over query tokens of the best cosine."""
    qn = F.normalize(q.float(), dim=-1)
    out = []
    for s, n in zip(starts.tolist(), lens.tolist()):
        if n == 0:
            out.append(torch.zeros((), device=q.device))
            continue
        dn = F.normalize(d.float()[s:s + n], dim=-1)
        out.append((qn @ dn.t()).max(-1).values.sum())
    return torch.stack(out)


def splade_pool(logits, starts, lens):
    out = []
    for s, n in zip(starts.tolist(), lens.tolist()):
        x = torch.log1p(F.relu(logits.float()[s:s + n]))
        out.append(x.max(0).values if n > 0 else torch.zeros(logits.shape[-1], device=logits.device))
    return torch.stack(out)


# ----------------------------------------------------------------------------------------------------------
# Rotary embedding (zig/lib/linalg/src/attention.zig:65-86)
# ----------------------------------------------------------------------------------------------------------
def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: Optional[int] = None,
         half_split: bool = True, freq_scale: float = 1.0, inv_freq: Optional[torch.Tensor] = None,
         mscale: float = 1.0) -> torch.Tensor:
    """x: [T, heads, D]; rotates the first rope_dim dims.  half_split pairs (j, j+rope_dim/2) (Llama);
    otherwise consecutive pairs (2j, 2j+1).  ``inv_freq`` [rope_dim / 2] replaces the closed-form frequencies and
    ``mscale`` then multiplies cos / sin (context-extension schemes)."""
    T, Hh, D = x.shape
    rd = rope_dim or D
    xf = x.float().clone()
    if inv_freq is not None:
        freq = inv_freq.to(x.device).float()
    else:
        j = torch.arange(rd // 2, device=x.device, dtype=torch.float32)
        freq = theta ** (-2.0 * j / rd)
        mscale = 1.0
    ang = positions.float()[:, None] * freq_scale * freq[None, :]
    c, s = ang.cos()[:, None, :] * mscale, ang.sin()[:, None, :] * mscale
    if half_split:
        a, b = xf[..., : rd // 2], xf[..., rd // 2: rd]
        xf[..., : rd // 2], xf[..., rd // 2: rd] = a * c - b * s, a * s + b * c
    else:
        a, b = xf[..., 0:rd:2], xf[..., 1:rd:2]
        xf[..., 0:rd:2], xf[..., 1:rd:2] = a * c - b * s, a * s + b * c
    return xf


# ----------------------------------------------------------------------------------------------------------
# Attention
# ----------------------------------------------------------------------------------------------------------
def varlen_attention(q, k, v, cu_seqlens, scale=None, causal=False, window=0):
    """Packed bidirectional (or causal) attention.  q: [T, Hq, D], k/v: [T, Hkv, D].  ``window`` > 0 keeps keys
    with key > query - window, and without the causal mask also key < query + window."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros((T, Hq, D), dtype=torch.float32, device=q.device)
    cs = cu_seqlens.tolist()
    for b in range(len(cs) - 1):
        s, e = cs[b], cs[b + 1]
        if e == s:
            continue
        qq = q[s:e].float().transpose(0, 1)  # [Hq, L, D]
        kk = k[s:e].float().transpose(0, 1).repeat_interleave(g, 0)
        vv = v[s:e].float().transpose(0, 1).repeat_interleave(g, 0)
        sc = qq @ kk.transpose(1, 2) * scale
        if causal:
            L = e - s
            m = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            sc = sc.masked_fill(~m, float("-inf"))
        if window > 0:
            i = torch.arange(e - s, device=q.device)
            d = i[None, :] - i[:, None]  # key - query
            m = (d > -window) & ((d < window) if not causal else torch.ones_like(d, dtype=torch.bool))
            sc = sc.masked_fill(~m, float("-inf"))
        out[s:e] = (sc.softmax(-1) @ vv).transpose(0, 1)
    return out


def alibi_slopes(num_heads: int) -> torch.Tensor:
    """Per-head ALiBi slopes: a geometric sequence starting at 2^(-8 / n) for n = the largest power of two <= heads,
    with the remaining heads interleaved from the sequence for 2n (Press et al., as used by BLOOM / MPT)."""
    n = 2 ** math.floor(math.log2(num_heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
    slopes = [base ** (i + 1) for i in range(n)]
    if n < num_heads:
        extra = 2.0 ** (-(2.0 ** -(math.log2(2 * n) - 3)))
        slopes += [extra ** (2 * i + 1) for i in range(num_heads - n)]
    return torch.tensor(slopes, dtype=torch.float32)


def paged_attention(q, k_cache, v_cache, block_tables, q_starts, q_lens, kv_lens, scale=None,
                    sliding_window: int = 0, alibi: Optional[torch.Tensor] = None, causal: bool = True,
                    sinks: Optional[torch.Tensor] = None, softcap: float = 0.0):
    """Causal attention of packed query tokens against a paged KV cache.

    q: [T, Hq, D]; k_cache / v_cache: [num_blocks, page, Hkv, D]; block_tables: [B, max_blocks] int32;
    sequence b owns query rows q_starts[b] .. +q_lens[b], which are the LAST q_lens[b] positions of a
    sequence whose total length (already written to the cache) is kv_lens[b].  Matches the masks of the
    reference's gqaPagedAttentionDirect (zig/pkg/inference/src/ops/native_compute.zig:35093-35173): query at
    absolute position p sees keys at positions <= p, and > p - sliding_window when a window is set.
    ``alibi`` [Hq] adds ``slope_h * (key position - query position)`` to the scores (linear position bias).
    ``sinks`` [Hq]: a per-head logit that takes part in the softmax without a value (attention sinks);
    ``softcap`` > 0: scaled scores become ``softcap * tanh(score / softcap)`` before masking.
    """
    T, Hq, D = q.shape
    page, Hkv = k_cache.shape[1], k_cache.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros((T, Hq, D), dtype=torch.float32, device=q.device)
    for b in range(block_tables.shape[0]):
        qs, ql, kl = int(q_starts[b]), int(q_lens[b]), int(kv_lens[b])
        if ql == 0:
            continue
        nblk = (kl + page - 1) // page
        blocks = block_tables[b, :nblk].long()
        kk = k_cache[blocks].float().reshape(-1, Hkv, D)[:kl]  # [kl, Hkv, D]
        vv = v_cache[blocks].float().reshape(-1, Hkv, D)[:kl]
        kk = kk.transpose(0, 1).repeat_interleave(g, 0)
        vv = vv.transpose(0, 1).repeat_interleave(g, 0)
        qq = q[qs:qs + ql].float().transpose(0, 1)
        sc = qq @ kk.transpose(1, 2) * scale  # [Hq, ql, kl]
        qpos = torch.arange(kl - ql, kl, device=q.device)[:, None]
        kpos = torch.arange(kl, device=q.device)[None, :]
        if alibi is not None:
            sc = sc + alibi.to(sc.device).float()[:, None, None] * (kpos - qpos).float()[None]
        m = (kpos <= qpos) if causal else torch.ones_like(kpos <= qpos)
        if sliding_window > 0:
            m = m & (kpos > qpos - sliding_window)
            if not causal:                       # two-sided window, as in the packed (non-paged) attention
                m = m & (kpos < qpos + sliding_window)
        if softcap > 0:
            sc = softcap * torch.tanh(sc / softcap)
        sc = sc.masked_fill(~m, float("-inf"))
        if sinks is not None:
            col = sinks.to(sc.device).float()[:, None, None].expand(Hq, ql, 1)
            pr = torch.cat([sc, col], -1).softmax(-1)[..., :-1]
        else:
            pr = sc.softmax(-1)
        out[qs:qs + ql] = (pr @ vv).transpose(0, 1)
    return out


# ----------------------------------------------------------------------------------------------------------
# Block-scaled fp8 (e4m3 values, one e8m0 power-of-two scale per 32 elements along K)
# ----------------------------------------------------------------------------------------------------------
def quantize_block_fp8(w: torch.Tensor, block: int = 32):
    """Returns (q [N, K] float8_e4m3fn, scales [K/block, N] uint8 e8m0).  Scale = 2^ceil(log2(amax/448))."""
    Nn, K = w.shape
    assert K % block == 0
    wf = w.float().reshape(Nn, K // block, block)
    amax = wf.abs().amax(-1).clamp_min(1e-30)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    scale = torch.exp2(e)
    q = (wf / scale[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).reshape(Nn, K)
    e8 = (e + 127).to(torch.uint8).t().contiguous()  # [K/block, N]
    return q, e8


def dequantize_block_fp8(q: torch.Tensor, e8: torch.Tensor, block: int = 32) -> torch.Tensor:
    Nn, K = q.shape
    scale = torch.exp2(e8.t().float() - 127.0)  # [N, K/block]
    return (q.float().reshape(Nn, K // block, block) * scale[..., None]).reshape(Nn, K)


def linear_w8(x, q, e8, bias=None, act=None, residual=None):
    """x @ dequant(q, e8).T with the weight rounded to bf16 after scaling (exact for power-of-two scales)."""
    w = dequantize_block_fp8(q, e8).to(torch.bfloat16)
    return linear(x, w, bias, act, residual)


def gated_act(gu: torch.Tensor, act: str = "silu", interleaved: bool = False, limit: float = 0.0) -> torch.Tensor:
    """act(gate) * up in fp32 from one GEMM output [T, 2F]: halves (gate | up) or interleaved (gate_j, up_j
    adjacent).  ``limit`` > 0 clamps gate from above and up to [-limit, limit] first."""
    y = gu.float()
    if interleaved:
        g, u = y[..., 0::2], y[..., 1::2]
    else:
        g, u = y[..., : y.shape[-1] // 2], y[..., y.shape[-1] // 2:]
    if limit > 0:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return act_fn(g, act) * u


def swiglu_interleaved(y: torch.Tensor) -> torch.Tensor:
    """Rows of the fused gate/up weight alternate gate_i, up_i; y[..., 2i] = gate, y[..., 2i+1] = up."""
    g, u = y[..., 0::2], y[..., 1::2]
    return F.silu(g.float()) * u.float()


# ----------------------------------------------------------------------------------------------------------
# Sampling (zig/pkg/inference/src/pipelines/generation.zig:3196-3226, 5062-5158)
# ----------------------------------------------------------------------------------------------------------
def apply_penalties(logits, prev_tokens, repetition_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0):
    """logits [V] fp32; prev_tokens: 1-D LongTensor of context + generated ids."""
    logits = logits.clone()
    if prev_tokens is None or prev_tokens.numel() == 0:
        return logits
    V = logits.shape[-1]
    counts = torch.bincount(prev_tokens.clamp(0, V - 1), minlength=V).to(logits.dtype)
    seen = counts > 0
    if repetition_penalty != 1.0:
        pos = logits > 0
        logits = torch.where(seen & pos, logits / repetition_penalty, logits)
        logits = torch.where(seen & ~pos, logits * repetition_penalty, logits)
    if frequency_penalty != 0.0:
        logits = logits - frequency_penalty * counts
    if presence_penalty != 0.0:
        logits = logits - presence_penalty * seen.to(logits.dtype)
    return logits


def filtered_probs(logits, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0):
    """Order: /T -> softmax -> top-k -> top-p -> min-p (p < min_p * p_max dropped); renormalised."""
    p = torch.softmax(logits.float() / max(temperature, 1e-6), -1)
    V = p.shape[-1]
    if 0 < top_k < V:
        kth = torch.topk(p, top_k).values[..., -1:]
        p = torch.where(p < kth, torch.zeros_like(p), p)
    if top_p < 1.0:
        sp, si = torch.sort(p, descending=True)
        cum = sp.cumsum(-1)
        keep_sorted = (cum - sp) < top_p * cum[..., -1:]
        keep = torch.zeros_like(p, dtype=torch.bool).scatter(-1, si, keep_sorted)
        p = torch.where(keep, p, torch.zeros_like(p))
    if min_p > 0.0:
        p = torch.where(p < min_p * p.max(-1, keepdim=True).values, torch.zeros_like(p), p)
    return p / p.sum(-1, keepdim=True)


def spec_verify(draft: torch.Tensor, target: torch.Tensor):
    """draft [B, K], target [B, K+1] (the target's own choice at each of the K+1 verified positions).
    Returns (n_matched [B], next_token [B]): tokens match while draft[i] == target[i]; the next token is
    target[n_matched] -- a correction after a mismatch, the bonus token when all K matched
    (zig/pkg/inference/src/pipelines/generation.zig:3228-3340)."""
    B, K = draft.shape
    eq = (draft == target[:, :K]).long()
    n = torch.cumprod(eq, dim=1).sum(1)
    nxt = target.gather(1, n[:, None]).squeeze(1)
    return n, nxt


# ----------------------------------------------------------------------------------------------------------
# Vector distances (zig/lib/vector/src/vector.zig:359-376): lower is closer for all three.
# ----------------------------------------------------------------------------------------------------------
def distances(q: torch.Tensor, x: torch.Tensor, metric: str) -> torch.Tensor:
    qf, xf = q.float(), x.float()
    dot = qf @ xf.t()
    if metric == "inner_product":
        return -dot
    qn = qf.pow(2).sum(-1, keepdim=True)
    xn = xf.pow(2).sum(-1)[None, :]
    if metric == "l2_squared":
        return (qn + xn - 2 * dot).clamp_min(0)
    if metric == "cosine":
        den = qn.sqrt() * xn.sqrt()
        return torch.where(den > 0, 1 - dot / den.clamp_min(1e-30), torch.ones_like(dot))
    raise ValueError(metric)
