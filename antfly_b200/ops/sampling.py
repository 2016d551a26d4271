"""On-device token selection: argmax, penalties, temperature/top-k/top-p/min-p sampling, speculative verify."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native as N
from . import reference as R

_c_int = ctypes.c_int
_c_long = ctypes.c_long


def argmax(logits: torch.Tensor, vocab_offset: int = 0, out: Optional[torch.Tensor] = None,
           want_val: bool = False):
    """Row-wise argmax of [rows, V] bf16/fp32 logits -> int32 [rows] (lowest index on ties)."""
    rows, V = logits.shape
    if not logits.is_cuda:
        idx = logits.float().argmax(-1).int() + vocab_offset
        return (idx, logits.float().max(-1).values) if want_val else idx
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    val = torch.empty((rows,), dtype=torch.float32, device=logits.device) if want_val else None
    rc = N.cuda().afb_argmax(N.ptr(logits), _c_int(1 if logits.dtype == torch.float32 else 0),
                             _c_long(logits.stride(0)), _c_int(rows), _c_int(V), N.ptr(out), N.ptr(val),
                             _c_int(vocab_offset), N.stream_ptr())
    N.check(rc, "afb_argmax")
    N.count_launch()
    return (out, val) if want_val else out


def argmax_tp(logits: torch.Tensor, vocab_offset: int, peer_slots, world: int, rank: int, max_rows: int,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Arg-max over vocabulary-sharded logits merged across the tensor-parallel ranks inside the kernel
    (``peer_slots``: ctypes array of every rank's key-slot buffer, see SymmetricWorkspace).  Returns global
    token ids, identical on every rank."""
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    rc = N.cuda().afb_argmax_tp(N.ptr(logits), _c_int(1 if logits.dtype == torch.float32 else 0),
                                _c_long(logits.stride(0)), _c_int(rows), _c_int(V), N.ptr(out), None,
                                _c_int(vocab_offset), peer_slots, _c_int(world), _c_int(rank), _c_int(max_rows),
                                N.stream_ptr())
    N.check(rc, "afb_argmax_tp")
    N.count_launch()
    return out


def count_tokens(counts: torch.Tensor, tokens: torch.Tensor, rows: torch.Tensor) -> None:
    """counts[rows[i], tokens[i]] += 1 (uint16 saturating; stored as int16 tensor [B, V])."""
    n = tokens.numel()
    if n == 0:
        return
    if not counts.is_cuda:
        c = counts.view(torch.int16)
        for t, r in zip(tokens.tolist(), rows.tolist()):
            if c[r, t] != -1:
                c[r, t] += 1
        return
    rc = N.cuda().afb_count_tokens(N.ptr(counts), N.ptr(tokens), N.ptr(rows), _c_int(n), _c_int(counts.shape[1]),
                                   N.stream_ptr())
    N.check(rc, "afb_count_tokens")
    N.count_launch()


def penalties(logits, counts, rep=None, freq=None, pres=None) -> torch.Tensor:
    """fp32 logits with repetition (divide if > 0 else multiply) / frequency / presence penalties applied to
    tokens whose count is non-zero."""
    rows, V = logits.shape
    if not logits.is_cuda:
        x = logits.float().clone()
        c = counts.view(torch.int16).float() if counts is not None else torch.zeros_like(x)
        c = torch.where(c < 0, c + 65536.0, c)
        seen = c > 0
        if rep is not None:
            r = rep[:, None]
            x = torch.where(seen & (x > 0), x / r, torch.where(seen, x * r, x))
        if freq is not None:
            x = x - freq[:, None] * c
        if pres is not None:
            x = x - pres[:, None] * seen.float()
        return x
    out = torch.empty((rows, V), dtype=torch.float32, device=logits.device)
    rc = N.cuda().afb_penalties(N.ptr(logits), _c_int(1 if logits.dtype == torch.float32 else 0),
                                _c_long(logits.stride(0)), N.ptr(out), N.ptr(counts), N.ptr(rep), N.ptr(freq),
                                N.ptr(pres), _c_int(rows), _c_int(V), N.stream_ptr())
    N.check(rc, "afb_penalties")
    N.count_launch()
    return out


def sample(logits: torch.Tensor, temperature, top_k, top_p, min_p, uniform, want_prob: bool = False):
    """logits fp32 [B, V]; per-row temperature (<= 0 greedy), top_k (<= 0 off), top_p (>= 1 off), min_p (<= 0 off);
    uniform in [0, 1) drives the draw."""
    B, V = logits.shape
    if not logits.is_cuda:
        out = torch.empty((B,), dtype=torch.int32)
        prob = torch.ones((B,), dtype=torch.float32)
        for b in range(B):
            t = float(temperature[b])
            if t <= 0:
                out[b] = int(logits[b].argmax())
                continue
            p = R.filtered_probs(logits[b], t, int(top_k[b]), float(top_p[b]), float(min_p[b]))
            cum = p.cumsum(-1)
            i = int(torch.searchsorted(cum, torch.tensor(float(uniform[b]) * float(cum[-1]), dtype=cum.dtype),
                                       right=True))
            i = min(i, V - 1)
            out[b] = i
            prob[b] = p[i]
        return (out, prob) if want_prob else out
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    prob = torch.empty((B,), dtype=torch.float32, device=logits.device) if want_prob else None
    rc = N.cuda().afb_sample(N.ptr(logits), _c_int(B), _c_int(V), N.ptr(temperature), N.ptr(top_k), N.ptr(top_p),
                             N.ptr(min_p), N.ptr(uniform), N.ptr(out), N.ptr(prob), N.stream_ptr())
    N.check(rc, "afb_sample")
    N.count_launch()
    return (out, prob) if want_prob else out


def spec_verify(draft: torch.Tensor, target: torch.Tensor):
    """draft int32 [B, K], target int32 [B, K+1] -> (n_matched int32 [B], next_token int32 [B])."""
    B, K = draft.shape
    if not draft.is_cuda:
        n, nxt = R.spec_verify(draft.long(), target.long())
        return n.int(), nxt.int()
    n = torch.empty((B,), dtype=torch.int32, device=draft.device)
    nxt = torch.empty((B,), dtype=torch.int32, device=draft.device)
    rc = N.cuda().afb_spec_verify(N.ptr(draft), N.ptr(target), _c_int(B), _c_int(K), N.ptr(n), N.ptr(nxt),
                                  N.stream_ptr())
    N.check(rc, "afb_spec_verify")
    N.count_launch()
    return n, nxt
