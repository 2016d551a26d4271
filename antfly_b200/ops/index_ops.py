"""ctypes wrappers of the vector-index kernels (persistent score/filter GEMM, arg-min assignment, top-k select,
k-means update, row norms, RaBitQ estimator).  CPU tensors take the fp32 oracle path."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from .. import _native as N
from . import reference as R

_c_int = ctypes.c_int
_c_long = ctypes.c_long
_c_float = ctypes.c_float


def gemm_persistent(a, w, bias=None, act=None, residual=None, out=None, out_dtype=torch.bfloat16, alpha=1.0):
    """Throughput bf16 GEMM (persistent, double-buffered accumulators); same contract as dense.gemm_bf16."""
    from .dense import ACT

    if not a.is_cuda:
        return R.linear(a, w, bias, act, residual, alpha).to(out_dtype)
    M, K = a.shape
    Nn = w.shape[0]
    if out is None:
        out = torch.empty((M, Nn), dtype=out_dtype, device=a.device)
    rc = N.cuda().afb_gemm_persistent(
        N.ptr(a), N.ptr(w), N.ptr(out), N.ptr(bias), N.ptr(residual), _c_int(M), _c_int(Nn), _c_int(K),
        _c_int(a.stride(0)), _c_int(w.stride(0)), _c_int(out.stride(0)),
        _c_int(residual.stride(0) if residual is not None else 0), _c_int(ACT[act]),
        _c_int(1 if out.dtype == torch.float32 else 0), _c_float(alpha), N.stream_ptr())
    N.check(rc, "afb_gemm_persistent")
    N.count_launch()
    return out


def row_sqnorm(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return x.float().pow(2).sum(-1)
    out = torch.empty((x.shape[0],), dtype=torch.float32, device=x.device)
    rc = N.cuda().afb_row_sqnorm(N.ptr(x), _c_long(x.stride(0)), N.ptr(out), _c_int(x.shape[0]), _c_int(x.shape[1]),
                                 N.stream_ptr())
    N.check(rc, "afb_row_sqnorm")
    N.count_launch()
    return out


def score_filter(q, x, row_term, col_term, scale, clamp_zero, threshold, cand_val, cand_idx, cand_count,
                 col_offset: int = 0) -> None:
    """Append (distance, col_offset + n) for every pair with distance < threshold[q] to the candidate lists."""
    M, K = q.shape
    Nn = x.shape[0]
    cap = cand_val.shape[1]
    if not q.is_cuda:
        d = scale * (q.float() @ x.float().t())
        if row_term is not None:
            d = d + row_term[:, None]
        if col_term is not None:
            d = d + col_term[None, :]
        if clamp_zero:
            d = d.clamp_min(0)
        for m in range(M):
            hit = torch.nonzero(d[m] < threshold[m]).flatten()
            c = int(cand_count[m])
            n = hit.numel()
            take = max(0, min(n, cap - c))
            cand_val[m, c:c + take] = d[m, hit[:take]]
            cand_idx[m, c:c + take] = (hit[:take] + col_offset).int()
            cand_count[m] = c + n
        return
    rc = N.cuda().afb_score_filter(
        N.ptr(q), N.ptr(x), _c_int(M), _c_int(Nn), _c_int(K), _c_int(q.stride(0)), _c_int(x.stride(0)),
        N.ptr(row_term), N.ptr(col_term), _c_float(scale), _c_int(1 if clamp_zero else 0), N.ptr(threshold),
        N.ptr(cand_val), N.ptr(cand_idx), N.ptr(cand_count), _c_int(cap), _c_long(col_offset), N.stream_ptr())
    N.check(rc, "afb_score_filter")
    N.count_launch()


def assign_argmin(x, c, col_term, scale, row_term=None, want_best: bool = True):
    """assign[m] = argmin_n (col_term[n] + scale * <x_m, c_n>); best adds row_term."""
    M, K = x.shape
    if not x.is_cuda:
        d = scale * (x.float() @ c.float().t())
        if col_term is not None:
            d = d + col_term[None, :]
        best, idx = d.min(-1)
        if row_term is not None:
            best = best + row_term
        return idx.int(), best
    assign = torch.empty((M,), dtype=torch.int32, device=x.device)
    best = torch.empty((M,), dtype=torch.float32, device=x.device) if want_best else None
    rc = N.cuda().afb_assign_argmin(N.ptr(x), N.ptr(c), _c_int(M), _c_int(c.shape[0]), _c_int(K), _c_int(x.stride(0)),
                                    _c_int(c.stride(0)), N.ptr(row_term), N.ptr(col_term), _c_float(scale),
                                    N.ptr(assign), N.ptr(best), N.stream_ptr())
    N.check(rc, "afb_assign_argmin")
    N.count_launch()
    return assign, best


def topk_select(sources: Sequence[tuple], n_queries: int, k: int, max_total: int, want_threshold: bool = True,
                overflow: Optional[torch.Tensor] = None, push=None, wait=None, src_flags=None):
    """sources: (vals [Q, stride], idxs [Q, stride], counts [Q] or None, fixed_len).  Tensors may live on peer GPUs
    (any address this device can read).  Returns (top_val [Q, k] ascending, top_idx [Q, k], thr [Q], overflow).

    overflow: an int32 [1] tensor to set (never cleared) instead of a fresh one -- one sticky word per search.
    push: (vals, ids, flags, counters) ctypes pointer arrays of the ranks that also receive the result (the push
    half of the sharded merge); the pushed flag is this call's overflow OR the sticky word's value on entry.
    wait: (counter tensor, target) -- the merge half waits, bounded, for the counter before reading the sources.
    src_flags: per source an int32 [Q] tensor whose non-zero entries are OR-ed into overflow."""
    dev = sources[0][0].device
    if dev.type != "cuda":
        vals, idxs = [], []
        flag = 0
        for si, (v, ix, cnt, fl) in enumerate(sources):
            for_q_v, for_q_i = [], []
            if cnt is not None and bool((cnt[:n_queries] > fl).any()):
                flag = 1            # a producer counted more candidates than its buffer holds
            if src_flags is not None and src_flags[si] is not None and bool((src_flags[si][:n_queries] != 0).any()):
                flag = 1
            for qi in range(n_queries):
                n = min(int(cnt[qi]), fl) if cnt is not None else fl
                for_q_v.append(v[qi, :n]); for_q_i.append(ix[qi, :n])
            vals.append(for_q_v); idxs.append(for_q_i)
        out_v = torch.full((n_queries, k), float("inf"))
        out_i = torch.full((n_queries, k), -1, dtype=torch.int32)
        thr = torch.full((n_queries,), float("inf"))
        for qi in range(n_queries):
            v = torch.cat([s[qi] for s in vals]); ix = torch.cat([s[qi] for s in idxs])
            if v.numel():
                order = torch.tensor(sorted(range(v.numel()), key=lambda j: (float(v[j]), int(ix[j]))))[:k]
                out_v[qi, :order.numel()] = v[order]
                out_i[qi, :order.numel()] = ix[order].int()
                if v.numel() >= k:
                    thr[qi] = out_v[qi, k - 1]
        if overflow is not None:
            if flag:
                overflow.fill_(1)
            return out_v, out_i, thr, overflow
        return out_v, out_i, thr, flag
    n = len(sources)
    PF, PI = ctypes.c_void_p * n, ctypes.c_void_p * n
    vals = PF(*[s[0].data_ptr() for s in sources])
    idxs = PI(*[s[1].data_ptr() for s in sources])
    counts = PI(*[(s[2].data_ptr() if s[2] is not None else 0) for s in sources])
    stride = (ctypes.c_long * n)(*[s[0].stride(0) for s in sources])
    fixed = (ctypes.c_int * n)(*[int(s[3]) for s in sources])
    out_v = torch.empty((n_queries, k), dtype=torch.float32, device=dev)
    out_i = torch.empty((n_queries, k), dtype=torch.int32, device=dev)
    thr = torch.empty((n_queries,), dtype=torch.float32, device=dev) if want_threshold else None
    ovf = overflow if overflow is not None else torch.zeros((1,), dtype=torch.int32, device=dev)
    n_push = len(push[0]) if push is not None else 0
    null = ctypes.c_void_p(0)
    flags = PI(*[(f.data_ptr() if f is not None else 0) for f in src_flags]) if src_flags is not None else null
    rc = N.cuda().afb_topk_select_x(
        vals, idxs, counts, stride, fixed, _c_int(n), _c_int(n_queries), _c_int(k), _c_int(max_total), N.ptr(out_v),
        N.ptr(out_i), N.ptr(thr), N.ptr(ovf), push[0] if push else null, push[1] if push else null,
        push[2] if push else null, push[3] if push else null, _c_int(n_push),
        N.ptr(overflow) if (push is not None and overflow is not None) else null,
        N.ptr(wait[0]) if wait is not None else null, _c_int(int(wait[1]) if wait is not None else 0), flags,
        N.stream_ptr())
    N.check(rc, "afb_topk_select")
    N.count_launch()
    return out_v, out_i, thr, ovf


def kmeans_accumulate(x, assign, sums, counts) -> None:
    if not x.is_cuda:
        sums.index_add_(0, assign.long(), x.float())
        counts += torch.bincount(assign.long(), minlength=counts.numel()).to(counts.dtype)
        return
    rc = N.cuda().afb_kmeans_accumulate(N.ptr(x), _c_long(x.stride(0)), N.ptr(assign), N.ptr(sums), N.ptr(counts),
                                        _c_int(x.shape[0]), _c_int(x.shape[1]), _c_int(sums.shape[0]), N.stream_ptr())
    N.check(rc, "afb_kmeans_accumulate")
    N.count_launch()


def kmeans_finalize(sums, counts, cent_f32, cent_bf16, cent_sqnorm, shift, normalize: bool) -> None:
    if not sums.is_cuda:
        n = counts.float().clamp_min(1)[:, None]
        new = sums / n
        if normalize:
            new = torch.nn.functional.normalize(new, dim=-1)
        new = torch.where((counts > 0)[:, None], new, cent_f32)
        shift += (new - cent_f32).pow(2).sum()
        cent_f32.copy_(new)
        cent_bf16.copy_(new.to(torch.bfloat16))
        cent_sqnorm.copy_(cent_bf16.float().pow(2).sum(-1))
        return
    rc = N.cuda().afb_kmeans_finalize(N.ptr(sums), N.ptr(counts), N.ptr(cent_f32), N.ptr(cent_bf16),
                                      N.ptr(cent_sqnorm), N.ptr(shift), _c_int(sums.shape[0]), _c_int(sums.shape[1]),
                                      _c_int(1 if normalize else 0), N.stream_ptr())
    N.check(rc, "afb_kmeans_finalize")
    N.count_launch()


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return x[idx.long().clamp_min(0)]
    out = torch.empty((idx.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    rc = N.cuda().afb_gather_rows(N.ptr(x), _c_long(x.stride(0)), N.ptr(idx), N.ptr(out), _c_int(idx.numel()),
                                  _c_int(x.shape[1]), _c_long(x.shape[0]), N.stream_ptr())
    N.check(rc, "afb_gather_rows")
    N.count_launch()
    return out


def ivf_scan(x, col_term, q, row_term, threshold, list_off, pair_off, pair_query, cand_val, cand_idx, cand_count,
             scale: float, clamp_zero: bool) -> None:
    """Grouped scoring of posting lists: for every list l, the rows x[list_off[l] : list_off[l + 1]] against the
    queries pair_query[pair_off[l] : pair_off[l + 1]]; pairs with distance < threshold[query] (all pairs when
    threshold is None) are appended as (distance, row) to the query's candidate list.  One launch, no host
    synchronisation; cand_count may end above the capacity (the select that follows reports it)."""
    n_lists = list_off.numel() - 1
    cap = cand_val.shape[1]
    if not x.is_cuda:
        lo_h, po_h, pq_h = list_off.tolist(), pair_off.tolist(), pair_query.tolist()
        for l in range(n_lists):
            a, b = lo_h[l], lo_h[l + 1]
            if b <= a or po_h[l + 1] <= po_h[l]:
                continue
            rows = x[a:b].float()
            for qi in pq_h[po_h[l]:po_h[l + 1]]:
                if qi < 0:
                    continue
                d = scale * (rows @ q[qi].float())
                if row_term is not None:
                    d = d + row_term[qi]
                if col_term is not None:
                    d = d + col_term[a:b]
                if clamp_zero:
                    d = d.clamp_min(0)
                hit = torch.nonzero(d < threshold[qi]).flatten() if threshold is not None else torch.arange(b - a)
                c = int(cand_count[qi])
                take = max(0, min(hit.numel(), cap - c))
                cand_val[qi, c:c + take] = d[hit[:take]]
                cand_idx[qi, c:c + take] = (hit[:take] + a).int()
                cand_count[qi] = c + hit.numel()
        return
    rc = N.cuda().afb_ivf_scan(
        N.ptr(x), _c_long(x.stride(0)), N.ptr(col_term), N.ptr(q), _c_long(q.stride(0)), N.ptr(row_term),
        N.ptr(threshold), N.ptr(list_off), N.ptr(pair_off), N.ptr(pair_query), N.ptr(cand_val), N.ptr(cand_idx),
        N.ptr(cand_count), _c_int(n_lists), _c_int(q.shape[0]), _c_int(pair_query.numel()), _c_long(x.shape[0]),
        _c_int(x.shape[1]), _c_int(cap), _c_float(scale), _c_int(1 if clamp_zero else 0), N.stream_ptr())
    N.check(rc, "afb_ivf_scan")
    N.count_launch()
