"""Dense-layer ops backed by the sm_100a kernels: bf16 GEMM with fused epilogues, LayerNorm / RMSNorm with
fused residual and partial-sum reduction, embedding lookups, pooling.

CUDA tensors always run the kernels, launched on the current stream so the calls can be captured in a CUDA
graph; a missing kernel library on a GPU machine is an error, never a silent fallback.  CPU tensors run the
fp32 oracle of :mod:`antfly_b200.ops.reference` (the path the CPU-only tests and the CPU baseline use).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native as N
from . import reference as R

ACT = {None: 0, "none": 0, "gelu": 1, "gelu_erf": 1, "gelu_tanh": 2, "gelu_new": 2, "relu": 3, "silu": 4,
       "quick_gelu": 5}

GATE_ACT = {"gelu": 1, "gelu_erf": 1, "gelu_tanh": 2, "gelu_new": 2, "gelu_pytorch_tanh": 2, "relu": 3, "silu": 4,
            "swish": 4, "quick_gelu": 5, "relu2": 6}

_c_int = ctypes.c_int
_c_long = ctypes.c_long
_c_float = ctypes.c_float


def _bf16(t: torch.Tensor) -> torch.Tensor:
    assert t.dtype == torch.bfloat16 and t.is_cuda, "expected a CUDA bf16 tensor"
    return t


def gated_act(gu: torch.Tensor, act: str = "silu", interleaved: bool = False, limit: float = 0.0,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(gate) * up`` -> [T, F] (in the input's dtype) from the [T, 2F] output of a fused gate / up projection: halves
    (gate = columns [0, F), up = [F, 2F)) or ``interleaved`` (gate_j, up_j adjacent).  One elementwise kernel
    (csrc/kernels/gated_act.cu) instead of a chain of tensor ops; ``limit`` > 0 clamps gate from above and up to
    [-limit, limit] first (clamped SwiGLU)."""
    T, F2 = gu.shape
    F = F2 // 2
    if not gu.is_cuda or gu.dtype != torch.bfloat16:
        y = R.gated_act(gu, act, interleaved, limit).to(gu.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    gu = _bf16(gu)
    if gu.stride(1) != 1:
        gu = gu.contiguous()
    if out is None:
        out = torch.empty((T, F), dtype=torch.bfloat16, device=gu.device)
    assert out.stride(1) == 1 and out.shape == (T, F)
    up = gu if interleaved else gu[:, F:]
    rc = N.cuda().afb_gated_act(N.ptr(gu), N.ptr(up), N.ptr(out), _c_long(gu.stride(0)), _c_long(out.stride(0)),
                                _c_long(T), _c_int(F), _c_int(GATE_ACT[act]), _c_int(1 if interleaved else 0),
                                _c_float(limit), N.stream_ptr())
    N.check(rc, "afb_gated_act")
    N.count_launch()
    return out


def gemm_bf16(
    a: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    act: Optional[str] = None,
    residual: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    split_k: int = 1,
    alpha: float = 1.0,
    tile_n: int = 0,
) -> torch.Tensor:
    """``act(alpha * a @ w.T + bias) + residual`` on tcgen05 tensor cores.

    ``a`` is [M, K] and ``w`` is [N, K] (an ``nn.Linear`` weight), both bf16 with unit inner stride.  With
    ``split_k > 1`` the result is the fp32 partial stack ``[splits, M, N]`` (no bias / activation / residual),
    to be summed by the consumer (e.g. :func:`norm` with ``partials=``).
    """
    if not a.is_cuda:
        y = R.linear(a, w, bias, act, residual, alpha)
        if split_k > 1:
            return y[None]
        return y.to(out_dtype)
    _bf16(a), _bf16(w)
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1]
    assert a.stride(1) == 1 and w.stride(1) == 1
    M, K = a.shape
    Nn = w.shape[0]
    if (split_k <= 1 and tile_n == 0 and K <= 1536 and ((M + 127) // 128) * ((Nn + 255) // 256) >= 296
            and (out is None or out.dim() == 2)):
        # Many tiles with a short K loop: the persistent kernel overlaps each tile's epilogue with the next
        # tile's MMAs (measured 15-25 % faster on the encoder shapes).
        from .index_ops import gemm_persistent

        return gemm_persistent(a, w, bias, act, residual, out, out_dtype, alpha)
    lib = N.cuda()
    splits = int(lib.afb_gemm_effective_splits(_c_int(K), _c_int(split_k))) if split_k > 1 else 1
    if splits > 1:
        assert bias is None and act in (None, "none") and residual is None
        if out is None:
            out = torch.empty((splits, M, Nn), dtype=torch.float32, device=a.device)
        out_f32 = 1
        ldc = Nn
    else:
        if out is None:
            out = torch.empty((M, Nn), dtype=out_dtype, device=a.device)
        out_f32 = 1 if out.dtype == torch.float32 else 0
        ldc = out.stride(0) if out.dim() == 2 else Nn
    ldr = residual.stride(0) if residual is not None else 0
    rc = lib.afb_gemm_bf16(
        N.ptr(a), N.ptr(w), N.ptr(out), N.ptr(bias), N.ptr(residual),
        _c_int(M), _c_int(Nn), _c_int(K), _c_int(a.stride(0)), _c_int(w.stride(0)), _c_int(ldc), _c_int(ldr),
        _c_int(ACT[act]), _c_int(out_f32), _c_int(splits), _c_float(alpha), _c_int(tile_n), N.stream_ptr(),
    )
    N.check(rc, "afb_gemm_bf16")
    N.count_launch()
    return out


def norm(
    x: Optional[torch.Tensor],
    gamma: torch.Tensor,
    beta: Optional[torch.Tensor] = None,
    *,
    eps: float = 1e-5,
    rms: bool = False,
    residual: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    partials: Optional[torch.Tensor] = None,
    want_sum: bool = False,
    want_norm: bool = True,
    gamma_plus_one: bool = False,
    out: Optional[torch.Tensor] = None,
    sum_out: Optional[torch.Tensor] = None,
    mx_terms: int = 0,
):
    """LayerNorm / RMSNorm of ``x + sum(partials) + bias + residual``.

    Returns ``y`` or ``(sum, y)`` when ``want_sum``.  ``partials`` is an fp32 stack [S, rows, H] as produced
    by a split-K GEMM.  With ``mx_terms`` 1 or 2 the normalised output is returned as MX-fp8 activations
    (:class:`antfly_b200.ops.quant.MxAct`) for the block-scaled GEMM instead of bf16.
    """
    src = x if x is not None else partials[0]
    rows, H = src.shape[-2], src.shape[-1]
    dev = src.device
    if not src.is_cuda:
        s_, y_ = R.norm(x, gamma, beta, eps, rms, residual, bias, partials, gamma_plus_one,
                        round_sum_bf16=want_sum)
        s_, y_ = s_.to(torch.bfloat16), y_.to(torch.bfloat16)
        if mx_terms:
            from . import quant as Q

            y_ = Q.quantize_mx(y_, terms=mx_terms)
        if want_sum and want_norm:
            return s_, y_
        return s_ if want_sum else y_
    mx = None
    if mx_terms and want_norm:
        from . import quant as Q

        mx = Q.new_mx(rows, H, mx_terms, dev)
    elif want_norm and out is None:
        out = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
    if want_sum and sum_out is None:
        sum_out = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
    nparts = 0 if partials is None else partials.shape[0]
    pstride = 0 if partials is None else partials.stride(0)
    rc = N.cuda().afb_norm(
        N.ptr(x), N.ptr(partials), _c_int(nparts), _c_long(pstride), N.ptr(residual), N.ptr(bias), N.ptr(gamma),
        N.ptr(beta), N.ptr(sum_out), N.ptr(out if (want_norm and mx is None) else None), ctypes.c_void_p(0),
        _c_int(rows), _c_int(H), _c_float(eps), _c_int(1 if rms else 0), _c_int(1 if gamma_plus_one else 0),
        N.ptr(mx.q0 if mx else None), N.ptr(mx.q1 if mx else None), N.ptr(mx.sf0 if mx else None),
        N.ptr(mx.sf1 if mx else None), N.stream_ptr(),
    )
    N.check(rc, "afb_norm")
    N.count_launch()
    y = mx if mx is not None else out
    if want_sum and want_norm:
        return sum_out, y
    return sum_out if want_sum else y


def layer_norm(x, gamma, beta, eps: float = 1e-12, residual=None):
    return norm(x, gamma, beta, eps=eps, rms=False, residual=residual)


def rms_norm(x, gamma, eps: float = 1e-5, residual=None, want_sum: bool = False):
    return norm(x, gamma, None, eps=eps, rms=True, residual=residual, want_sum=want_sum)


def bert_embed_ln(ids, positions, type_ids, word, pos, typ, gamma, beta, eps: float = 1e-12) -> torch.Tensor:
    """word[ids] + pos[positions] + typ[type_ids] followed by LayerNorm; ids are int32 [T]."""
    T = ids.numel()
    H = word.shape[1]
    if not word.is_cuda:
        return R.bert_embed_ln(ids, positions, type_ids, word, pos, typ, gamma, beta, eps).to(torch.bfloat16)
    y = torch.empty((T, H), dtype=torch.bfloat16, device=word.device)
    rc = N.cuda().afb_bert_embed_ln(
        N.ptr(ids), N.ptr(positions), N.ptr(type_ids), N.ptr(word), N.ptr(pos), N.ptr(typ), N.ptr(gamma),
        N.ptr(beta), N.ptr(y), _c_int(T), _c_int(H), _c_int(word.shape[0]), _c_int(pos.shape[0]),
        _c_int(typ.shape[0]), _c_float(eps), N.stream_ptr(),
    )
    N.check(rc, "afb_bert_embed_ln")
    N.count_launch()
    return y


def embed_gather(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0, out=None) -> torch.Tensor:
    T = ids.numel()
    H = table.shape[1]
    if not table.is_cuda:
        return (table.float()[ids.long()] * scale).to(torch.bfloat16)
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=table.device)
    rc = N.cuda().afb_embed_gather(N.ptr(ids), N.ptr(table), N.ptr(out), _c_int(T), _c_int(H),
                                   _c_int(table.shape[0]), _c_float(scale), N.stream_ptr())
    N.check(rc, "afb_embed_gather")
    N.count_launch()
    return out


POOL_MODES = {"mean": 0, "cls": 1, "max": 2, "last": 3}


def pool(h: torch.Tensor, starts: torch.Tensor, lens: torch.Tensor, mode: str = "mean", normalize: bool = True,
         mask: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pool token rows ``h`` [T, H] per document (rows starts[b] .. starts[b]+lens[b]) to fp32 [B, H]."""
    B = starts.numel()
    H = h.shape[-1]
    if not h.is_cuda:
        return R.pool(h, starts, lens, mode, normalize, mask)
    if out is None:
        out = torch.empty((B, H), dtype=torch.float32, device=h.device)
    rc = N.cuda().afb_pool(N.ptr(h), N.ptr(starts), N.ptr(lens), N.ptr(mask), N.ptr(out), _c_int(B), _c_int(H),
                           _c_int(POOL_MODES[mode]), _c_int(1 if normalize else 0), N.stream_ptr())
    N.check(rc, "afb_pool")
    N.count_launch()
    return out


def maxsim(q: torch.Tensor, d: torch.Tensor, starts: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
    """ColBERT MaxSim of one query [nq, D] against packed document token embeddings [T, D]."""
    n_docs = starts.numel()
    if not q.is_cuda:
        return R.maxsim(q, d, starts, lens)
    out = torch.empty((n_docs,), dtype=torch.float32, device=q.device)
    rc = N.cuda().afb_maxsim(N.ptr(q), _c_int(q.shape[0]), N.ptr(d), N.ptr(starts), N.ptr(lens), N.ptr(out),
                             _c_int(n_docs), _c_int(q.shape[1]), N.stream_ptr())
    N.check(rc, "afb_maxsim")
    N.count_launch()
    return out


def splade_pool(logits: torch.Tensor, starts: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
    B = starts.numel()
    V = logits.shape[-1]
    if not logits.is_cuda:
        return R.splade_pool(logits, starts, lens)
    out = torch.empty((B, V), dtype=torch.float32, device=logits.device)
    rc = N.cuda().afb_splade_pool(N.ptr(logits), N.ptr(starts), N.ptr(lens), N.ptr(out), _c_int(B), _c_int(V),
                                  N.stream_ptr())
    N.check(rc, "afb_splade_pool")
    N.count_launch()
    return out
