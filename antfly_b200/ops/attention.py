"""Attention and rotary ops: packed varlen encoder attention, paged-KV prefill/decode attention, fused
QKV -> (head-norm, RoPE, KV-cache write).  CUDA tensors run the sm_100a kernels; CPU tensors run the fp32 oracle.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from .. import _native as N
from . import reference as R

_c_int = ctypes.c_int
_c_long = ctypes.c_long
_c_float = ctypes.c_float


# The tcgen05 / tensor-memory flash kernel (csrc/kernels/attention_tc.cu) serves the compute-bound shapes -- encoder
# attention and paged prefill with 64- or 128-wide heads -- when it is switched on: ANTFLY_B200_ATTN_TC=1 in the
# environment or set_tensor_core_attention(True).  It is off by default until it has been validated on the
# hardware it runs on; the mma.sync kernel in attention.cu is the default and the fallback.
_TC = {"on": None}


def tensor_core_attention_enabled() -> bool:
    if _TC["on"] is None:
        import os

        _TC["on"] = os.environ.get("ANTFLY_B200_ATTN_TC", "0") == "1"
    return bool(_TC["on"])


def set_tensor_core_attention(on: bool) -> None:
    _TC["on"] = bool(on)


def attention_tc(q, k, v, starts, lens, kv_lens, max_q_len: int, causal: bool, window: int = 0,
                 scale: Optional[float] = None, out: Optional[torch.Tensor] = None, k_cache=None, v_cache=None,
                 block_tables=None) -> torch.Tensor:
    """Direct entry to the tensor-core flash kernel.  Contiguous mode: k / v [T, Hkv, D] views (kv_lens = lens).
    Paged mode: k_cache / v_cache [num_blocks, page, Hkv, D] + block_tables, query rows = the last lens[b]
    positions of kv_lens[b] keys.  D in (64, 128).  Raises NativeError for shapes the kernel does not take."""
    T, Hq, D = q.shape
    paged = k_cache is not None
    Hkv = k_cache.shape[2] if paged else k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    assert q.is_cuda and q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == D
    if out is None:
        out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    if paged:
        assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
        page, nblk = k_cache.shape[1], k_cache.shape[0]
        args = (None, None, _c_long(0), N.ptr(k_cache), N.ptr(v_cache), N.ptr(block_tables),
                _c_int(block_tables.shape[1]), _c_int(page), _c_long(nblk))
    else:
        assert k.stride(2) == 1 and k.stride(1) == D and v.stride(1) == D and k.stride(0) == v.stride(0)
        args = (N.ptr(k), N.ptr(v), _c_long(k.stride(0)), None, None, None, _c_int(0), _c_int(16), _c_long(0))
    rc = N.cuda().afb_attention_tc(
        N.ptr(q), _c_long(q.stride(0)), *args, N.ptr(starts), N.ptr(lens), N.ptr(kv_lens), N.ptr(out),
        _c_long(out.stride(0)), _c_int(starts.numel()), _c_int(T), _c_int(Hq), _c_int(Hkv), _c_int(D),
        _c_int(max_q_len), _c_int(1 if causal else 0), _c_int(window), _c_float(scale), _c_int(1 if paged else 0),
        N.stream_ptr())
    N.check(rc, "afb_attention_tc")
    N.count_launch()
    return out


def varlen_attention(q, k, v, starts, lens, max_len: int, causal: bool = False, scale: Optional[float] = None,
                     out: Optional[torch.Tensor] = None, window: int = 0) -> torch.Tensor:
    """q [T, Hq, D], k/v [T, Hkv, D] (may be strided views of one fused QKV buffer); sequences are the packed
    row ranges starts[b] .. starts[b]+lens[b].  ``window`` > 0: keys with key > query - window, and for
    bidirectional attention also key < query + window."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        cu = torch.cat([starts.long(), (starts[-1:] + lens[-1:]).long()])
        return R.varlen_attention(q, k, v, cu, scale, causal, window).to(torch.bfloat16)
    if D not in (64, 128, 256):
        # The kernel is built for 64-, 128- and 256-wide heads.  Zero columns change neither a dot product nor the
        # softmax (the scale is fixed from the true width), so other widths run zero-padded to the next size
        # (vision towers with 80-wide heads, small test models); beyond 256 the tensor-op restatement runs.
        if D > 256:
            cu = torch.cat([starts.long(), (starts[-1:] + lens[-1:]).long()])
            return R.varlen_attention(q, k, v, cu, scale, causal, window).to(torch.bfloat16)
        Dp = 64 if D < 64 else 128 if D < 128 else 256
        pad = lambda t: torch.nn.functional.pad(t, (0, Dp - D)).contiguous()
        o = varlen_attention(pad(q), pad(k), pad(v), starts, lens, max_len, causal, scale, None, window)
        o = o[..., :D].contiguous()
        if out is not None:
            out.copy_(o)
            return out
        return o
    assert q.stride(2) == 1 and q.stride(1) == D and k.stride(1) == D and v.stride(1) == D
    assert k.stride(0) == v.stride(0)
    if out is None:
        out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    B = starts.numel()
    if tensor_core_attention_enabled() and D in (64, 128) and q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0 \
            and out.stride(0) % 8 == 0 and out.stride(1) == D:
        return attention_tc(q, k, v, starts, lens, lens, max_len, causal, window, scale, out)
    rc = N.cuda().afb_attention(
        N.ptr(q), _c_long(q.stride(0)), N.ptr(k), N.ptr(v), _c_long(k.stride(0)), None, None, None, _c_int(0),
        _c_int(16), N.ptr(starts), N.ptr(lens), N.ptr(lens), N.ptr(out), _c_long(out.stride(0)), None, None,
        _c_int(B), _c_int(T), _c_int(Hq), _c_int(Hkv), _c_int(D), _c_int(max_len), _c_int(1 if causal else 0),
        _c_int(window), _c_float(scale), _c_int(0), _c_int(0), _c_int(1), N.stream_ptr(),
    )
    N.check(rc, "afb_attention")
    N.count_launch()
    return out


class PagedAttnScratch:
    """Split-KV partial buffers, sized once for the largest decode batch (scratch memory reused every step)."""

    def __init__(self, max_tokens: int, Hq: int, D: int, max_splits: int, device):
        self.max_tokens, self.max_splits = max_tokens, max_splits
        self.part_o = torch.empty((max_splits, max_tokens * Hq, D), dtype=torch.float32, device=device)
        self.part_lse = torch.empty((max_splits, max_tokens * Hq), dtype=torch.float32, device=device)


def paged_attention_sink(q, k_cache, v_cache, block_tables, q_starts, q_lens, kv_lens, scale: Optional[float] = None,
                         window: int = 0, sinks: Optional[torch.Tensor] = None, softcap: float = 0.0,
                         out: Optional[torch.Tensor] = None, alibi: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal paged attention whose softmax has a per-head sink logit (``sinks`` fp32 [Hq]), a soft cap on the scaled
    scores and / or a linear position bias (``alibi`` fp32 [Hq] slopes times key position minus query position): the
    variants that change the scores or the normalisation, served by a kernel of their own
    (csrc/kernels/attention_sink.cu; one warp per (token, head)).  Same tensors as :func:`paged_attention`, bf16
    caches only."""
    T, Hq, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        return R.paged_attention(q, k_cache, v_cache, block_tables, q_starts, q_lens, kv_lens, scale, window,
                                 sinks=sinks, softcap=softcap, alibi=alibi).to(torch.bfloat16)
    if k_cache.dtype != torch.bfloat16 or q.dtype != torch.bfloat16:
        raise NotImplementedError("attention with sinks / soft cap reads bf16 queries and a bf16 KV cache")
    assert q.stride(2) == 1 and q.stride(1) == D and k_cache.is_contiguous() and v_cache.is_contiguous()
    nblk, page, Hkv = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    B = q_lens.numel()
    if out is None:
        out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    # sequence of every query row (q_starts ascends; rows past the last sequence's own fail the kernel's range check
    # and come back as zeros)
    token_seq = (torch.searchsorted(q_starts.int(), torch.arange(T, dtype=torch.int32, device=q.device), right=True)
                 - 1).clamp_min(0).int()
    sk = sinks.float().contiguous() if sinks is not None else None
    al = alibi.float().contiguous() if alibi is not None else None
    rc = N.cuda().afb_attention_sink(
        N.ptr(q), _c_long(q.stride(0)), N.ptr(k_cache), N.ptr(v_cache), N.ptr(block_tables),
        _c_int(block_tables.shape[1]), _c_int(page), _c_int(nblk), N.ptr(token_seq), N.ptr(q_starts), N.ptr(q_lens),
        N.ptr(kv_lens), N.ptr(sk), N.ptr(al), N.ptr(out), _c_long(out.stride(0)), _c_int(B), _c_int(T), _c_int(Hq), _c_int(Hkv),
        _c_int(D), _c_int(window), _c_float(scale), _c_float(softcap), N.stream_ptr())
    N.check(rc, "afb_attention_sink")
    N.count_launch()
    return out


def paged_attention(q, k_cache, v_cache, block_tables, q_starts, q_lens, kv_lens, max_q_len: int,
                    scale: Optional[float] = None, window: int = 0, decode: Optional[bool] = None,
                    num_splits: int = 1, scratch: Optional[PagedAttnScratch] = None,
                    out: Optional[torch.Tensor] = None, mx_terms: int = 0, causal: bool = True, max_kv: int = 0):
    """Causal attention (``causal=False``: every query row of a sequence sees all of its ``kv_lens`` keys, within a
    two-sided ``window`` if one is set) of packed query tokens q [T, Hq, D] against the paged cache
    k_cache / v_cache [num_blocks, page, Hkv, D].  ``decode`` selects the split-keys organisation (<= 16
    (position, head-in-group) rows per KV head); default: when max_q_len * group <= 16.
    ``k_cache`` / ``v_cache`` may also be :class:`antfly_b200.ops.kv_quant.CodecLayer` objects (a cache kept in a
    quantised codec); ``max_kv`` (the largest ``kv_lens`` entry, known on the host) then bounds the pages that a
    prefill step expands.
    ``mx_terms`` 1 or 2 returns the context rows [T, Hq * D] as MX-fp8 activations
    (:class:`antfly_b200.ops.quant.MxAct`) for the output projection: emitted by the split merge kernel when the
    KV range is split, by a quantisation pass otherwise."""
    T, Hq, D = q.shape
    from .kv_quant import CodecLayer

    if isinstance(k_cache, CodecLayer):
        return _paged_attention_codec(q, k_cache, v_cache, block_tables, q_starts, q_lens, kv_lens, max_q_len, scale,
                                      window, decode, num_splits, scratch, out, mx_terms, causal, max_kv)
    page, Hkv = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        y = R.paged_attention(q, k_cache, v_cache, block_tables, q_starts, q_lens, kv_lens, scale,
                              window, causal=causal).to(torch.bfloat16)
        if mx_terms:
            from . import quant as Q

            return Q.quantize_mx(y.reshape(T, Hq * D), terms=mx_terms)
        return y
    if k_cache.dtype != torch.bfloat16:
        raise NotImplementedError("this entry reads a bf16 KV cache; quantised caches are passed as CodecLayer "
                                  "objects (ops.kv_quant)")
    if D not in (64, 128, 256):
        # Head widths the tensor-core kernels are not built for (80 / 96-wide heads of some small decoders): the
        # general one-warp-per-row kernel reads the cache at its own width.
        if not causal or D % 8 or D > 256:
            raise NotImplementedError(f"paged attention needs a head width that is a multiple of 8 up to 256 "
                                      f"(non-causal: 64, 128 or 256); got {D}")
        y = paged_attention_sink(q, k_cache, v_cache, block_tables, q_starts, q_lens, kv_lens, scale=scale,
                                 window=window, out=out)
        if mx_terms:
            from . import quant as Q

            return Q.quantize_mx(y.reshape(T, Hq * D), terms=mx_terms)
        return y
    G = Hq // Hkv
    if decode is None:
        decode = max_q_len * G <= 16
    if not decode:
        num_splits = 1
        if (tensor_core_attention_enabled() and causal and D in (64, 128) and page % 8 == 0
                and (128 if D == 64 else 64) % page == 0 and q.stride(0) % 8 == 0 and k_cache.is_contiguous()
                and v_cache.is_contiguous()):
            o = attention_tc(q, None, None, q_starts, q_lens, kv_lens, max_q_len, True, window, scale, out,
                             k_cache=k_cache, v_cache=v_cache, block_tables=block_tables)
            if mx_terms:
                from . import quant as Q

                return Q.quantize_mx(o.view(T, Hq * D), terms=mx_terms)
            return o
    mx = None
    if mx_terms and num_splits > 1 and (Hq * D) % 128 == 0:
        from . import quant as Q

        mx = Q.new_mx(T, Hq * D, mx_terms, q.device)
    elif out is None:
        out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    part_o = part_lse = None
    if num_splits > 1:
        if scratch is None:
            scratch = PagedAttnScratch(T, Hq, D, num_splits, q.device)
        assert scratch.max_splits >= num_splits and scratch.part_lse.shape[1] >= T * Hq
        part_o, part_lse = scratch.part_o, scratch.part_lse
    B = q_starts.numel()
    rc = N.cuda().afb_attention_mx(
        N.ptr(q), _c_long(q.stride(0)), None, None, _c_long(0), N.ptr(k_cache), N.ptr(v_cache),
        N.ptr(block_tables), _c_int(block_tables.shape[1]), _c_int(page), N.ptr(q_starts), N.ptr(q_lens),
        N.ptr(kv_lens), N.ptr(out), _c_long(out.stride(0) if out is not None else Hq * D), N.ptr(part_o),
        N.ptr(part_lse), _c_int(B), _c_int(T), _c_int(Hq), _c_int(Hkv), _c_int(D), _c_int(max_q_len),
        _c_int(1 if causal else 0), _c_int(window), _c_float(scale), _c_int(1), _c_int(1 if decode else 0), _c_int(num_splits),
        N.ptr(mx.q0 if mx else None), N.ptr(mx.q1 if mx else None), N.ptr(mx.sf0 if mx else None),
        N.ptr(mx.sf1 if mx else None), N.stream_ptr(),
    )
    N.check(rc, "afb_attention")
    N.count_launch(2 if num_splits > 1 else 1)
    if mx is not None:
        return mx
    if mx_terms:
        from . import quant as Q

        return Q.quantize_mx(out.view(T, Hq * D), terms=mx_terms)
    return out


def _paged_attention_codec(q, kl, vl, block_tables, q_starts, q_lens, kv_lens, max_q_len, scale, window, decode,
                           num_splits, scratch, out, mx_terms, causal, max_kv):
    """Attention over a cache kept in a quantised codec (fp8 / int8 / int4 / polar4 / turbo3).

    * One new token per sequence: keys are scored straight from their codes.  An fp8 cache on the GPU takes the
      tensor-core decode kernel with the codes expanded in shared memory (``afb_attention_kv8``); the other codecs
      take the code-scoring kernel of ``attention_kvq.cu``.
    * Several query rows per sequence (prefill chunks, speculative verification): the pages the step can see are
      expanded to a bf16 scratch with a block table of its own and the bf16 kernels run on that; the cache itself
      stays compressed.  (turbo3 keys expand to their 3-bit base values.)
    """
    from . import kv_quant as KQ

    T, Hq, D = q.shape
    Hkv, page, codec = kl.Hkv, kl.page, kl.codec
    B = q_starts.numel()
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    G = Hq // Hkv
    single = max_q_len == 1 and T == B and causal
    ctx = None
    if single and q.is_cuda and codec == "fp8" and G <= 8 and D in (64, 128, 256):
        mx = None
        if mx_terms and num_splits > 1 and (Hq * D) % 128 == 0:
            from . import quant as Q

            mx = Q.new_mx(T, Hq * D, mx_terms, q.device)
        elif out is None:
            out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
        part_o = part_lse = None
        if num_splits > 1:
            if scratch is None:
                scratch = PagedAttnScratch(T, Hq, D, num_splits, q.device)
            part_o, part_lse = scratch.part_o, scratch.part_lse
        rc = N.cuda().afb_attention_kv8(
            N.ptr(q), _c_long(q.stride(0)), N.ptr(kl.data), N.ptr(vl.data), N.ptr(block_tables),
            _c_int(block_tables.shape[1]), _c_int(page), N.ptr(q_starts), N.ptr(q_lens), N.ptr(kv_lens), N.ptr(out),
            _c_long(out.stride(0) if out is not None else Hq * D), N.ptr(part_o), N.ptr(part_lse), _c_int(B),
            _c_int(T), _c_int(Hq), _c_int(Hkv), _c_int(D), _c_int(1), _c_int(window), _c_float(scale), _c_float(1.0),
            _c_float(1.0), _c_int(num_splits), N.ptr(mx.q0 if mx else None), N.ptr(mx.q1 if mx else None),
            N.ptr(mx.sf0 if mx else None), N.ptr(mx.sf1 if mx else None), N.stream_ptr())
        N.check(rc, "afb_attention_kv8")
        N.count_launch(2 if num_splits > 1 else 1)
        if mx is not None:
            return mx
        ctx = out
    elif single and (not q.is_cuda or G <= 8):
        ctx = KQ.decode_attention(codec, q.contiguous(), kl.data, vl.data, block_tables, kv_lens, Hkv, scale,
                                  window=window, out=out)
    if ctx is None:
        nb = block_tables.shape[1]
        if max_kv > 0:
            nb = min(nb, (max_kv + page - 1) // page)
        tab = block_tables[:, :nb]
        rows = (tab.long().clamp_min(0) * page)[:, :, None] + torch.arange(page, device=tab.device)[None, None, :]
        rows = rows.reshape(-1).int()
        kb = kl.expand(rows).view(B * nb, page, Hkv, D)
        vb = vl.expand(rows).view(B * nb, page, Hkv, D)
        new_tab = torch.arange(B * nb, dtype=torch.int32, device=tab.device).view(B, nb)
        return paged_attention(q, kb, vb, new_tab, q_starts, q_lens, kv_lens, max_q_len, scale, window, decode,
                               num_splits, scratch, out, mx_terms, causal)
    if mx_terms:
        from . import quant as Q

        return Q.quantize_mx(ctx.reshape(T, Hq * D), terms=mx_terms)
    return ctx


def rope_kv_write(qkv: Optional[torch.Tensor], positions, slots, k_cache, v_cache, Hq: int, Hkv: int, D: int,
                  theta: float, *, partials: Optional[torch.Tensor] = None, bias=None, rope_dim: Optional[int] = None,
                  half_split: bool = True, freq_scale: float = 1.0, q_norm_w=None, k_norm_w=None,
                  norm_eps: float = 1e-6, norm_plus_one: bool = False, q_out: Optional[torch.Tensor] = None,
                  kv_scale: float = 1.0, inv_freq: Optional[torch.Tensor] = None,
                  rope_mscale: float = 1.0) -> torch.Tensor:
    """Takes fused QKV rows (bf16, or fp32 split-K partials), applies optional head RMS-norm and RoPE to Q and
    K, writes K/V into the cache at ``slots`` and returns Q [T, Hq, D] bf16.  ``inv_freq`` (fp32 [rope_dim / 2] on
    the tensors' device) replaces the closed-form frequencies and ``rope_mscale`` then scales cos / sin."""
    src = qkv if qkv is not None else partials[0]
    T = src.shape[0]
    rd = rope_dim or D
    from .kv_quant import CodecLayer

    if isinstance(k_cache, CodecLayer):
        if k_cache.codec == "fp8" and src.is_cuda:
            # e4m3 rows are exactly the [Hkv, D] byte layout the kernel's fp8 store writes: no staging
            k_cache, v_cache = k_cache.data, v_cache.data
        else:
            # rotate / normalise into a bf16 staging "cache" of T single-token rows, then encode into the codec
            ks = torch.zeros((1, T, Hkv, D), dtype=torch.float32 if not src.is_cuda else torch.bfloat16,
                             device=src.device)
            vs = torch.zeros_like(ks)
            q_res = rope_kv_write(qkv, positions, torch.arange(T, dtype=torch.int32, device=src.device), ks, vs, Hq,
                                  Hkv, D, theta, partials=partials, bias=bias, rope_dim=rope_dim,
                                  half_split=half_split, freq_scale=freq_scale, q_norm_w=q_norm_w, k_norm_w=k_norm_w,
                                  norm_eps=norm_eps, norm_plus_one=norm_plus_one, q_out=q_out, inv_freq=inv_freq,
                                  rope_mscale=rope_mscale)
            k_cache.write(slots, ks[0])
            v_cache.write(slots, vs[0])
            return q_res
    if not src.is_cuda:
        row = (qkv.float() if qkv is not None else 0) + (partials.float().sum(0) if partials is not None else 0)
        if bias is not None:
            row = row + bias.float()
        row = row.reshape(T, Hq + 2 * Hkv, D)
        qh, kh, vh = row[:, :Hq], row[:, Hq:Hq + Hkv], row[:, Hq + Hkv:]
        if q_norm_w is not None:
            qh = R.norm(qh, q_norm_w, eps=norm_eps, rms=True, gamma_plus_one=norm_plus_one, round_sum_bf16=False)[1]
        if k_norm_w is not None:
            kh = R.norm(kh, k_norm_w, eps=norm_eps, rms=True, gamma_plus_one=norm_plus_one, round_sum_bf16=False)[1]
        qh = R.rope(qh, positions, theta, rd, half_split, freq_scale, inv_freq, rope_mscale)
        kh = R.rope(kh, positions, theta, rd, half_split, freq_scale, inv_freq, rope_mscale)
        kc = k_cache.view(-1, Hkv, D)
        vc = v_cache.view(-1, Hkv, D)
        ok = slots >= 0
        kc[slots[ok].long()] = kh[ok].to(kc.dtype)
        vc[slots[ok].long()] = vh[ok].to(vc.dtype)
        return qh.to(torch.bfloat16)
    if q_out is None:
        q_out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=src.device)
    nparts = 0 if partials is None else partials.shape[0]
    pstride = 0 if partials is None else partials.stride(0)
    kv_fp8 = 1 if k_cache.dtype in (torch.float8_e4m3fn, torch.uint8) else 0
    num_slots = k_cache.shape[0] * k_cache.shape[1]
    args = (
        N.ptr(qkv), N.ptr(partials), _c_int(nparts), _c_long(pstride), N.ptr(bias), N.ptr(positions), N.ptr(slots),
        N.ptr(q_norm_w), N.ptr(k_norm_w), N.ptr(q_out), N.ptr(k_cache), N.ptr(v_cache), _c_int(T), _c_int(Hq),
        _c_int(Hkv), _c_int(D), _c_int(rd), _c_int(1 if half_split else 0), _c_float(theta), _c_float(freq_scale),
        _c_float(norm_eps), _c_int(1 if norm_plus_one else 0), _c_int(kv_fp8), _c_float(kv_scale),
        _c_long(num_slots))
    if inv_freq is None:
        rc = N.cuda().afb_rope_kv_write(*args, N.stream_ptr())
    else:
        assert inv_freq.dtype == torch.float32 and inv_freq.is_cuda and inv_freq.numel() == rd // 2
        rc = N.cuda().afb_rope_kv_write_x(*args, N.ptr(inv_freq), _c_float(rope_mscale), N.stream_ptr())
    N.check(rc, "afb_rope_kv_write")
    N.count_launch()
    return q_out


def rope_(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: Optional[int] = None,
          half_split: bool = True, freq_scale: float = 1.0) -> torch.Tensor:
    """In-place RoPE on x [T, heads, D] bf16; x may be a view whose token rows are further apart than heads * D
    (the Q and K heads inside a fused QKV buffer)."""
    T, Hh, D = x.shape
    rd = rope_dim or D
    if not x.is_cuda:
        x.copy_(R.rope(x, positions, theta, rd, half_split, freq_scale).to(x.dtype))
        return x
    assert x.stride(2) == 1 and x.stride(1) == D
    rc = N.cuda().afb_rope_inplace_strided(N.ptr(x), N.ptr(positions), _c_int(T), _c_int(Hh), _c_int(D), _c_int(rd),
                                           _c_int(1 if half_split else 0), _c_float(theta), _c_float(freq_scale),
                                           _c_long(x.stride(0)), N.stream_ptr())
    N.check(rc, "afb_rope_inplace")
    N.count_launch()
    return x


def kv_copy_blocks(k_cache, v_cache, src: torch.Tensor, dst: torch.Tensor) -> None:
    """Copy whole cache blocks src[i] -> dst[i] (copy-on-write of shared prefix blocks)."""
    n = src.numel()
    if n == 0:
        return
    if not k_cache.is_cuda:
        k_cache[dst.long()] = k_cache[src.long()]
        v_cache[dst.long()] = v_cache[src.long()]
        return
    block_bytes = k_cache[0].numel() * k_cache.element_size()
    rc = N.cuda().afb_kv_copy_blocks(N.ptr(k_cache), N.ptr(v_cache), N.ptr(src), N.ptr(dst), _c_int(n),
                                     _c_long(block_bytes), N.stream_ptr())
    N.check(rc, "afb_kv_copy_blocks")
    N.count_launch()
