"""Block-scaled fp8 weights: packing and the W8A16 tcgen05 GEMM.

A packed weight is ``(q, scales)``: ``q`` [N, K] e4m3 bytes and ``scales`` [K/32, N] e8m0 exponent bytes (one
power-of-two scale per 32 consecutive K elements of a row -- the MX block format).  Activations stay bf16.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N
from . import reference as R
from .dense import ACT

_c_int = ctypes.c_int


@dataclass
class Fp8Weight:
    q: torch.Tensor        # [N, K] float8_e4m3fn (or uint8 view)
    scales: torch.Tensor   # [K/32, N] uint8
    interleaved_swiglu: bool = False

    @property
    def out_features(self) -> int:
        return self.q.shape[0]

    @property
    def in_features(self) -> int:
        return self.q.shape[1]

    def to(self, device) -> "Fp8Weight":
        return Fp8Weight(self.q.to(device), self.scales.to(device), self.interleaved_swiglu)

    def nbytes(self) -> int:
        return self.q.numel() + self.scales.numel()


def pack_fp8(w: torch.Tensor) -> Fp8Weight:
    """Quantise an [N, K] weight to block-scaled e4m3 (K padded to a multiple of 32 is the caller's job)."""
    q, e8 = R.quantize_block_fp8(w)
    return Fp8Weight(q.contiguous(), e8.contiguous())


def pack_fp8_swiglu(gate: torch.Tensor, up: torch.Tensor) -> Fp8Weight:
    """Interleave gate/up rows (row 2i = gate_i, row 2i+1 = up_i) so the GEMM epilogue can apply SwiGLU."""
    w = torch.stack([gate, up], dim=1).reshape(-1, gate.shape[1])
    p = pack_fp8(w)
    p.interleaved_swiglu = True
    return p


def random_fp8(n: int, k: int, device, seed: int = 0, interleaved_swiglu: bool = False) -> Fp8Weight:
    """Random-init packed weight drawn directly in the quantised domain (no fp32 master copy), for benchmarks
    of model sizes whose fp32 weights would not be worth materialising.  Values are uniform random e4m3 bytes
    with exponent limited so |w| <= 1.75, scale exponent chosen so the dequantised std is ~ k^-0.5."""
    g = torch.Generator(device=device).manual_seed(seed)
    # e4m3: sign(1) exp(4) mant(3); keep exponent field in [0, 7] -> |v| < 2.
    b = torch.randint(0, 64, (n, k), generator=g, device=device, dtype=torch.uint8)
    sign = torch.randint(0, 2, (n, k), generator=g, device=device, dtype=torch.uint8) << 7
    q = (b | sign).view(torch.float8_e4m3fn)
    import math

    # uniform over those codes has std ~0.6; target std k^-0.5
    e = int(round(math.log2((k ** -0.5) / 0.6)))
    scales = torch.full((k // 32, n), 127 + e, dtype=torch.uint8, device=device)
    return Fp8Weight(q, scales, interleaved_swiglu)


def gemm_w8a16(
    x: torch.Tensor,
    w: Fp8Weight,
    bias: Optional[torch.Tensor] = None,
    act: Optional[str] = None,
    residual: Optional[torch.Tensor] = None,
    split_k: int = 1,
    swiglu: bool = False,
    out: Optional[torch.Tensor] = None,
    partials: bool = False,
) -> torch.Tensor:
    """``x @ dequant(w).T`` with bf16 activations.  ``partials=True`` (or split_k > 1) returns fp32
    [splits, M, N]; ``swiglu=True`` needs an interleaved gate/up weight and returns [M, N/2]."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    M, K = x.shape
    Nn = w.out_features
    assert K == w.in_features
    if not x.is_cuda:
        y = R.linear_w8(x, w.q, w.scales, bias, None if swiglu else act, None if swiglu else residual)
        if swiglu:
            return R.swiglu_interleaved(y).to(torch.bfloat16)
        if partials or split_k > 1:
            return y[None]
        return y.to(torch.bfloat16)
    lib = N.cuda()
    if split_k > 1 or partials:
        splits = int(lib.afb_gemm_effective_splits(_c_int(K), _c_int(max(split_k, 1))))
        mode = 1
        if out is None:
            out = torch.empty((splits, M, Nn), dtype=torch.float32, device=x.device)
        ldc = Nn
    elif swiglu:
        assert w.interleaved_swiglu and Nn % 2 == 0
        splits, mode = 1, 2
        if out is None:
            out = torch.empty((M, Nn // 2), dtype=torch.bfloat16, device=x.device)
        ldc = out.stride(0)
    else:
        splits, mode = 1, 0
        if out is None:
            out = torch.empty((M, Nn), dtype=torch.bfloat16, device=x.device)
        ldc = out.stride(0)
    ldr = residual.stride(0) if residual is not None else 0
    rc = lib.afb_gemm_w8a16(
        N.ptr(x), N.ptr(w.q), N.ptr(w.scales), N.ptr(out), N.ptr(bias), N.ptr(residual), _c_int(M), _c_int(Nn),
        _c_int(K), _c_int(x.stride(0)), _c_int(ldc), _c_int(ldr), _c_int(ACT[act]), _c_int(mode), _c_int(splits),
        N.stream_ptr(),
    )
    N.check(rc, "afb_gemm_w8a16")
    N.count_launch()
    return out


# ----------------------------------------------------------------------------------------------------------
# Native MX path: fp8 activations (one or two terms) x fp8 weights with tensor-core block scaling.
# ----------------------------------------------------------------------------------------------------------
_c_long = ctypes.c_long


def sf_atoms_from_scales(scales: torch.Tensor) -> torch.Tensor:
    """[K/32, N] e8m0 bytes -> [ceil(N/128), K/128, 512] scale-factor atoms
    (byte (r % 32) * 16 + (r / 32) * 4 + kblock for row r of the 128-row tile)."""
    kb, n = scales.shape
    assert kb % 4 == 0, "K must be a multiple of 128 for the MX path"
    n_pad = (n + 127) // 128 * 128
    if n_pad != n:
        pad = torch.full((kb, n_pad - n), 127, dtype=scales.dtype, device=scales.device)
        scales = torch.cat([scales, pad], 1)
    v = scales.view(kb // 4, 4, n_pad // 128, 4, 32)           # [chunk, j, tile, r/32, r%32]
    return v.permute(2, 0, 4, 3, 1).contiguous().view(n_pad // 128, kb // 4, 512)


def weight_sf_atoms(w: Fp8Weight) -> torch.Tensor:
    a = getattr(w, "_sf_atoms", None)
    if a is None:
        a = sf_atoms_from_scales(w.scales)
        w._sf_atoms = a
    return a


@dataclass
class MxAct:
    """MX-fp8 activations: e4m3 terms [T, K] and their scale-factor atoms [ceil(T/128), K/128, 512]."""
    q0: torch.Tensor
    sf0: torch.Tensor
    q1: Optional[torch.Tensor] = None
    sf1: Optional[torch.Tensor] = None

    @property
    def terms(self) -> int:
        return 2 if self.q1 is not None else 1

    def dequant(self) -> torch.Tensor:
        def one(q, sf):
            T, K = q.shape
            tiles, chunks = sf.shape[0], sf.shape[1]
            s = sf.view(tiles, chunks, 32, 4, 4).permute(1, 4, 0, 3, 2).reshape(chunks * 4, tiles * 128)[:, :T]
            return R.dequantize_block_fp8(q.view(torch.float8_e4m3fn), s.contiguous())
        y = one(self.q0, self.sf0)
        if self.q1 is not None:
            y = y + one(self.q1, self.sf1)
        return y


def new_mx(T: int, K: int, terms: int, device) -> MxAct:
    """Uninitialised MX activation buffers.  The scale bytes of the padding rows of the last 128-row atom stay
    undefined on the GPU: a row's scale only ever multiplies that row's own output column, and columns past T
    are not stored, so no fill kernel is spent on them."""
    tiles = (T + 127) // 128
    mk = lambda: torch.empty((T, K), dtype=torch.uint8, device=device)
    if torch.device(device).type == "cuda":
        mks = lambda: torch.empty((tiles, K // 128, 512), dtype=torch.uint8, device=device)
    else:
        mks = lambda: torch.full((tiles, K // 128, 512), 127, dtype=torch.uint8, device=device)
    return MxAct(mk(), mks(), mk() if terms == 2 else None, mks() if terms == 2 else None)


def swiglu_quantize_mx(parts: torch.Tensor, terms: int = 2, bias: Optional[torch.Tensor] = None,
                       want_bf16: bool = False):
    """fp32 split-K partial slices [S, T, 2F] of an interleaved gate/up GEMM -> silu(gate) * up -> MX activations
    [T, F] (and the bf16 rows too when ``want_bf16``): the consumer side of a split gate/up GEMM."""
    S, T, N2 = parts.shape
    F = N2 // 2
    assert F % 128 == 0
    if not parts.is_cuda:
        y = parts.sum(0)
        if bias is not None:
            y = y + bias.float()
        y = R.swiglu_interleaved(y).to(torch.bfloat16)
        mx = quantize_mx(y, terms=terms)
        return (mx, y) if want_bf16 else mx
    mx = new_mx(T, F, terms, parts.device)
    y = torch.empty((T, F), dtype=torch.bfloat16, device=parts.device) if want_bf16 else None
    rc = N.cuda().afb_swiglu_quantize_mx(
        N.ptr(parts), _c_int(S), _c_long(parts.stride(0)), _c_long(parts.stride(1)), N.ptr(bias), N.ptr(mx.q0),
        N.ptr(mx.q1), N.ptr(mx.sf0), N.ptr(mx.sf1), N.ptr(y), _c_long(F), _c_int(T), _c_int(F), N.stream_ptr())
    N.check(rc, "afb_swiglu_quantize_mx")
    N.count_launch()
    return (mx, y) if want_bf16 else mx


def quantize_mx(x: torch.Tensor, terms: int = 2, out: Optional[MxAct] = None) -> MxAct:
    """bf16 [T, K] -> MX fp8 (``terms`` = 1: x ~ hi; 2: x ~ hi + lo with lo the quantised residual)."""
    T, K = x.shape
    assert K % 128 == 0
    tiles = (T + 127) // 128
    dev = x.device
    if out is None:
        out = new_mx(T, K, terms, dev)
    if not x.is_cuda:
        def q_one(v):
            q, e8 = R.quantize_block_fp8(v)
            return q, e8
        q0, e0 = q_one(x.float())
        out.q0.copy_(q0.view(torch.uint8))
        pad = tiles * 128 - T
        def atoms(e8):  # e8: [K/32, T]
            if pad:
                e8 = torch.cat([e8, torch.full((e8.shape[0], pad), 127, dtype=e8.dtype)], 1)
            return sf_atoms_from_scales(e8)
        out.sf0.copy_(atoms(e0))
        if terms == 2:
            r = x.float() - R.dequantize_block_fp8(q0, e0)
            q1, e1 = q_one(r)
            out.q1.copy_(q1.view(torch.uint8))
            out.sf1.copy_(atoms(e1))
        return out
    rc = N.cuda().afb_quantize_mx(N.ptr(x), _c_long(x.stride(0)), N.ptr(out.q0), N.ptr(out.q1), N.ptr(out.sf0),
                                  N.ptr(out.sf1), _c_int(T), _c_int(K), N.stream_ptr())
    N.check(rc, "afb_quantize_mx")
    N.count_launch()
    return out


def gemm_mxfp8(x: MxAct, w: Fp8Weight, bias=None, act=None, residual=None, split_k: int = 1, swiglu: bool = False,
               partials: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dequant(x) @ dequant(w).T`` through tcgen05 block-scaled MMA.  Same output modes as gemm_w8a16."""
    M, K = x.q0.shape
    Nn = w.out_features
    assert K == w.in_features and K % 128 == 0
    if not x.q0.is_cuda:
        y = R.linear(x.dequant(), R.dequantize_block_fp8(w.q, w.scales), bias, None if swiglu else act,
                     None if swiglu else residual)
        if swiglu:
            return R.swiglu_interleaved(y).to(torch.bfloat16)
        return y[None] if (partials or split_k > 1) else y.to(torch.bfloat16)
    lib = N.cuda()
    if split_k > 1 or partials:
        splits = int(lib.afb_mx_effective_splits(_c_int(K), _c_int(max(split_k, 1))))
        mode = 1
        if out is None:
            out = torch.empty((splits, M, Nn), dtype=torch.float32, device=x.q0.device)
        ldc = Nn
    elif swiglu:
        splits, mode = 1, 2
        if out is None:
            out = torch.empty((M, Nn // 2), dtype=torch.bfloat16, device=x.q0.device)
        ldc = out.stride(0)
    else:
        splits, mode = 1, 0
        if out is None:
            out = torch.empty((M, Nn), dtype=torch.bfloat16, device=x.q0.device)
        ldc = out.stride(0)
    ldr = residual.stride(0) if residual is not None else 0
    rc = lib.afb_gemm_mxfp8(N.ptr(x.q0), N.ptr(x.q1), N.ptr(x.sf0), N.ptr(x.sf1), N.ptr(w.q), N.ptr(weight_sf_atoms(w)),
                            N.ptr(out), N.ptr(bias), N.ptr(residual), _c_int(M), _c_int(Nn), _c_int(K), _c_int(ldc),
                            _c_int(ldr), _c_int(ACT[act]), _c_int(mode), _c_int(splits), _c_int(x.terms),
                            N.stream_ptr())
    N.check(rc, "afb_gemm_mxfp8")
    N.count_launch()
    return out
