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
