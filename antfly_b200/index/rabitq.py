"""RaBitQ 1-bit quantiser with 4-bit query quantisation and the weighted-popcount distance estimator.

Restates the reference's RaBitQuantizer (zig/lib/vector/src/quantizer.zig:110-470, rabitq.zig:40-200): a vector is
centred on the node centroid and normalised; its code is the sign pattern packed MSB-first into u64 words; stored
per vector: code, popcount, distance to the centroid, and the inverse of <o_bar, o> (0 when the vector equals the
centroid), plus <v, c> for inner-product / cosine.  A query is centred the same way, quantised to 4 bits per
dimension with a per-dimension random unbias offset, split into four bit planes, and scored with
``pop(c&q1) + 2 pop(c&q2) + 4 pop(c&q3) + 8 pop(c&q4)``; the estimator and its error bound follow the paper
(arXiv 2405.12497).  The scorer runs on the GPU (one thread per code) or on the CPU through the same formulas.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from .. import _native as N

_METRIC = {"l2_squared": 0, "inner_product": 1, "cosine": 2}


def code_width(dims: int) -> int:
    return (dims + 63) // 64


@dataclass
class RaBitQSet:
    metric: str
    centroid: torch.Tensor          # [D] fp32
    codes: torch.Tensor             # [n, width] int64 (bit pattern of the u64 words)
    code_counts: torch.Tensor       # [n] int32
    centroid_distances: torch.Tensor  # [n] fp32
    inv_dot: torch.Tensor           # [n] fp32 (stored inverted)
    centroid_dot: Optional[torch.Tensor] = None  # [n] <v, c> for ip / cosine
    centroid_norm: float = 0.0
    data_norms: Optional[torch.Tensor] = None    # [n] |v| for cosine

    def to(self, device) -> "RaBitQSet":
        f = lambda t: None if t is None else t.to(device)
        return RaBitQSet(self.metric, f(self.centroid), f(self.codes), f(self.code_counts), f(self.centroid_distances),
                         f(self.inv_dot), f(self.centroid_dot), self.centroid_norm, f(self.data_norms))


class RaBitQuantizer:
    def __init__(self, dims: int, metric: str = "l2_squared", seed: int = 42):
        self.dims, self.metric = dims, metric
        self.sqrt_dims = math.sqrt(dims)
        g = torch.Generator().manual_seed(seed)
        self.unbias = torch.rand(dims, generator=g)

    def _pack(self, bits: torch.Tensor) -> torch.Tensor:
        """bits [n, D] {0,1} -> [n, width] int64, MSB-first within each word."""
        n, D = bits.shape
        w = code_width(D)
        pad = w * 64 - D
        if pad:
            bits = torch.cat([bits, torch.zeros(n, pad, dtype=bits.dtype, device=bits.device)], 1)
        b = bits.view(n, w, 64).to(torch.int64)
        shifts = torch.arange(63, -1, -1, device=bits.device, dtype=torch.int64)
        return (b << shifts).sum(-1)  # two's-complement wrap gives the right bit pattern for bit 63

    def quantize(self, centroid: torch.Tensor, vectors: torch.Tensor) -> RaBitQSet:
        c = centroid.float()
        v = vectors.float()
        diff = v - c
        dist = diff.norm(dim=-1)
        unit = torch.where(dist[:, None] > 0, diff / dist[:, None].clamp_min(1e-30), diff)
        bits = (unit >= 0)
        dot = (unit.abs().sum(-1) / self.sqrt_dims)
        inv = torch.where(dot != 0, 1.0 / dot.clamp_min(1e-30), torch.zeros_like(dot))
        cdot = (v @ c) if self.metric != "l2_squared" else None
        return RaBitQSet(self.metric, c, self._pack(bits.to(torch.uint8)), bits.sum(-1).int(), dist, inv, cdot,
                         float(c.norm()) if self.metric != "l2_squared" else 0.0,
                         v.norm(dim=-1) if self.metric == "cosine" else None)

    def _query_planes(self, qs: RaBitQSet, query: torch.Tensor):
        q = query.float().to(qs.centroid.device)
        qd = q - qs.centroid
        qdist = float(qd.norm())
        if qdist == 0:
            return None
        qd = qd / qdist
        lo, hi = float(qd.min()), float(qd.max())
        delta = (hi - lo) / 15.0
        if delta != 0:
            qv = torch.floor((qd - lo) / delta + self.unbias.to(qd.device)).clamp(0, 15).to(torch.int64)
        else:
            qv = torch.zeros_like(qd, dtype=torch.int64)
        planes = torch.stack([self._pack(((qv >> b) & 1).to(torch.uint8)[None])[0] for b in range(4)])
        qsum = float(qv.sum())
        inv_sd = 1.0 / self.sqrt_dims
        t1 = 2.0 * delta * inv_sd
        t2 = 2.0 * lo * inv_sd
        t34 = delta * inv_sd * qsum + self.sqrt_dims * lo
        qcdot = float(q @ qs.centroid) if self.metric != "l2_squared" else 0.0
        return planes.contiguous(), qdist, t1, t2, t34, qcdot, float(q.norm())

    def estimate(self, qs: RaBitQSet, query: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(distances [n], error_bounds [n]) under the set's metric."""
        n = qs.codes.shape[0]
        dev = qs.codes.device
        prep = self._query_planes(qs, query)
        if prep is None:  # query sits on the centroid
            d = qs.centroid_distances
            if self.metric == "l2_squared":
                return d * d, torch.zeros_like(d)
            ip = qs.centroid_dot
            if self.metric == "inner_product":
                return -ip, torch.zeros_like(d)
            den = float(query.float().norm()) * qs.data_norms
            return torch.where(den > 0, 1 - ip / den.clamp_min(1e-30), torch.ones_like(ip)), torch.zeros_like(d)
        planes, qdist, t1, t2, t34, qcdot, qnorm = prep
        if dev.type == "cuda":
            dist = torch.empty(n, dtype=torch.float32, device=dev)
            err = torch.empty(n, dtype=torch.float32, device=dev)
            rc = N.cuda().afb_rabitq_estimate(
                N.ptr(qs.codes), N.ptr(planes), N.ptr(qs.code_counts), N.ptr(qs.centroid_distances), N.ptr(qs.inv_dot),
                N.ptr(qs.centroid_dot), N.ptr(qs.data_norms), N.ptr(dist), N.ptr(err), None, ctypes.c_int(n),
                ctypes.c_int(qs.codes.shape[1]), ctypes.c_int(_METRIC[self.metric]), ctypes.c_float(t1),
                ctypes.c_float(t2), ctypes.c_float(t34), ctypes.c_float(qdist), ctypes.c_float(qcdot),
                ctypes.c_float(qs.centroid_norm ** 2), ctypes.c_float(self.sqrt_dims), ctypes.c_float(qnorm),
                N.stream_ptr())
            N.check(rc, "afb_rabitq_estimate")
            N.count_launch()
            return dist, err
        bp = bit_product(qs.codes, planes).float()
        est = (t1 * bp + t2 * qs.code_counts.float() - t34) * qs.inv_dot
        dcd = qs.centroid_distances
        if self.metric == "l2_squared":
            mult = 2.0 * dcd * qdist
            d = dcd * dcd + qdist * qdist - mult * est
            e = mult / self.sqrt_dims
            neg = d < 0
            e = torch.where(neg, (e + d).clamp_min(0), e)
            return d.clamp_min(0), e
        mult = dcd * qdist
        ip = mult * est + qs.centroid_dot + qcdot - qs.centroid_norm ** 2
        e = mult / self.sqrt_dims
        if self.metric == "inner_product":
            return -ip, e
        den = qnorm * qs.data_norms
        return torch.where(den > 0, 1 - ip / den.clamp_min(1e-30), torch.ones_like(ip)), \
            torch.where(den > 0, e / den.clamp_min(1e-30), torch.zeros_like(e))


def _popcount64(x: torch.Tensor) -> torch.Tensor:
    x = x.clone()
    cnt = torch.zeros_like(x)
    # bit 63 first (sign bit), then the rest by shifting a masked copy
    cnt += (x < 0).to(torch.int64)
    x = x & 0x7FFFFFFFFFFFFFFF
    m1, m2, m4 = 0x5555555555555555, 0x3333333333333333, 0x0F0F0F0F0F0F0F0F
    x = x - ((x >> 1) & m1)
    x = (x & m2) + ((x >> 2) & m2)
    x = (x + (x >> 4)) & m4
    x = (x * 0x0101010101010101) >> 56
    return cnt + (x & 0xFF)


def bit_product(codes: torch.Tensor, planes: torch.Tensor) -> torch.Tensor:
    """[n, width] codes x [4, width] query planes -> [n] weighted popcount (CPU / torch restatement)."""
    out = torch.zeros(codes.shape[0], dtype=torch.int64, device=codes.device)
    for b in range(4):
        out += _popcount64(codes & planes[b][None]).sum(-1) << b
    return out
