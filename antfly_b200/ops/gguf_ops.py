"""GGUF-quantised weights on the device: block bytes -> bf16 on the GPU (``afb_gguf_dequant_device``) and a linear
layer over them (expand, then the tcgen05 bf16 GEMM).  Artifact-format parity with the reference's Q8_0 / Q4_0 /
Q4_K linears (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:873-1553); CPU tensors go through
the C++ block decoders."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import numpy as np
import torch

from .. import _native as N
from . import dense as Dn

DEVICE_TYPES = {2: "Q4_0", 8: "Q8_0", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 39: "MXFP4"}


def block_geometry(type_id: int) -> Tuple[int, int]:
    lib = N.host()
    lib.afb_gguf_block_bytes.restype = ctypes.c_long
    lib.afb_gguf_block_values.restype = ctypes.c_long
    bv, bb = int(lib.afb_gguf_block_values(type_id)), int(lib.afb_gguf_block_bytes(type_id))
    if bv < 0:
        raise NotImplementedError(f"GGUF tensor type {type_id} is not supported")
    return bv, bb


def dequantize(raw: torch.Tensor, type_id: int, shape: Tuple[int, ...],
               dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """raw: uint8 tensor holding whole blocks of ``type_id``; returns the ``shape``-d tensor of ``dtype``
    (bf16 or fp32) on raw's device."""
    n = int(np.prod(shape))
    bv, bb = block_geometry(type_id)
    assert n % bv == 0 and raw.numel() == n // bv * bb and raw.dtype == torch.uint8
    if raw.is_cuda and type_id in DEVICE_TYPES:
        assert dtype in (torch.bfloat16, torch.float32)
        out = torch.empty(n, dtype=dtype, device=raw.device)
        rc = N.cuda().afb_gguf_dequant_device(ctypes.c_int(type_id), N.ptr(raw.contiguous()), N.ptr(out),
                                              ctypes.c_long(n), ctypes.c_int(1 if dtype == torch.float32 else 0),
                                              N.stream_ptr())
        N.check(rc, "afb_gguf_dequant_device")
        N.count_launch()
        return out.view(shape)
    src = np.ascontiguousarray(raw.detach().cpu().numpy())
    out = np.empty(n, dtype=np.float32)
    rc = N.host().afb_gguf_dequantize(ctypes.c_int(type_id), src.ctypes.data_as(ctypes.c_void_p),
                                      out.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(n))
    if rc != 0:
        raise NotImplementedError(f"GGUF tensor type {type_id} is not supported")
    return torch.from_numpy(out).view(shape).to(dtype).to(raw.device)


ACT_CODES = {None: 0, "none": 0, "gelu": 1, "gelu_tanh": 2, "relu": 3, "silu": 4}
# Rows of the weight expanded per GEMM call on the large-batch path: the bf16 slab (rows x K x 2 bytes) stays well
# inside the 126 MB L2, so it is written and read back on chip instead of through HBM.
EXPAND_SLAB_BYTES = 48 << 20


def mul_mv(x: torch.Tensor, raw_weight: torch.Tensor, type_id: int, out_features: int, in_features: int,
           bias: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """The fused kernel (csrc/kernels/gemm_gguf.cu): up to 8 rows of bf16 activations against a weight in its GGUF
    block format, expanded in registers only."""
    M = x.shape[0]
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.stride(1) == 1 and M <= 8 and type_id in DEVICE_TYPES
    out = torch.empty((M, out_features), dtype=torch.bfloat16, device=x.device)
    rc = N.cuda().afb_gguf_mul_mv(
        ctypes.c_int(type_id), N.ptr(raw_weight), N.ptr(x), N.ptr(bias), N.ptr(out), ctypes.c_int(M),
        ctypes.c_int(out_features), ctypes.c_int(in_features), ctypes.c_long(x.stride(0)),
        ctypes.c_long(out.stride(0)), ctypes.c_int(ACT_CODES[act]), N.stream_ptr())
    N.check(rc, "afb_gguf_mul_mv")
    N.count_launch()
    return out


def linear_gguf(x: torch.Tensor, raw_weight: torch.Tensor, type_id: int, out_features: int, in_features: int,
                bias: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """``act(x @ dequant(W).T + bias)`` for a GGUF-quantised weight [out_features, in_features] kept in its block
    format in memory (4.25 - 8.5 bits per weight).  Up to 8 tokens: one fused kernel that reads the quantised bytes
    once (the batch is bound by weight traffic).  More tokens: the weight is expanded slab by slab, each slab small
    enough to stay in L2 between the expansion and the tcgen05 GEMM that consumes it."""
    if x.is_cuda and type_id in DEVICE_TYPES:
        xb = x.to(torch.bfloat16)
        if xb.stride(-1) != 1 or xb.stride(0) % 8 or xb.data_ptr() % 16:
            xb = xb.contiguous()
        if x.shape[0] <= 8 and in_features % 8 == 0:
            return mul_mv(xb, raw_weight, type_id, out_features, in_features,
                          bias.to(torch.bfloat16) if bias is not None else None, act)
        bv, bb = block_geometry(type_id)
        row_bytes = in_features // bv * bb
        rows = max(256, (EXPAND_SLAB_BYTES // (2 * in_features)) // 256 * 256)
        if rows >= out_features:
            w = dequantize(raw_weight, type_id, (out_features, in_features), torch.bfloat16)
            return Dn.gemm_bf16(xb, w, bias=bias, act=act)
        out = torch.empty((x.shape[0], out_features), dtype=torch.bfloat16, device=x.device)
        raw2 = raw_weight.view(out_features, row_bytes)
        for n0 in range(0, out_features, rows):
            n1 = min(out_features, n0 + rows)
            w = dequantize(raw2[n0:n1].reshape(-1), type_id, (n1 - n0, in_features), torch.bfloat16)
            Dn.gemm_bf16(xb, w, bias=bias[n0:n1] if bias is not None else None, act=act, out=out[:, n0:n1])
        return out
    w = dequantize(raw_weight, type_id, (out_features, in_features), torch.bfloat16)
    return Dn.gemm_bf16(x.to(torch.bfloat16), w, bias=bias, act=act)


def decode32(type_id: int, block: bytes, sub: int) -> np.ndarray:
    """Values [32 sub, 32 sub + 32) of one block through the fused kernel's decoder (host build of the same code)."""
    out = np.empty(32, dtype=np.float32)
    buf = np.frombuffer(block, dtype=np.uint8)
    N.host().afb_gguf_decode32(ctypes.c_int(type_id), buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(sub),
                               out.ctypes.data_as(ctypes.c_void_p))
    return out


def mul_mv_host(x: torch.Tensor, raw_weight: torch.Tensor, type_id: int, out_features: int, in_features: int):
    """The fused kernel's work split replayed on the host (same decoder, same chunk / lane / row arithmetic):
    -> (out fp32 [M, N], number of (row, sub-block) units visited)."""
    xf = np.ascontiguousarray(x.detach().float().cpu().numpy())
    w = np.ascontiguousarray(raw_weight.detach().cpu().numpy())
    out = np.zeros((xf.shape[0], out_features), dtype=np.float32)
    lib = N.host()
    lib.afb_gguf_mul_mv_host.restype = ctypes.c_long
    units = lib.afb_gguf_mul_mv_host(ctypes.c_int(type_id), w.ctypes.data_as(ctypes.c_void_p),
                                     xf.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                     ctypes.c_int(xf.shape[0]), ctypes.c_int(out_features), ctypes.c_int(in_features),
                                     ctypes.c_long(xf.shape[1]))
    if units < 0:
        raise NotImplementedError(f"GGUF tensor type {type_id} has no fused kernel")
    return torch.from_numpy(out), int(units)


class GgufWeight:
    """A linear layer's weight kept in GGUF block bytes on the device: one or more row segments (fused projections
    whose parts may be stored in different block formats), applied segment by segment through :func:`linear_gguf`.
    ``interleave`` lays two equal segments out column-alternating (gate_0, up_0, gate_1, ...), the layout the gated
    MLP reads."""

    def __init__(self, segments, in_features: int, interleave: bool = False):
        self.segments = list(segments)            # [(raw uint8 tensor, type id, rows)]
        self.in_features, self.interleave = in_features, interleave
        self.out_features = sum(r for _, _, r in self.segments)

    def nbytes(self) -> int:
        return sum(int(raw.numel()) for raw, _, _ in self.segments)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        outs = [linear_gguf(x, raw, ty, rows, self.in_features) for raw, ty, rows in self.segments]
        if self.interleave:
            assert len(outs) == 2 and outs[0].shape == outs[1].shape
            return torch.stack(outs, -1).flatten(1)
        return outs[0] if len(outs) == 1 else torch.cat(outs, 1)
