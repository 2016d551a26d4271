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


def linear_gguf(x: torch.Tensor, raw_weight: torch.Tensor, type_id: int, out_features: int, in_features: int,
                bias: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """``act(x @ dequant(W).T + bias)`` for a GGUF-quantised weight [out_features, in_features] kept in its block
    format in memory (4.5 - 8.5 bits per weight) and expanded for the GEMM."""
    w = dequantize(raw_weight, type_id, (out_features, in_features), torch.bfloat16)
    return Dn.gemm_bf16(x.to(torch.bfloat16), w, bias=bias, act=act)
