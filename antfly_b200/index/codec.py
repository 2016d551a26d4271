"""Wire encodings of vectors in the API: float arrays, base64 little-endian f32 ("packed"), and sparse
{indices, values} either as arrays or as packed u32 / f32 base64 (specs/openapi/antfly/metadata.yaml:4243-4253,
zig/lib/vector/src/codec.zig:34-164)."""
from __future__ import annotations

import base64
import struct
from typing import Dict, List, Sequence, Union

import numpy as np
import torch


def encode_packed(v: torch.Tensor) -> str:
    return base64.b64encode(v.detach().float().cpu().numpy().astype("<f4").tobytes()).decode("ascii")


def decode_packed(s: str, dim: int = 0) -> torch.Tensor:
    raw = base64.b64decode(s, validate=True)
    if len(raw) % 4:
        raise ValueError("packed vector length is not a multiple of 4 bytes")
    a = np.frombuffer(raw, dtype="<f4").astype(np.float32)
    if dim:
        if a.size % dim:
            raise ValueError(f"packed vector has {a.size} floats, not a multiple of dimension {dim}")
        return torch.from_numpy(a.copy()).view(-1, dim)
    return torch.from_numpy(a.copy()).view(1, -1)


def decode_vectors(x: Union[str, Sequence[float], Sequence[Sequence[float]]], dim: int = 0) -> torch.Tensor:
    """Any accepted dense encoding -> fp32 [Q, D]."""
    if isinstance(x, str):
        return decode_packed(x, dim)
    if len(x) == 0:
        raise ValueError("empty vector")
    if isinstance(x[0], (int, float)):
        return torch.tensor([list(x)], dtype=torch.float32)
    return torch.tensor([list(r) for r in x], dtype=torch.float32)


def encode_sparse_packed(indices: Sequence[int], values: Sequence[float]) -> Dict[str, str]:
    return {"indices": base64.b64encode(np.asarray(indices, dtype="<u4").tobytes()).decode("ascii"),
            "values": base64.b64encode(np.asarray(values, dtype="<f4").tobytes()).decode("ascii")}


def decode_sparse(obj: Dict) -> Dict[str, List]:
    idx, val = obj["indices"], obj["values"]
    if isinstance(idx, str):
        idx = np.frombuffer(base64.b64decode(idx), dtype="<u4").tolist()
    if isinstance(val, str):
        val = np.frombuffer(base64.b64decode(val), dtype="<f4").tolist()
    if len(idx) != len(val):
        raise ValueError("sparse vector indices and values differ in length")
    order = sorted(range(len(idx)), key=lambda i: idx[i])
    return {"indices": [int(idx[i]) for i in order], "values": [float(val[i]) for i in order]}
