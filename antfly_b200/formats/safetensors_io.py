"""safetensors reader / writer without the upstream wheel: 8-byte little-endian header length, a JSON header
``{name: {dtype, shape, data_offsets}}``, then raw tensor bytes (zig/pkg/inference/src/models/safetensors.zig:15-24;
writer: zig/pkg/inference/src/finetune/safetensors_checkpoint.zig:15-33).  Reading memory-maps the file and
returns zero-copy views; sharded checkpoints are resolved through ``*.safetensors.index.json``."""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Optional

import numpy as np
import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._mm[:8])
        if n > len(self._mm) - 8:
            raise ValueError(f"{path}: header length {n} exceeds the file size")
        self.header = json.loads(self._mm[8:8 + n].decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n

    def keys(self) -> Iterable[str]:
        return self.header.keys()

    def tensor(self, name: str) -> torch.Tensor:
        e = self.header[name]
        lo, hi = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        if hi == lo:
            return torch.empty(e["shape"], dtype=dt)
        buf = memoryview(self._mm)[self._base + lo:self._base + hi]
        return torch.frombuffer(buf, dtype=dt).view(e["shape"])

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass  # views are still alive; the mapping is released with them
        self._f.close()


def read_metadata(path: str) -> Dict[str, str]:
    """The ``__metadata__`` string map of a safetensors file (no tensor data is touched)."""
    f = SafetensorsFile(path)
    try:
        return dict(f.metadata)
    finally:
        f.close()


def load_file(path: str) -> Dict[str, torch.Tensor]:
    f = SafetensorsFile(path)
    return {k: f.tensor(k) for k in f.keys()}


def load_model_dir(model_dir: str) -> Dict[str, torch.Tensor]:
    """model.safetensors | pytorch_model.safetensors | sharded index (zig/.../models/manifest.zig:112-120)."""
    for name in ("model.safetensors", "pytorch_model.safetensors"):
        p = os.path.join(model_dir, name)
        if os.path.exists(p):
            return load_file(p)
        idx = p + ".index.json"
        if os.path.exists(idx):
            with open(idx, encoding="utf-8") as f:
                weight_map = json.load(f)["weight_map"]
            out: Dict[str, torch.Tensor] = {}
            for shard in sorted(set(weight_map.values())):
                out.update(load_file(os.path.join(model_dir, shard)))
            return out
    raise FileNotFoundError(f"no safetensors weights in {model_dir}")


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for b in blobs:
            f.write(b)
