"""Paged KV cache: device-resident block pool + the C++ block allocator / block tables.

Layout per layer: ``k[num_blocks, page, n_kv_heads, head_dim]`` and the same for ``v`` (bf16, or e4m3 bytes with
a per-tensor scale).  The allocator (``csrc/host/kv_blocks.cpp``) hands out block ids and slot numbers; kernels
address tokens as ``slot = block * page + offset``.  Semantics follow the reference's KvManager
(zig/pkg/inference/src/runtime/kv/manager.zig:77-378).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native as N

_i64 = ctypes.c_int64
_int = ctypes.c_int
_pint = ctypes.POINTER(ctypes.c_int)

# Plain tensor caches [layers, blocks, page, Hkv, D].  "f16" is served from bf16 storage (same size; the kernels
# read bf16).  "f32" exists on the CPU path only (tests and the dequantised-cache reference).
KV_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "f16": torch.bfloat16, "f32": torch.float32}
# Caches kept in a quantised codec: byte rows, see ops/kv_quant.py (the reference's pool dtypes,
# zig/pkg/inference/src/runtime/kv/pool.zig:26-35 and runtime/kv/turboquant.zig).
KV_CODECS = ("fp8", "int8", "int4", "polar4", "turbo3")


class KvOutOfBlocks(RuntimeError):
    pass


def _lib():
    lib = N.host()
    if not getattr(lib, "_kv_ready", False):
        lib.afb_kv_create.restype = ctypes.c_void_p
        lib.afb_kv_create.argtypes = [_int, _int]
        lib.afb_kv_destroy.argtypes = [ctypes.c_void_p]
        for name in ("afb_kv_free_blocks", "afb_kv_num_sequences"):
            getattr(lib, name).argtypes = [ctypes.c_void_p]
        lib.afb_kv_attach.argtypes = [ctypes.c_void_p, _i64]
        lib.afb_kv_attach_shared.argtypes = [ctypes.c_void_p, _i64, _i64, _int]
        lib.afb_kv_take_cow.argtypes = [ctypes.c_void_p, _pint, _pint, _int]
        lib.afb_kv_append.argtypes = [ctypes.c_void_p, _i64, _int, _pint]
        lib.afb_kv_truncate.argtypes = [ctypes.c_void_p, _i64, _int]
        lib.afb_kv_trim_window.argtypes = [ctypes.c_void_p, _i64, _int]
        lib.afb_kv_len.argtypes = [ctypes.c_void_p, _i64]
        lib.afb_kv_block_table.argtypes = [ctypes.c_void_p, _i64, _pint, _int]
        lib.afb_kv_detach.argtypes = [ctypes.c_void_p, _i64]
        lib.afb_kv_refcount.argtypes = [ctypes.c_void_p, _int]
        lib.afb_kv_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64)]
        lib.afb_kv_append_batch.argtypes = [ctypes.c_void_p, ctypes.POINTER(_i64), _pint, _int, _pint, _pint, _pint,
                                            _int]
        lib._kv_ready = True
    return lib


class BlockAllocator:
    """Thin wrapper over the C++ pool (no tensors): block ids, block tables, slots."""

    def __init__(self, num_blocks: int, page: int = 16):
        self.lib = _lib()
        self.num_blocks, self.page = num_blocks, page
        self.h = ctypes.c_void_p(self.lib.afb_kv_create(num_blocks, page))
        if not self.h:
            raise ValueError("invalid pool geometry")

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.lib.afb_kv_destroy(self.h)
                self.h = None
        except Exception:
            pass

    @property
    def free_blocks(self) -> int:
        return self.lib.afb_kv_free_blocks(self.h)

    def attach(self, seq: int) -> None:
        if self.lib.afb_kv_attach(self.h, seq) != 0:
            raise KeyError(f"sequence {seq} already attached")

    def attach_shared(self, seq: int, parent: int, prefix_tokens: int) -> None:
        rc = self.lib.afb_kv_attach_shared(self.h, seq, parent, prefix_tokens)
        if rc == -2:
            raise KvOutOfBlocks("no free block for the copied prefix tail")
        if rc != 0:
            raise KeyError("bad sequence ids or prefix length")

    def take_cow(self, max_pairs: int = 1024) -> Tuple[np.ndarray, np.ndarray]:
        src = np.empty(max_pairs, dtype=np.int32)
        dst = np.empty(max_pairs, dtype=np.int32)
        n = self.lib.afb_kv_take_cow(self.h, src.ctypes.data_as(_pint), dst.ctypes.data_as(_pint), max_pairs)
        return src[:n], dst[:n]

    def append(self, seq: int, n_tokens: int) -> np.ndarray:
        slots = np.empty(max(n_tokens, 1), dtype=np.int32)
        rc = self.lib.afb_kv_append(self.h, seq, n_tokens, slots.ctypes.data_as(_pint))
        if rc == -2:
            raise KvOutOfBlocks(f"KV pool exhausted appending {n_tokens} tokens to sequence {seq}")
        if rc != 0:
            raise KeyError(f"unknown sequence {seq}")
        return slots[:n_tokens]

    def append_batch(self, seqs: np.ndarray, n_tokens: np.ndarray, max_blocks: int, tables: Optional[np.ndarray]):
        """Append n_tokens[i] to seqs[i]; returns (slots, lens).  ``tables`` [n, max_blocks] int32 is refreshed."""
        n = len(seqs)
        slots = np.empty(int(n_tokens.sum()), dtype=np.int32)
        lens = np.empty(n, dtype=np.int32)
        seqs = np.ascontiguousarray(seqs, dtype=np.int64)
        n_tokens = np.ascontiguousarray(n_tokens, dtype=np.int32)
        done = self.lib.afb_kv_append_batch(
            self.h, seqs.ctypes.data_as(ctypes.POINTER(_i64)), n_tokens.ctypes.data_as(_pint), n,
            slots.ctypes.data_as(_pint), lens.ctypes.data_as(_pint),
            tables.ctypes.data_as(_pint) if tables is not None else None, max_blocks)
        if done != n:
            raise KvOutOfBlocks(f"KV pool exhausted at batch item {done}")
        return slots, lens

    def truncate(self, seq: int, new_len: int) -> None:
        if self.lib.afb_kv_truncate(self.h, seq, new_len) != 0:
            raise KeyError("unknown sequence or bad length")

    def trim_window(self, seq: int, window: int) -> int:
        return self.lib.afb_kv_trim_window(self.h, seq, window)

    def length(self, seq: int) -> int:
        return self.lib.afb_kv_len(self.h, seq)

    def block_table(self, seq: int, max_blocks: Optional[int] = None) -> np.ndarray:
        cap = max_blocks or (self.length(seq) + self.page - 1) // self.page + 1
        out = np.zeros(cap, dtype=np.int32)
        n = self.lib.afb_kv_block_table(self.h, seq, out.ctypes.data_as(_pint), cap)
        if n < 0:
            raise KeyError(f"unknown sequence {seq}")
        return out[: min(n, cap)] if max_blocks is None else out

    def detach(self, seq: int) -> None:
        self.lib.afb_kv_detach(self.h, seq)

    def refcount(self, block: int) -> int:
        return self.lib.afb_kv_refcount(self.h, block)

    def stats(self) -> dict:
        out = (ctypes.c_uint64 * 3)()
        self.lib.afb_kv_stats(self.h, out)
        return {"acquired": int(out[0]), "released": int(out[1]), "oom": int(out[2])}


class PagedKvCache:
    """Device tensors for every layer plus one allocator shared by all layers."""

    def __init__(self, n_layers: int, num_blocks: int, n_kv_heads: int, head_dim: int, page: int = 16,
                 dtype: str = "bf16", device="cuda"):
        self.page, self.num_blocks = page, num_blocks
        self.kv_scale = 1.0
        self.alloc = BlockAllocator(num_blocks, page)
        self.codec: Optional[str] = None
        if dtype in KV_CODECS:
            from ..ops.kv_quant import CodecCache

            self.codec, self.dtype = dtype, torch.uint8
            self.k = CodecCache(dtype, n_layers, num_blocks, page, n_kv_heads, head_dim, device, value=False)
            self.v = CodecCache(dtype, n_layers, num_blocks, page, n_kv_heads, head_dim, device, value=True)
            return
        if dtype not in KV_DTYPES:
            raise ValueError(f"unknown KV cache dtype {dtype!r}; one of {sorted(set(KV_DTYPES) | set(KV_CODECS))}")
        if dtype == "f32" and torch.device(device).type == "cuda":
            raise ValueError("an f32 KV cache is available on the CPU path only (the GPU kernels read bf16 or codecs)")
        self.dtype = KV_DTYPES[dtype]
        shape = (n_layers, num_blocks, page, n_kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=self.dtype, device=device)
        self.v = torch.zeros(shape, dtype=self.dtype, device=device)

    def layer(self, i: int):
        return self.k[i], self.v[i]

    def nbytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def run_pending_copies(self) -> int:
        from ..ops import attention as A

        src, dst = self.alloc.take_cow()
        if len(src) == 0:
            return 0
        s = torch.from_numpy(src.copy()).to(self.k.device)
        d = torch.from_numpy(dst.copy()).to(self.k.device)
        for l in range(self.k.shape[0]):
            if self.codec is not None:      # byte rows: a block copy is a block copy
                kd, vd = self.k.data[l], self.v.data[l]
                kd[d.long()] = kd[s.long()]
                vd[d.long()] = vd[s.long()]
            else:
                A.kv_copy_blocks(self.k[l], self.v[l], s, d)
        return len(src)


def estimate_kv_bytes(n_layers: int, n_kv_heads: int, head_dim: int, tokens: int, dtype: str = "bf16") -> int:
    """HBM needed to hold ``tokens`` tokens of KV (the reference's estimateGptGeneration,
    zig/pkg/inference/src/runtime/tier/memory.zig:455, reduced to the device tier)."""
    if dtype in KV_CODECS:
        from ..ops.kv_quant import row_bytes

        return n_layers * tokens * (row_bytes(dtype, n_kv_heads, head_dim) + row_bytes(dtype, n_kv_heads, head_dim, True))
    el = 4 if dtype == "f32" else 2
    return 2 * n_layers * n_kv_heads * head_dim * tokens * el
