"""Quantised KV-cache codecs and decode attention over compressed cache rows.

Codecs (row formats in ``csrc/common/kvq_elem.h``): ``bf16``, ``fp8`` (e4m3 bytes), ``int8`` (per-head f32 scale),
``int4`` (groups of 32 with an f16 scale), ``polar4`` (4-bit keys on a fixed grid, int8 values) and ``turbo3``
(3-bit keys plus a 32-bit residual sign sketch per head, int8 values).  They are the cache dtypes of the reference's
KV pool (zig/pkg/inference/src/runtime/kv/pool.zig:30-130, runtime/kv/turboquant.zig).

Three implementations of the same formats live here:

* the C++ host library (``csrc/host/kv_codecs.cpp``): row encode / decode and a CPU decode attention that scores
  queries straight against the codes;
* torch encoders (:func:`encode_rows_torch`) that produce the same bytes with tensor ops on whatever device the
  cache lives on -- this is how new tokens are written into a GPU-resident quantised cache;
* the CUDA decode-attention kernel (``csrc/kernels/attention_kvq.cu``), which shares the per-element decoders with
  the host library.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import numpy as np
import torch

from .. import _native as N

CODECS = {"bf16": 0, "fp8": 1, "int8": 2, "int4": 3, "polar4": 4, "turbo3": 5}
SKETCH_BITS = 32
RESIDUAL_SCALE = 0.125

_c_int, _c_long, _c_float = ctypes.c_int, ctypes.c_long, ctypes.c_float


def _host():
    lib = N.host()
    lib.afb_kvq_row_bytes.restype = ctypes.c_long
    return lib


def row_bytes(codec: str, heads: int, D: int, value: bool = False) -> int:
    n = int(_host().afb_kvq_row_bytes(_c_int(CODECS[codec]), _c_int(heads), _c_int(D), _c_int(1 if value else 0)))
    if n <= 0:
        raise ValueError(f"KV codec {codec!r} does not support head size {D}")
    return n


def encode_rows(codec: str, x: torch.Tensor, value: bool = False) -> torch.Tensor:
    """x [T, heads, D] (any float dtype, CPU) -> uint8 [T, row_bytes] through the C++ encoder."""
    T, H, D = x.shape
    xf = x.detach().float().contiguous().cpu()
    out = torch.empty((T, row_bytes(codec, H, D, value)), dtype=torch.uint8)
    rc = _host().afb_kvq_encode_rows(_c_int(CODECS[codec]), _c_int(1 if value else 0), N.ptr(xf), N.ptr(out),
                                     _c_long(T), _c_int(H), _c_int(D))
    if rc != 0:
        raise ValueError(f"KV codec {codec!r}: unsupported shape")
    return out


def decode_rows(codec: str, rows: torch.Tensor, heads: int, D: int, value: bool = False) -> torch.Tensor:
    """uint8 [T, row_bytes] -> fp32 [T, heads, D] (for turbo3 keys: the 3-bit base values, without the sketch)."""
    rows = rows.contiguous().cpu()
    T = rows.shape[0]
    assert rows.shape[1] == row_bytes(codec, heads, D, value)
    out = torch.empty((T, heads, D), dtype=torch.float32)
    rc = _host().afb_kvq_decode_rows(_c_int(CODECS[codec]), _c_int(1 if value else 0), N.ptr(rows), N.ptr(out),
                                     _c_long(T), _c_int(heads), _c_int(D))
    assert rc == 0
    return out


# ----------------------------------------------------------------------------------------------------------
# torch encoders (any device)
# ----------------------------------------------------------------------------------------------------------
def _round_away(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


def _int8_rows(x: torch.Tensor) -> torch.Tensor:
    T, H, D = x.shape
    mx = x.abs().amax(-1)
    scale = torch.where(mx == 0, torch.ones_like(mx), mx / 127.0)
    codes = _round_away(x * (1.0 / scale)[..., None]).clamp_(-127, 127).to(torch.int8)
    return torch.cat([scale.contiguous().view(torch.uint8).view(T, H, 4), codes.view(torch.uint8)], -1).reshape(T, -1)


_SIGN_CACHE = {}


def random_signs(heads: int, D: int, device="cpu") -> torch.Tensor:
    """[heads, 32, D] of +-1: the residual-sketch projections (a 64-bit integer mix of head, projection, dim)."""
    key = (heads, D, str(device))
    if key not in _SIGN_CACHE:
        with np.errstate(over="ignore"):
            h = (np.arange(heads, dtype=np.uint64) + np.uint64(1))[:, None, None] * np.uint64(0x9E3779B97F4A7C15)
            p = (np.arange(SKETCH_BITS, dtype=np.uint64) + np.uint64(1))[None, :, None] * np.uint64(0xBF58476D1CE4E5B9)
            d = (np.arange(D, dtype=np.uint64) + np.uint64(1))[None, None, :] * np.uint64(0x94D049BB133111EB)
            x = h ^ p ^ d
            x ^= x >> np.uint64(30)
            x *= np.uint64(0xBF58476D1CE4E5B9)
            x ^= x >> np.uint64(27)
            x *= np.uint64(0x94D049BB133111EB)
            x ^= x >> np.uint64(31)
        s = np.where((x & np.uint64(1)) == 0, 1.0, -1.0).astype(np.float32)
        _SIGN_CACHE[key] = torch.from_numpy(s).to(device)
    return _SIGN_CACHE[key]


def _pack_bits(bits: torch.Tensor) -> torch.Tensor:
    """bits [T, n] of 0/1 (little-endian within a byte) -> uint8 [T, ceil(n / 8)]."""
    T, n = bits.shape
    pad = (-n) % 8
    if pad:
        bits = torch.nn.functional.pad(bits, (0, pad))
    w = (2 ** torch.arange(8, device=bits.device)).to(torch.int32)
    return (bits.view(T, -1, 8).to(torch.int32) * w).sum(-1).to(torch.uint8)


def encode_rows_torch(codec: str, x: torch.Tensor, value: bool = False) -> torch.Tensor:
    """Same bytes as :func:`encode_rows`, computed with tensor ops on x's device.  (The turbo3 sketch sums its
    projections in a different order than the C++ loop, so a bit whose projection is within rounding of zero can
    differ.)"""
    T, H, D = x.shape
    x = x.float()
    if value and codec in ("polar4", "turbo3"):
        codec = "int8"
    if codec == "bf16":
        return x.to(torch.bfloat16).contiguous().view(torch.uint8).view(T, -1)
    if codec == "fp8":
        return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).contiguous().view(torch.uint8).view(T, -1)
    if codec == "int8":
        return _int8_rows(x)
    flat = x.reshape(T, H * D)
    if codec == "int4":
        pad = (-flat.shape[1]) % 32
        g = torch.nn.functional.pad(flat, (0, pad)).view(T, -1, 32)
        mx = g.abs().amax(-1)
        sh = torch.where(mx == 0, torch.ones_like(mx), mx / 7.0).to(torch.float16)
        codes = _round_away(g * (1.0 / sh.float())[..., None]).clamp_(-7, 7).to(torch.int32) & 0xF
        packed = (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)
        return torch.cat([sh.contiguous().view(torch.uint8).view(T, -1, 2), packed], -1).reshape(T, -1)
    if codec == "polar4":
        row_bytes("polar4", H, D)
        q = torch.floor((flat.clamp(-1, 1) + 1.0) * 7.5 + 0.5).clamp_(0, 15).to(torch.int32)
        if q.shape[1] % 2:
            q = torch.nn.functional.pad(q, (0, 1))
        return (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)
    if codec == "turbo3":
        row_bytes("turbo3", H, D)
        q = torch.floor((flat.clamp(-1, 1) + 1.0) * 3.5 + 0.5).clamp_(0, 7).to(torch.int32)
        bits = ((q[..., None] >> torch.arange(3, device=x.device)) & 1).reshape(T, -1)
        base = _pack_bits(bits)
        resid = x - (q.view(T, H, D).float() / 3.5 - 1.0)
        proj = torch.einsum("thd,hpd->thp", resid, random_signs(H, D, x.device))
        return torch.cat([base, _pack_bits((proj >= 0).reshape(T, -1).to(torch.int32))], -1)
    raise ValueError(codec)


# ----------------------------------------------------------------------------------------------------------
# decode attention
# ----------------------------------------------------------------------------------------------------------
def attention_host(codec: str, q: torch.Tensor, k_rows: torch.Tensor, v_rows: torch.Tensor, Hkv: int,
                   scale: Optional[float] = None, k_scale: float = 1.0, v_scale: float = 1.0,
                   window: int = 0) -> torch.Tensor:
    """One sequence's decode step on the CPU: q [Hq, D] against token-major code rows -> fp32 [Hq, D]."""
    Hq, D = q.shape
    qf = q.detach().float().contiguous().cpu()
    k_rows, v_rows = k_rows.contiguous().cpu(), v_rows.contiguous().cpu()
    out = torch.empty((Hq, D), dtype=torch.float32)
    rc = _host().afb_kvq_attention_host(
        _c_int(CODECS[codec]), N.ptr(qf), N.ptr(k_rows), N.ptr(v_rows), _c_long(k_rows.shape[0]), _c_int(Hq),
        _c_int(Hkv), _c_int(D), _c_float(scale if scale is not None else 1.0 / math.sqrt(D)), _c_float(k_scale),
        _c_float(v_scale), _c_int(window), N.ptr(out))
    if rc != 0:
        raise ValueError(f"KV codec {codec!r}: unsupported shape")
    return out


def decode_attention(codec: str, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_tables: torch.Tensor, kv_lens: torch.Tensor, Hkv: int, scale: Optional[float] = None,
                     k_scale: float = 1.0, v_scale: float = 1.0, window: int = 0,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode attention of a batch over a paged quantised cache.

    q [B, Hq, D] bf16 (one new token per sequence); k_cache / v_cache uint8 [num_blocks, page, row_bytes];
    block_tables int32 [B, max_blocks]; kv_lens int32 [B] (tokens in the cache, the new one included).
    Returns bf16 [B, Hq, D]."""
    B, Hq, D = q.shape
    num_blocks, page = k_cache.shape[0], k_cache.shape[1]
    assert k_cache.dtype == torch.uint8 and v_cache.dtype == torch.uint8
    assert k_cache.shape[2] == row_bytes(codec, Hkv, D) and v_cache.shape[2] == row_bytes(codec, Hkv, D, True)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        res = torch.empty((B, Hq, D), dtype=torch.bfloat16)
        for b in range(B):
            n = int(kv_lens[b])
            t = torch.arange(n)
            rows = block_tables[b, t // page].long() * page + t % page
            res[b] = attention_host(codec, q[b], k_cache.view(num_blocks * page, -1)[rows],
                                    v_cache.view(num_blocks * page, -1)[rows], Hkv, scale, k_scale, v_scale,
                                    window).to(torch.bfloat16)
        return res
    assert q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == D
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and block_tables.is_contiguous()
    assert block_tables.dtype == torch.int32 and kv_lens.dtype == torch.int32
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=q.device)
    rc = N.cuda().afb_kvq_decode_attention(
        N.ptr(q), _c_long(q.stride(0)), N.ptr(k_cache), N.ptr(v_cache), N.ptr(block_tables),
        _c_int(block_tables.shape[1]), _c_int(page), _c_int(num_blocks), N.ptr(kv_lens), N.ptr(out),
        _c_long(out.stride(0)), _c_int(B), _c_int(Hq), _c_int(Hkv), _c_int(D), _c_int(CODECS[codec]),
        _c_int(window), _c_float(scale), _c_float(k_scale), _c_float(v_scale), N.stream_ptr())
    N.check(rc, "afb_kvq_decode_attention")
    N.count_launch()
    return out


class QuantizedPagedKV:
    """A paged KV cache of one layer stored in a quantised codec: byte tensors [num_blocks, page, row_bytes] for keys
    and for values, written token by token (encoded with tensor ops on the cache's device) and read by
    :func:`decode_attention`.  Memory per token against bf16: fp8 1/2, int8 ~1/2, int4 ~0.27, polar4 ~0.38,
    turbo3 ~0.33 of the bytes."""

    def __init__(self, codec: str, num_blocks: int, page: int, Hkv: int, D: int, device="cpu"):
        self.codec, self.page, self.Hkv, self.D = codec, page, Hkv, D
        self.k = torch.zeros((num_blocks, page, row_bytes(codec, Hkv, D)), dtype=torch.uint8, device=device)
        self.v = torch.zeros((num_blocks, page, row_bytes(codec, Hkv, D, True)), dtype=torch.uint8, device=device)

    def write(self, slots: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        """k / v [T, Hkv, D]; slots [T] = block * page + offset (negative: skip the token)."""
        keep = slots >= 0
        s = slots[keep].long()
        self.k.view(-1, self.k.shape[2])[s] = encode_rows_torch(self.codec, k[keep])
        self.v.view(-1, self.v.shape[2])[s] = encode_rows_torch(self.codec, v[keep], value=True)

    def attend(self, q: torch.Tensor, block_tables: torch.Tensor, kv_lens: torch.Tensor, **kw) -> torch.Tensor:
        return decode_attention(self.codec, q, self.k, self.v, block_tables, kv_lens, self.Hkv, **kw)

    def bytes_per_token(self) -> int:
        return self.k.shape[2] + self.v.shape[2]


# ----------------------------------------------------------------------------------------------------------
# Codec caches inside the generation engine
# ----------------------------------------------------------------------------------------------------------
def expand_rows(codec: str, cache_rows: torch.Tensor, row_idx: torch.Tensor, heads: int, D: int,
                value: bool = False, scale: float = 1.0) -> torch.Tensor:
    """Decodes code rows ``cache_rows[row_idx]`` (cache_rows uint8 [N, row_bytes]) to bf16 [n, heads, D]."""
    n = row_idx.numel()
    if not cache_rows.is_cuda:
        rows = cache_rows[row_idx.long().clamp_min(0)]
        return (decode_rows(codec, rows, heads, D, value) * scale).to(torch.bfloat16)
    out = torch.empty((n, heads, D), dtype=torch.bfloat16, device=cache_rows.device)
    rc = N.cuda().afb_kvq_expand_rows(N.ptr(cache_rows), N.ptr(row_idx.int().contiguous()), N.ptr(out), _c_long(n),
                                      _c_long(cache_rows.shape[0]), _c_int(heads), _c_int(D), _c_int(CODECS[codec]),
                                      _c_int(1 if value else 0), _c_float(scale), N.stream_ptr())
    N.check(rc, "afb_kvq_expand_rows")
    N.count_launch()
    return out


class CodecLayer:
    """One layer's keys (or values) of a paged cache kept in a quantised codec: bytes [num_blocks, page, row_bytes].
    The attention and KV-write wrappers (``ops.attention``) recognise this type where they otherwise take a
    bf16 cache tensor [num_blocks, page, Hkv, D]."""

    def __init__(self, codec: str, data: torch.Tensor, Hkv: int, D: int, value: bool):
        self.codec, self.data, self.Hkv, self.D, self.value = codec, data, Hkv, D, value

    @property
    def device(self):
        return self.data.device

    @property
    def is_cuda(self) -> bool:
        return self.data.is_cuda

    @property
    def page(self) -> int:
        return self.data.shape[1]

    @property
    def num_blocks(self) -> int:
        return self.data.shape[0]

    def rows(self) -> torch.Tensor:
        return self.data.view(-1, self.data.shape[2])

    def write(self, slots: torch.Tensor, x: torch.Tensor) -> None:
        """x [T, Hkv, D]; slots [T] = block * page + offset.  A negative slot (a padded token) is sent to the spare
        row behind the last block, so no data-dependent filtering -- and no host synchronisation -- is needed."""
        spare = self.data.shape[0] * self.data.shape[1] - 1
        s = torch.where(slots >= 0, slots, torch.full_like(slots, spare)).long()
        self.rows().index_copy_(0, s, encode_rows_torch(self.codec, x, value=self.value))

    def expand(self, row_idx: torch.Tensor) -> torch.Tensor:
        return expand_rows(self.codec, self.rows(), row_idx, self.Hkv, self.D, self.value)


class CodecCache:
    """All layers' keys (or values) in a codec: ``cache[l]`` is a :class:`CodecLayer`.  One spare block follows the
    allocator's blocks (the target of padded tokens' writes)."""

    def __init__(self, codec: str, n_layers: int, num_blocks: int, page: int, Hkv: int, D: int, device, value: bool):
        if codec not in CODECS:
            raise ValueError(f"unknown KV codec {codec!r}")
        self.codec, self.Hkv, self.D, self.value = codec, Hkv, D, value
        self.data = torch.zeros((n_layers, num_blocks + 1, page, row_bytes(codec, Hkv, D, value)), dtype=torch.uint8,
                                device=device)

    def __getitem__(self, l: int) -> CodecLayer:
        return CodecLayer(self.codec, self.data[l], self.Hkv, self.D, self.value)

    @property
    def shape(self):
        return self.data.shape

    def numel(self) -> int:
        return self.data.numel()

    def element_size(self) -> int:
        return 1

    @property
    def device(self):
        return self.data.device
