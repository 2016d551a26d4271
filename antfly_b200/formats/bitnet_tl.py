"""BitNet lookup-table weight layouts TL1 and TL2 of GGUF files written by the BitNet tool chain.

Unlike the block formats these are whole-tensor layouts: ternary weights are stored as 4-bit codes of value pairs
(TL1) or as 4-bit codes of value triples plus a sign bit (TL2), tiled for the lookup-table kernels by a per-shape
configuration (bm, by, bmm), and followed by one fp32 scale for the whole tensor.  Only the matrix shapes with a
preset tiling exist.  Layouts and presets follow the reference's reader
(zig/pkg/inference/src/gguf/quant_codec.zig:1347-1672; byte lengths zig/pkg/inference/src/gguf/tensor_types.zig:238-277).
Type ids: TL1 = 38; TL2 = 39 in files whose general.architecture is "bitnet" / "bitnet-b1.58" (39 is MXFP4 elsewhere).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import numpy as np

# (rows, cols) -> (bm, by, bmm)
TL1_CONFIGS: Dict[Tuple[int, int], Tuple[int, int, int]] = {
    (1536, 4096): (256, 128, 32), (1536, 1536): (128, 64, 64), (4096, 1536): (256, 128, 32),
    (3200, 8640): (160, 64, 32), (3200, 3200): (320, 128, 64), (8640, 3200): (320, 64, 32),
    (14336, 4096): (256, 128, 32), (4096, 14336): (128, 64, 64), (1024, 4096): (256, 128, 32),
    (4096, 4096): (128, 64, 64)}
TL2_CONFIGS: Dict[Tuple[int, int], Tuple[int, int, int]] = {
    (1536, 4096): (256, 96, 32), (1536, 1536): (128, 192, 32), (4096, 1536): (256, 96, 64),
    (3200, 8640): (160, 96, 32), (3200, 3200): (320, 96, 32), (8640, 3200): (320, 96, 32),
    (14336, 4096): (256, 96, 32), (4096, 14336): (128, 96, 32), (1024, 4096): (256, 96, 32),
    (4096, 4096): (128, 96, 32)}

# triple code -> three ternary values (codes 14 and 15 are unused); a set sign bit negates all three
_TRIPLES = np.array([[0, 0, 0], [0, 0, 1], [0, 1, -1], [0, 1, 0], [0, 1, 1], [1, -1, -1], [1, -1, 0], [1, -1, 1],
                     [1, 0, -1], [1, 0, 0], [1, 0, 1], [1, 1, -1], [1, 1, 0], [1, 1, 1], [0, 0, 0], [0, 0, 0]],
                    dtype=np.float32)


def tl1_nbytes(rows: int, cols: int) -> int:
    return -(-(rows * cols) // 4) + 32


def tl2_nbytes(rows: int, cols: int) -> int:
    ternary = (((cols - 256) * rows) // 3 * 5) // 8
    dense = ((256 * rows) // 2 * 4) // 8
    return (ternary + dense + 31) // 32 * 32 + 32


def _pair_values(code: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    return (code // 3 - 1).astype(np.float32), (code % 3 - 1).astype(np.float32)


def _swap_groups(g: np.ndarray) -> np.ndarray:
    """Row groups of eight are stored in the order 0, 2, 1, 3."""
    return np.where(g == 1, 2, np.where(g == 2, 1, g))


def dequantize_tl1(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    cfg = TL1_CONFIGS.get((rows, cols))
    if cfg is None:
        raise NotImplementedError(f"TL1 has no preset tiling for a {rows} x {cols} matrix")
    bm, by_, bmm = cfg
    packed_len = rows * cols // 4
    if raw.size < packed_len + 4:
        raise ValueError("TL1 tensor data is too short")
    scale = float(raw[packed_len:packed_len + 4].view("<f4")[0])
    row = np.arange(rows, dtype=np.int64)[:, None]
    pc = np.arange(cols // 2, dtype=np.int64)[None, :]
    row_outer, row_in_bm = row // bm, row % bm
    col_block, col_in_block = pc // (by_ // 2), pc % (by_ // 2)
    bm_block, row_in_bmm = row_in_bm // bmm, row_in_bm % bmm
    by = 256 // bmm
    by_block, pair_in_by = col_in_block // (by // 2), col_in_block % (by // 2)
    row16, bmm16 = row_in_bmm % 16, row_in_bmm // 16
    by4, nibble = pair_in_by // 2, pair_in_by % 2
    idx = ((((((row_outer * (cols // by_) + col_block) * (bm // bmm) + bm_block) * (by_ // by) + by_block)
             * (bmm // 16) + bmm16) * (by // 4) + by4) * 16 + row16)
    byte = raw[:packed_len][idx]
    code = np.where(nibble == 0, byte >> 4, byte & 0x0F).astype(np.int64)
    a, b = _pair_values(code)
    out = np.empty((rows, cols), dtype=np.float32)
    out[:, 0::2], out[:, 1::2] = a * scale, b * scale
    return out


def dequantize_tl2(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    cfg = TL2_CONFIGS.get((rows, cols))
    if cfg is None or cols < 256:
        raise NotImplementedError(f"TL2 has no preset tiling for a {rows} x {cols} matrix")
    bm, by_, bmm = cfg
    three_cols = cols - cols % by_
    two_cols = cols - three_cols
    if three_cols % 3 or two_cols % 2:
        raise NotImplementedError("TL2: column split does not divide into triples and pairs")
    v_len, s_len, t_len = rows * three_cols // 6, rows * three_cols // 24, rows * two_cols // 4
    scale_off = tl2_nbytes(rows, cols) - 32
    if v_len + s_len + t_len > scale_off or raw.size < scale_off + 4:
        raise ValueError("TL2 tensor data is too short")
    scale = float(raw[scale_off:scale_off + 4].view("<f4")[0])
    values, signs, twos = raw[:v_len], raw[v_len:v_len + s_len], raw[v_len + s_len:v_len + s_len + t_len]
    out = np.empty((rows, cols), dtype=np.float32)
    row = np.arange(rows, dtype=np.int64)[:, None]
    tc = np.arange(three_cols // 3, dtype=np.int64)[None, :]
    by = 192 // bmm
    row_outer, row_in_bm = row // bm, row % bm
    col_block, col_in_block = tc // (by_ // 3), tc % (by_ // 3)
    bm_block, row_in_bmm = row_in_bm // bmm, row_in_bm % bmm
    # codes
    by_block, triple_in_by = col_in_block // (by // 3), col_in_block % (by // 3)
    group, offset = _swap_groups(row_in_bmm // 8), row_in_bmm % 8
    base = ((row_outer * (cols // by_) + col_block) * (bm // bmm) + bm_block)
    idx = (base * (by_ // by) + by_block) * bmm + group * 8 + offset
    byte = values[idx]
    code = np.where(triple_in_by == 0, byte >> 4, byte & 0x0F).astype(np.int64)
    # signs
    sub_count = by // 3 * 4
    sign_block, sign_sub = col_in_block // sub_count, col_in_block % sub_count
    line = sign_sub * bmm + row_in_bmm
    bit_lane, half = line // (bmm // 2), line % (bmm // 2)
    bit_index = 15 - bit_lane
    sidx = (base * (by_ // (by * 4)) + sign_block) * bmm + half * 2 + bit_index // 8
    neg = ((signs[sidx] >> (bit_index % 8).astype(np.uint8)) & 1).astype(bool)
    tri = _TRIPLES[code] * np.where(neg, -1.0, 1.0)[..., None].astype(np.float32)
    out[:, :three_cols] = (tri * scale).reshape(rows, three_cols)
    if two_cols:
        if two_cols % 32:
            raise NotImplementedError("TL2: the pair tail must be a multiple of 32 columns")
        pc = np.arange(two_cols // 2, dtype=np.int64)[None, :]
        r_outer, r_in = row // 32, row % 32
        c_block, c_in = pc // 16, pc % 16
        b_block, pair_in = c_in // 2, c_in % 2
        grp, off = _swap_groups(r_in // 8), r_in % 8
        tidx = ((r_outer * (two_cols // 32) + c_block) * 8 + b_block) * 32 + grp * 8 + off
        tb = twos[tidx]
        pcode = np.where(pair_in == 0, tb >> 4, tb & 0x0F).astype(np.int64)
        a, b = _pair_values(pcode)
        out[:, three_cols + 0::2], out[:, three_cols + 1::2] = a * scale, b * scale
    return out
