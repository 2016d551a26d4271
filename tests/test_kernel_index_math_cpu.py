"""Index arithmetic of CUDA kernels restated on the host (no GPU needed): the shared-memory layout the attention
kernel's tile loader writes must be the one its ldmatrix reads expect, for every head width it is built for."""
import pytest


@pytest.mark.parametrize("D", [64, 128, 256])
def test_attention_kv_tile_swizzle_loader_matches_readers(D):
    TILE_KEYS, THREADS = 64, 128
    CH = D // 8                              # 16-byte chunks per row
    RPP = THREADS // CH                      # rows covered by one pass of the 128 threads
    assert TILE_KEYS % RPP == 0
    where = {}                               # (row, chunk) -> element offset in the tile, as the loader computes it
    for tid in range(THREADS):
        ch, r0 = tid % CH, tid // CH
        dst0 = r0 * D + ((ch ^ (r0 & 7)) * 8)
        for i in range(TILE_KEYS // RPP):
            row = r0 + i * RPP
            dst = dst0 + i * RPP * D if RPP % 8 == 0 else row * D + ((ch ^ (row & 7)) * 8)
            assert (row, ch) not in where
            where[(row, ch)] = dst
    assert len(where) == TILE_KEYS * CH
    offs = sorted(where.values())
    assert offs == [8 * i for i in range(TILE_KEYS * CH)]                 # a bijection onto the tile, 16-byte aligned
    for key in range(TILE_KEYS):
        for chunk in range(CH):
            assert where[(key, chunk)] == key * D + ((chunk ^ (key & 7)) * 8)   # the readers' address


# ---------------------------------------------------------------------------------------------------------------
# Tensor-core attention (csrc/kernels/attention_tc.cu): the bytes a TMA box with the 128-byte swizzle leaves in shared
# memory must be the bytes the matrix descriptors make the MMA fetch -- K-major for Q and K, MN-major for V -- and
# the packed-bf16 P tile must sit where the A-from-tensor-memory operand of step kk starts.
# ---------------------------------------------------------------------------------------------------------------
def _tma_sw128_offset(row, col_elem):
    """Byte offset, inside a box destination that is 1024-byte aligned, of bf16 element (row, col) of a
    [rows x 64] box written with SWIZZLE_128B: rows of 128 bytes, 16-byte chunk index XOR (row mod 8)."""
    chunk, within = (col_elem * 2) // 16, (col_elem * 2) % 16
    return row * 128 + ((chunk ^ (row & 7)) * 16) + within


def _k_major_fetch(base, row, k):
    """Where a K-major SWIZZLE_128B descriptor (8-row groups 1024 bytes apart, start address advanced by 32 bytes
    per 16-element K step) finds element (row, k) of a [rows x 64] tile."""
    kstep, kin = k // 16, k % 16
    start = base + 32 * kstep                      # the descriptor's start address for this K step
    # the hardware applies the swizzle to the final address bits: chunk = address bits [4,7) XOR row-in-group
    addr = start + (row // 8) * 1024 + (row % 8) * 128 + kin * 2
    chunk = (addr >> 4) & 7
    return (addr & ~0x70) | ((chunk ^ (row % 8)) << 4)


def _mn_major_fetch(base, n, k, lbo):
    """MN-major SWIZZLE_128B descriptor: element (n, k) -- n along the contiguous dimension -- lives in panel
    n // 64 (panels lbo bytes apart), K row k (rows 128 bytes apart, 8-row groups 1024 = SBO apart), 16-byte
    chunk (n % 64) // 8 XOR (k mod 8)."""
    panel, nin = n // 64, n % 64
    return base + panel * lbo + (k // 8) * 1024 + (k % 8) * 128 + (((nin // 8) ^ (k % 8)) * 16) + (nin % 8) * 2


@pytest.mark.parametrize("D,BN", [(64, 128), (128, 64)])
def test_attention_tc_operand_layouts_agree_with_tma_boxes(D, BN):
    panels = D // 64
    # Q / K: panel pn of a tile holds columns [64 pn, 64 pn + 64) of every row, as one box (or BN / page boxes)
    for rows, boxes in ((128, 1), (BN, 1), (BN, BN // 16)):
        box_rows = rows // boxes
        panel_bytes = rows * 128
        for pn in range(panels):
            for row in range(0, rows, 5):
                for k in range(64):
                    bx, r_in = row // box_rows, row % box_rows
                    written = pn * panel_bytes + bx * box_rows * 128 + _tma_sw128_offset(r_in, k)
                    assert box_rows % 8 == 0                                   # boxes start on swizzle-atom boundaries
                    assert written == _k_major_fetch(pn * panel_bytes, row, k)
    # V: B operand of O += P V is [N = D, K = keys], fetched 16 keys per instruction from base + kk * 2048
    lbo = BN * 128
    for key in range(BN):
        for d in range(0, D, 3):
            pn, col = d // 64, d % 64
            written = pn * lbo + _tma_sw128_offset(key, col)
            kk, kin = key // 16, key % 16
            assert written == _mn_major_fetch(kk * 2048, d, kin, lbo)
    # P: two bf16 keys per 32-bit column; the A operand of key step kk starts at column 8 kk, and the softmax pass
    # over S columns [c, c + 32) writes P columns [c / 2, c / 2 + 16): never a column it still has to read
    for c in range(0, BN, 32):
        assert (c >> 1) + 16 <= c + 32 and (c >> 1) + 16 <= max(c, 16)
        for i in range(16):
            key_lo = c + 2 * i
            assert (key_lo // 16) * 8 + (key_lo % 16) // 2 == (c >> 1) + i
    # tensor-memory budget: S (BN) + O (D) inside the 256 allocated columns, two CTAs per SM
    assert BN + D <= 256


def test_attention_tc_tile_ranges_and_masks_match_the_reference_masks():
    """The per-CTA key-tile range and the per-row [k_beg, k_end) interval of attention_tc.cu, against the mask of
    ops/reference.py: causal / bidirectional, with and without a window, with a cache prefix (pos_off > 0)."""
    import itertools

    def kernel_visible(q_len, kv_len, causal, window, BN, qi, key):
        pos_off = kv_len - q_len
        q0 = (qi // 128) * 128
        q_last = min(q_len, q0 + 128) - 1
        kv_hi = kv_len
        if causal:
            kv_hi = min(kv_len, pos_off + q_last + 1)
        elif window > 0:
            kv_hi = min(kv_len, pos_off + q_last + window)
        kv_lo = max(0, pos_off + q0 - window + 1) if window > 0 else 0
        tile_lo, tile_hi = kv_lo // BN, (kv_hi + BN - 1) // BN
        if not (tile_lo * BN <= key < tile_hi * BN):
            return False
        qpos = pos_off + qi
        k_end = kv_len
        if causal:
            k_end = min(k_end, qpos + 1)
        elif window > 0:
            k_end = min(k_end, qpos + window)
        k_beg = max(0, qpos - window + 1) if window > 0 else 0
        return k_beg <= key < k_end

    def reference_visible(q_len, kv_len, causal, window, qi, key):
        qpos = kv_len - q_len + qi
        ok = key <= qpos if causal else True
        if window > 0:
            ok = ok and key > qpos - window
            if not causal:
                ok = ok and key < qpos + window
        return ok and key < kv_len

    for q_len, extra, causal, window, BN in itertools.product((1, 100, 128, 300), (0, 77), (True, False), (0, 50, 200),
                                                              (64, 128)):
        kv_len = q_len + extra
        if not causal and extra:
            continue                         # bidirectional attention is the packed (no cache prefix) case
        for qi in range(0, q_len, 37):
            for key in range(0, kv_len, 11):
                assert kernel_visible(q_len, kv_len, causal, window, BN, qi, key) == \
                    reference_visible(q_len, kv_len, causal, window, qi, key), (q_len, kv_len, causal, window, qi, key)
