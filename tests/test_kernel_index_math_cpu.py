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
