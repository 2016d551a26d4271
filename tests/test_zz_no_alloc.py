"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate GPU memory when they need attention: a serving process whose
memory pool is fully committed to weights and KV cache, a latency-critical thread that must stay away from
cudaMalloc / cudaFree (both can synchronise the device), or a host program in another language that links the
shared object and has no tensor allocator.  For them the library carries its own fixed-size scratch.  This test
checks that the symbol gives the same answer as the regular entry point (whose scratch the caller allocates), on
two calls in a row -- the second call sees the first call's leftovers in the shared scratch -- and that an
oversized request is refused with a message instead of being run.

This file sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, ctx, Hq, Hkv, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    page = 16
    nblk = (ctx + page - 1) // page
    kc = torch.randn(B * nblk + 2, page, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
    vc = torch.randn(B * nblk + 2, page, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
    perm = torch.randperm(B * nblk + 2, generator=g, device="cuda")[: B * nblk].int()
    tables = perm.view(B, nblk).contiguous()
    q = torch.randn(B, Hq, D, generator=g, device="cuda").to(torch.bfloat16)
    kv_lens = torch.randint(1, ctx + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    kv_lens[0] = ctx
    return q, kc, vc, tables, kv_lens


def _call_noalloc(lib, q, kc, vc, tables, kv_lens, splits, q_starts=None):
    """q: [T, Hq, D] token slots; sequence b's single query token sits in slot q_starts[b] (default: slot b)."""
    T, Hq, D = q.shape
    B = tables.shape[0]
    Hkv, page = kc.shape[2], kc.shape[1]
    out = torch.full_like(q, float("nan"))
    ar = q_starts if q_starts is not None else torch.arange(B, dtype=torch.int32, device="cuda")
    ones = torch.ones(B, dtype=torch.int32, device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    fn = lib.afb_paged_decode_attention_noalloc
    fn.restype = ctypes.c_int
    rc = fn(vp(q), ctypes.c_long(q.stride(0)), vp(kc), vp(vc), vp(tables), ctypes.c_int(tables.shape[1]),
            ctypes.c_int(page), vp(ar), vp(ones), vp(kv_lens), vp(out), ctypes.c_long(out.stride(0)), ctypes.c_int(B),
            ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(D), ctypes.c_int(1), ctypes.c_int(0),
            ctypes.c_float(D ** -0.5), ctypes.c_int(splits),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_noalloc_entry_point_matches_regular_entry_point_twice_in_a_row():
    from antfly_b200 import _native
    from antfly_b200.ops import attention as A

    lib = _native.cuda()
    for call, (B, ctx, splits, seed) in enumerate([(8, 700, 4, 1), (5, 300, 3, 2)]):
        q, kc, vc, tables, kv_lens = _case(B, ctx, 32, 8, 128, seed)
        rc, got = _call_noalloc(lib, q, kc, vc, tables, kv_lens, splits)
        assert rc == 0, lib.afb_last_error()
        ar = torch.arange(B, dtype=torch.int32, device="cuda")
        ref = A.paged_attention(q, kc, vc, tables, ar, torch.ones_like(ar), kv_lens, 1, num_splits=splits)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all(), f"call {call}: output not fully written"
        torch.testing.assert_close(got.float(), ref.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("Hq,Hkv,D,splits", [(16, 1, 128, 3),   # 16 query heads per KV head: the 9..16-row kernel
                                             (16, 4, 64, 2), (8, 2, 256, 2),
                                             (32, 8, 128, 1)])  # one split: no scratch at all
def test_noalloc_entry_point_other_shapes_match_the_regular_entry_point(Hq, Hkv, D, splits):
    from antfly_b200 import _native
    from antfly_b200.ops import attention as A

    lib = _native.cuda()
    for B, ctx, seed in [(6, 500, 4), (3, 260, 5)]:
        q, kc, vc, tables, kv_lens = _case(B, ctx, Hq, Hkv, D, seed)
        rc, got = _call_noalloc(lib, q, kc, vc, tables, kv_lens, splits)
        assert rc == 0, lib.afb_last_error()
        ar = torch.arange(B, dtype=torch.int32, device="cuda")
        ref = A.paged_attention(q, kc, vc, tables, ar, torch.ones_like(ar), kv_lens, 1, num_splits=splits)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_noalloc_entry_point_padded_batch_rows_of_real_tokens_are_right():
    """More token slots than sequences (a padded batch): the rows that belong to a sequence must match; the slots
    that belong to none are documented as unspecified and are not looked at."""
    from antfly_b200 import _native
    from antfly_b200.ops import attention as A

    lib = _native.cuda()
    B, T, ctx, splits = 4, 9, 400, 3
    q, kc, vc, tables, kv_lens = _case(B, ctx, 32, 8, 128, 6)
    g = torch.Generator(device="cuda").manual_seed(7)
    q_slots = torch.randn(T, 32, 128, generator=g, device="cuda").to(torch.bfloat16)
    starts = torch.tensor([0, 2, 5, 7], dtype=torch.int32, device="cuda")
    q_slots[starts.long()] = q
    for _ in range(2):
        rc, got = _call_noalloc(lib, q_slots, kc, vc, tables, kv_lens, splits, q_starts=starts)
        assert rc == 0, lib.afb_last_error()
        ar = torch.arange(B, dtype=torch.int32, device="cuda")
        ref = A.paged_attention(q, kc, vc, tables, ar, torch.ones_like(ar), kv_lens, 1, num_splits=splits)
        torch.cuda.synchronize()
        torch.testing.assert_close(got[starts.long()].float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_noalloc_entry_point_single_split_has_no_row_limit():
    from antfly_b200 import _native

    lib = _native.cuda()
    q, kc, vc, tables, kv_lens = _case(300, 48, 32, 8, 128, 8)   # 300 * 32 = 9600 rows > 8192, but one split
    rc, got = _call_noalloc(lib, q, kc, vc, tables, kv_lens, 1)
    assert rc == 0, lib.afb_last_error()
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()


def test_noalloc_entry_point_rejects_oversized_requests():
    from antfly_b200 import _native

    lib = _native.cuda()
    q, kc, vc, tables, kv_lens = _case(64, 64, 32, 8, 128, 3)
    rc, _ = _call_noalloc(lib, q, kc, vc, tables, kv_lens, 8)  # 8 * 64 * 32 = 16384 rows > 8192
    assert rc != 0
    assert b"scratch" in lib.afb_last_error()
    torch.cuda.synchronize()
