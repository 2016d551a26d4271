"""GPU numerics: flash attention (varlen encoder, paged prefill, paged decode with split-KV), RoPE + KV write."""
import math

import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 12, 12), (128, 8, 2), (64, 6, 6)])
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_attention(D, Hq, Hkv, causal):
    from antfly_b200.ops import attention as A

    lens = torch.tensor([1, 17, 64, 65, 200, 512, 33], dtype=torch.int32)
    starts = (torch.cumsum(lens, 0) - lens).int()
    T = int(lens.sum())
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=1)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    out = A.varlen_attention(q, k, v, starts.cuda(), lens.cuda(), int(lens.max()), causal=causal)
    cu = torch.cat([starts, torch.tensor([T], dtype=torch.int32)])
    ref = R.varlen_attention(q, k, v, cu, causal=causal)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


def _build_paged(B, kv_lens, Hkv, D, page, seed):
    nblk_per = [(l + page - 1) // page for l in kv_lens]
    total = sum(nblk_per) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total, generator=g)
    max_blocks = max(nblk_per)
    bt = torch.zeros((B, max_blocks), dtype=torch.int32)
    off = 0
    for b, n in enumerate(nblk_per):
        bt[b, :n] = perm[off: off + n].int()
        off += n
    kc = _rand(total, page, Hkv, D, seed=seed + 1)
    vc = _rand(total, page, Hkv, D, seed=seed + 2)
    return kc, vc, bt.cuda()


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 32, 8), (64, 8, 8), (128, 8, 1)])
@pytest.mark.parametrize("splits", [1, 4])
def test_paged_decode(D, Hq, Hkv, splits):
    from antfly_b200.ops import attention as A

    kv_lens = [1, 15, 16, 17, 300, 2048, 777, 64]
    B = len(kv_lens)
    kc, vc, bt = _build_paged(B, kv_lens, Hkv, D, 16, seed=5)
    q = _rand(B, Hq, D, seed=9)
    q_starts = torch.arange(B, dtype=torch.int32, device="cuda")
    q_lens = torch.ones(B, dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    out = A.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl, 1, num_splits=splits)
    ref = R.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("window", [0, 100])
def test_paged_prefill_and_verify(window):
    from antfly_b200.ops import attention as A

    D, Hq, Hkv = 128, 16, 4
    kv_lens = [100, 5, 600, 64, 257]
    q_lens = [100, 5, 88, 1, 5]  # full prefill, short, chunk continuation, decode, spec-verify (k+1 = 5)
    B = len(kv_lens)
    kc, vc, bt = _build_paged(B, kv_lens, Hkv, D, 16, seed=11)
    T = sum(q_lens)
    q = _rand(T, Hq, D, seed=12)
    ql = torch.tensor(q_lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int().cuda()
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    out = A.paged_attention(q, kc, vc, bt, qs, ql.cuda(), kvl, max(q_lens), window=window)
    ref = R.paged_attention(q, kc, vc, bt, qs, ql.cuda(), kvl, sliding_window=window)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("half_split,rope_dim,norm", [(True, None, False), (False, 64, False), (True, None, True)])
def test_rope_kv_write(half_split, rope_dim, norm):
    from antfly_b200.ops import attention as A

    T, Hq, Hkv, D, page = 37, 8, 2, 128, 16
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=20)
    pos = torch.randint(0, 8192, (T,), device="cuda", dtype=torch.int32)
    nblocks = 8
    slots = torch.randperm(nblocks * page, device="cuda")[:T].int()
    slots[3] = -1
    kc = torch.zeros(nblocks, page, Hkv, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    qw = _rand(D, seed=21) if norm else None
    kw = _rand(D, seed=22) if norm else None
    q = A.rope_kv_write(qkv, pos, slots, kc, vc, Hq, Hkv, D, 500000.0, rope_dim=rope_dim, half_split=half_split,
                        q_norm_w=qw, k_norm_w=kw)
    kc2, vc2 = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    qr = A.rope_kv_write(qkv.cpu(), pos.cpu(), slots.cpu(), kc2, vc2, Hq, Hkv, D, 500000.0, rope_dim=rope_dim,
                         half_split=half_split, q_norm_w=None if qw is None else qw.cpu(),
                         k_norm_w=None if kw is None else kw.cpu())
    torch.testing.assert_close(q.float().cpu(), qr.float(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(kc.float().cpu(), kc2.float(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(vc.float().cpu(), vc2.float(), atol=1e-2, rtol=1e-2)
    # split-K partial input path gives the same result as the bf16 path on the same values
    parts = torch.stack([qkv.float() * 0.25, qkv.float() * 0.75])
    kc3, vc3 = torch.zeros_like(kc), torch.zeros_like(vc)
    q3 = A.rope_kv_write(None, pos, slots, kc3, vc3, Hq, Hkv, D, 500000.0, partials=parts, rope_dim=rope_dim,
                         half_split=half_split, q_norm_w=qw, k_norm_w=kw)
    torch.testing.assert_close(q3.float(), q.float(), atol=2e-2, rtol=2e-2)
    x = _rand(T, Hq, D, seed=23)
    xr = R.rope(x, pos, 10000.0, rope_dim, half_split)
    A.rope_(x, pos, 10000.0, rope_dim, half_split)
    torch.testing.assert_close(x.float(), xr, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("B,Hq,Hkv,ctx", [(64, 32, 8, 130), (6, 4, 1, 700)])
@pytest.mark.parametrize("terms", [1, 2])
def test_paged_decode_emits_mx_activations(B, Hq, Hkv, ctx, terms):
    """Split-KV decode whose merge kernel writes MX-fp8 context rows: same values as quantising the bf16 output.
    The two shapes cover the two- and three-deep tile rings (large and small grids)."""
    from antfly_b200.ops import attention as A
    from antfly_b200.ops import quant

    D = 128
    kv_lens = [ctx - (i % 7) for i in range(B)]
    kc, vc, bt = _build_paged(B, kv_lens, Hkv, D, 16, seed=11)
    q = _rand(B, Hq, D, seed=12)
    q_starts = torch.arange(B, dtype=torch.int32, device="cuda")
    q_lens = torch.ones(B, dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    ref = R.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl)
    out = A.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl, 1, num_splits=2)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    mx = A.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl, 1, num_splits=2, mx_terms=terms)
    assert isinstance(mx, quant.MxAct) and mx.terms == terms
    want = quant.quantize_mx(out.view(B, Hq * D), terms=terms)
    assert torch.equal(mx.q0, want.q0)
    torch.testing.assert_close(mx.dequant(), want.dequant(), atol=0, rtol=0)
    # unsplit: falls back to a quantisation pass, same contract
    mx1 = A.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl, 1, num_splits=1, mx_terms=terms)
    torch.testing.assert_close(mx1.dequant().view(B, Hq, D), ref, atol=3e-2 if terms == 2 else 1e-1, rtol=5e-2)


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (8, 1), (16, 1)])
def test_paged_decode_sliding_window_and_legacy_agree(Hq, Hkv):
    """Decode with a sliding window (masked first and last tiles) on both decode organisations: groups of up to 8
    rows take the transposed-MMA kernel, a group of 16 the 16-row one."""
    from antfly_b200.ops import attention as A

    D, window = 128, 100
    kv_lens = [1, 99, 100, 101, 333, 1500]
    B = len(kv_lens)
    kc, vc, bt = _build_paged(B, kv_lens, Hkv, D, 16, seed=21)
    q = _rand(B, Hq, D, seed=22)
    q_starts = torch.arange(B, dtype=torch.int32, device="cuda")
    q_lens = torch.ones(B, dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    ref = R.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl, None, window)
    for splits in (1, 3):
        out = A.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl, 1, window=window, num_splits=splits)
        torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
