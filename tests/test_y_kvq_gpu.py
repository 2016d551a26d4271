"""Decode attention over quantised paged KV caches on the GPU against the C++ host attention over the same bytes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("codec", ["bf16", "fp8", "int8", "int4", "polar4", "turbo3"])
@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (8, 8, 64), (8, 1, 80), (4, 2, 256)])
def test_quantised_decode_attention_matches_host(codec, Hq, Hkv, D):
    from antfly_b200 import _native as N
    from antfly_b200.ops import kv_quant as KQ

    g = torch.Generator().manual_seed(Hq + D)
    B, page, nblk = 5, 16, 40
    lens = [1, 3, 64, 130, 277]
    perm = torch.randperm(nblk, generator=g)
    bt = torch.zeros((B, 18), dtype=torch.int32)
    cache = KQ.QuantizedPagedKV(codec, nblk, page, Hkv, D, device="cuda")
    off = 0
    for b, n in enumerate(lens):
        nb = (n + page - 1) // page
        bt[b, :nb] = perm[off: off + nb].int()
        off += nb
        k = torch.randn(n, Hkv, D, generator=g) * 0.4
        v = torch.randn(n, Hkv, D, generator=g)
        t = torch.arange(n)
        slots = bt[b, t // page].long() * page + t % page
        cache.write(slots.cuda(), k.cuda(), v.cuda())
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16)
    kv_lens = torch.tensor(lens, dtype=torch.int32)
    for window in (0, 50):
        out = cache.attend(q.cuda(), bt.cuda(), kv_lens.cuda(), window=window)
        assert N.status() == 0
        want = KQ.decode_attention(codec, q, cache.k.cpu(), cache.v.cpu(), bt, kv_lens, Hkv, window=window)
        torch.testing.assert_close(out.float().cpu(), want.float(), atol=2e-2, rtol=2e-2)


def test_bad_block_id_is_skipped_and_reported():
    from antfly_b200 import _native as N
    from antfly_b200.ops import kv_quant as KQ

    cache = KQ.QuantizedPagedKV("int8", 4, 16, 2, 64, device="cuda")
    q = torch.randn(1, 4, 64).to(torch.bfloat16).cuda()
    bt = torch.tensor([[1, 99]], dtype=torch.int32).cuda()       # second block id is out of range
    out = cache.attend(q, bt, torch.tensor([20], dtype=torch.int32).cuda())
    assert N.status() & 32                                         # the bad-index code; the keys were skipped
    assert bool(torch.isfinite(out.float()).all())
