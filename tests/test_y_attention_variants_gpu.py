"""GPU numerics of the attention variants: two-sided windows, sink logits, soft caps, ALiBi slopes, head widths outside
the tensor-core set."""
import math

import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("window", [9, 65, 300])
def test_varlen_attention_two_sided_window(window):
    """Bidirectional local attention (|key - query| < window), fused-QKV views with RoPE applied in place on the
    strided Q / K heads: the local layers of ModernBERT-style encoders."""
    from antfly_b200.ops import attention as A

    D, Hh = 64, 6
    lens = torch.tensor([1, 17, 64, 130, 257, 512, 33], dtype=torch.int32)
    starts = (torch.cumsum(lens, 0) - lens).int()
    T = int(lens.sum())
    qkv = _rand(T, 3 * Hh * D, seed=5)
    pos = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in lens]).cuda()
    ref_qk = R.rope(qkv[:, : 2 * Hh * D].reshape(T, 2 * Hh, D).cpu(), pos.cpu(), 10000.0)
    A.rope_(qkv[:, : 2 * Hh * D].view(T, 2 * Hh, D), pos, 10000.0)
    torch.testing.assert_close(qkv[:, : 2 * Hh * D].float().cpu().view(T, 2 * Hh, D), ref_qk, atol=3e-2, rtol=2e-2)
    q = qkv[:, : Hh * D].view(T, Hh, D)
    k = qkv[:, Hh * D: 2 * Hh * D].view(T, Hh, D)
    v = qkv[:, 2 * Hh * D:].view(T, Hh, D)
    out = A.varlen_attention(q, k, v, starts.cuda(), lens.cuda(), int(lens.max()), causal=False, window=window)
    cu = torch.cat([starts, torch.tensor([T], dtype=torch.int32)])
    ref = R.varlen_attention(q, k, v, cu, causal=False, window=window)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 64), (4, 4, 128), (6, 3, 80), (4, 1, 256)])
@pytest.mark.parametrize("sinks,softcap,window", [(True, 0.0, 0), (False, 30.0, 0), (True, 20.0, 37)])
def test_sink_softcap_attention_kernel_matches_fp32_reference(Hq, Hkv, D, sinks, softcap, window):
    """afb_attention_sink (one warp per (token, head), sink logit and tanh cap inside the softmax) on mixed prefill /
    decode rows against the fp32 oracle; an out-of-range block id is skipped and reported."""
    import torch

    from antfly_b200 import _native as N
    from antfly_b200.ops import attention as A
    from antfly_b200.ops import reference as R

    g = torch.Generator().manual_seed(Hq * 31 + D)
    page, nblk = 16, 64
    q_lens = [1, 40, 1, 150, 3]
    kv_lens = [1, 40, 300, 150, 131]
    B = len(q_lens)
    T = sum(q_lens)
    kc = (torch.randn(nblk, page, Hkv, D, generator=g) * 0.5).to(torch.bfloat16)
    vc = torch.randn(nblk, page, Hkv, D, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nblk, generator=g)
    bt = torch.zeros((B, 20), dtype=torch.int32)
    off = 0
    for b, n in enumerate(kv_lens):
        nb = (n + page - 1) // page
        bt[b, :nb] = perm[off: off + nb].int()
        off += nb
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    ql = torch.tensor(q_lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int()
    kl = torch.tensor(kv_lens, dtype=torch.int32)
    sk = torch.randn(Hq, generator=g) if sinks else None
    got = A.paged_attention_sink(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), qs.cuda(), ql.cuda(), kl.cuda(),
                                 window=window, sinks=sk.cuda() if sinks else None, softcap=softcap)
    assert N.status() == 0
    want = R.paged_attention(q, kc, vc, bt, qs, ql, kl, D ** -0.5, window, sinks=sk, softcap=softcap)
    torch.testing.assert_close(got.float().cpu(), want, atol=2e-2, rtol=2e-2)
    bad = bt.clone()
    bad[2, 3] = nblk + 7
    out = A.paged_attention_sink(q.cuda(), kc.cuda(), vc.cuda(), bad.cuda(), qs.cuda(), ql.cuda(), kl.cuda(),
                                 sinks=sk.cuda() if sinks else None, softcap=softcap)
    assert N.status() & 32 and bool(torch.isfinite(out.float()).all())


@pytest.mark.gpu
@pytest.mark.parametrize("Hq,Hkv,D,window", [(8, 8, 64, 0), (16, 16, 128, 0), (6, 2, 80, 29)])
def test_alibi_position_bias_in_the_attention_kernel(Hq, Hkv, D, window):
    """Per-head slopes times (key position - query position) are added to the scores inside afb_attention_sink; mixed
    prefill / decode rows against the fp32 oracle."""
    import torch

    from antfly_b200 import _native as N
    from antfly_b200.ops import attention as A
    from antfly_b200.ops import reference as R

    g = torch.Generator().manual_seed(Hq + D)
    page, nblk = 16, 48
    q_lens, kv_lens = [1, 33, 5, 130], [200, 33, 70, 130]
    B, T = len(q_lens), sum(q_lens)
    kc = (torch.randn(nblk, page, Hkv, D, generator=g) * 0.5).to(torch.bfloat16)
    vc = torch.randn(nblk, page, Hkv, D, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nblk, generator=g)
    bt = torch.zeros((B, 16), dtype=torch.int32)
    off = 0
    for b, n in enumerate(kv_lens):
        nb = (n + page - 1) // page
        bt[b, :nb] = perm[off: off + nb].int()
        off += nb
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    ql = torch.tensor(q_lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int()
    kl = torch.tensor(kv_lens, dtype=torch.int32)
    slopes = R.alibi_slopes(Hq)
    got = A.paged_attention_sink(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), qs.cuda(), ql.cuda(), kl.cuda(),
                                 window=window, alibi=slopes.cuda())
    assert N.status() == 0
    want = R.paged_attention(q, kc, vc, bt, qs, ql, kl, D ** -0.5, window, alibi=slopes)
    torch.testing.assert_close(got.float().cpu(), want, atol=2e-2, rtol=2e-2)
    plain = R.paged_attention(q, kc, vc, bt, qs, ql, kl, D ** -0.5, window)
    assert (want - plain).abs().max() > 1e-2                       # the bias does change the result


@pytest.mark.gpu
@pytest.mark.parametrize("D", [80, 96])
def test_paged_attention_with_head_widths_outside_the_tensor_core_set(D):
    """80- and 96-wide heads go through the general kernel at their own width (prefill rows and decode rows)."""
    import torch

    from antfly_b200.ops import attention as A
    from antfly_b200.ops import reference as R

    g = torch.Generator().manual_seed(D)
    Hq, Hkv, page, nblk = 8, 4, 16, 32
    q_lens, kv_lens = [1, 33, 1], [70, 33, 5]
    kc = (torch.randn(nblk, page, Hkv, D, generator=g) * 0.5).to(torch.bfloat16)
    vc = torch.randn(nblk, page, Hkv, D, generator=g).to(torch.bfloat16)
    bt = torch.randperm(nblk, generator=g).int()[:15].view(3, 5)
    q = torch.randn(sum(q_lens), Hq, D, generator=g).to(torch.bfloat16)
    ql = torch.tensor(q_lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int()
    kl = torch.tensor(kv_lens, dtype=torch.int32)
    got = A.paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), qs.cuda(), ql.cuda(), kl.cuda(), 33)
    want = R.paged_attention(q, kc, vc, bt, qs, ql, kl, D ** -0.5, 0)
    torch.testing.assert_close(got.float().cpu(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("kind", ["llama3", "yarn"])
def test_rope_kv_write_with_a_frequency_table(kind):
    """Context-extension schemes: the kernel reads rope_dim / 2 frequencies from a table and scales cos / sin by the
    scheme's attention factor; against the fp32 formula, and different from the closed-form rotation."""
    from antfly_b200.models.rope_scaling import rope_frequencies
    from antfly_b200.ops import attention as A

    T, Hq, Hkv, D, page = 29, 8, 2, 128, 16
    rope = {"llama3": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                       "original_max_position_embeddings": 8192},
            "yarn": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 4096}}[kind]
    inv, ms = rope_frequencies(rope, 500000.0, D, 131072)
    table = torch.tensor(inv, dtype=torch.float32)
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=30)
    pos = torch.randint(0, 100000, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(8 * page, device="cuda")[:T].int()
    kc = torch.zeros(8, page, Hkv, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q = A.rope_kv_write(qkv, pos, slots, kc, vc, Hq, Hkv, D, 500000.0, inv_freq=table.cuda(), rope_mscale=ms)
    kc2, vc2 = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    qr = A.rope_kv_write(qkv.cpu(), pos.cpu(), slots.cpu(), kc2, vc2, Hq, Hkv, D, 500000.0, inv_freq=table,
                         rope_mscale=ms)
    torch.testing.assert_close(q.float().cpu(), qr.float(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(kc.float().cpu(), kc2.float(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(vc.float().cpu(), vc2.float(), atol=1e-2, rtol=1e-2)
    plain = A.rope_kv_write(qkv, pos, slots, torch.zeros_like(kc), torch.zeros_like(vc), Hq, Hkv, D, 500000.0)
    assert float((plain.float() - q.float()).abs().max()) > 0.5
