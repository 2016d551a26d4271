"""Quantised KV-cache codecs (fp8 / int8 / int4 / polar4 / turbo3): row sizes, C++ encoders against an independent
torch restatement byte for byte, reconstruction error bounds, compressed-key decode attention against attention over
the dequantised cache, the turbo3 residual sketch improving score fidelity, and the paged cache wrapper."""
import math

import pytest
import torch

from antfly_b200.ops import kv_quant as KQ


def test_row_sizes_match_the_documented_layouts():
    # 8 KV heads of 128: the sizes the reference's pool tests state (pool.zig "asymmetric key and value row sizes")
    assert KQ.row_bytes("polar4", 8, 128) == 512
    assert KQ.row_bytes("polar4", 8, 128, value=True) == 1024 + 8 * 4
    assert KQ.row_bytes("turbo3", 8, 128) == 384 + 32
    assert KQ.row_bytes("turbo3", 8, 128, value=True) == 1024 + 8 * 4
    assert KQ.row_bytes("int8", 8, 128) == 8 * (128 + 4)
    assert KQ.row_bytes("int4", 8, 128) == (1024 // 32) * 18
    assert KQ.row_bytes("fp8", 8, 128) == 1024 and KQ.row_bytes("bf16", 8, 128) == 2048
    assert KQ.row_bytes("polar4", 8, 80) == 320 and KQ.row_bytes("polar4", 8, 256) == 1024
    with pytest.raises(ValueError):
        KQ.row_bytes("polar4", 8, 96)


@pytest.mark.parametrize("codec", ["bf16", "fp8", "int8", "int4", "polar4", "turbo3"])
@pytest.mark.parametrize("H,D", [(2, 64), (3, 80), (1, 128)])
def test_cpp_and_torch_encoders_agree(codec, H, D):
    g = torch.Generator().manual_seed(hash((codec, H, D)) % 1000)
    x = torch.randn(37, H, D, generator=g) * (0.5 if codec in ("polar4", "turbo3") else 3.0)
    x[5] = 0.0                                              # an all-zero row: scales fall back to 1
    for value in (False, True):
        a, b = KQ.encode_rows(codec, x, value), KQ.encode_rows_torch(codec, x, value)
        assert a.shape == b.shape == (37, KQ.row_bytes(codec, H, D, value))
        if codec == "turbo3" and not value:
            base = KQ.row_bytes("turbo3", H, D) - 4 * H
            assert torch.equal(a[:, :base], b[:, :base])
            diff = (a[:, base:] ^ b[:, base:]).to(torch.int32)
            flipped = sum(int(((diff >> k) & 1).sum()) for k in range(8))
            assert flipped <= 2                              # summation-order ties only
        else:
            assert torch.equal(a, b), (codec, value)


@pytest.mark.parametrize("codec,tol", [("bf16", 0.004), ("fp8", 0.07), ("int8", 0.005), ("int4", 0.08)])
def test_reconstruction_error(codec, tol):
    x = torch.randn(64, 4, 128, generator=torch.Generator().manual_seed(1))
    for value in (False, True):
        y = KQ.decode_rows(codec, KQ.encode_rows(codec, x, value), 4, 128, value)
        rel = (y - x).abs().amax(-1) / x.abs().amax(-1)
        assert float(rel.max()) <= tol, (codec, float(rel.max()))
    # fp8 decode agrees with torch's e4m3 for every finite byte
    allb = torch.arange(256, dtype=torch.uint8)
    mine = KQ.decode_rows("fp8", allb.view(1, 256), 2, 128)[0].flatten()
    ref = allb.view(torch.float8_e4m3fn).float()
    ok = ~ref.isnan()
    assert torch.equal(mine[ok], ref[ok]) and bool(mine[~ok].isnan().all())


def test_fixed_grid_key_codecs():
    x = torch.linspace(-1.2, 1.2, 128).view(1, 1, 128)
    p4 = KQ.decode_rows("polar4", KQ.encode_rows("polar4", x), 1, 128)
    t3 = KQ.decode_rows("turbo3", KQ.encode_rows("turbo3", x), 1, 128)
    xc = x.clamp(-1, 1)
    assert float((p4 - xc).abs().max()) <= 1 / 15 + 1e-6     # half a step of the 16-level grid
    assert float((t3 - xc).abs().max()) <= 1 / 7 + 1e-6      # half a step of the 8-level grid
    assert float(p4.min()) == -1.0 and float(p4.max()) == 1.0


def _ref_attention(q, k, v, Hkv, scale, window=0):
    Hq, D = q.shape
    g = Hq // Hkv
    if window > 0:
        k, v = k[-window:], v[-window:]
    kk = k.transpose(0, 1).repeat_interleave(g, 0)           # [Hq, T, D]
    vv = v.transpose(0, 1).repeat_interleave(g, 0)
    s = torch.einsum("hd,htd->ht", q, kk) * scale
    return torch.einsum("ht,htd->hd", s.softmax(-1), vv)


@pytest.mark.parametrize("codec", ["bf16", "fp8", "int8", "int4", "polar4"])
def test_host_attention_equals_attention_over_the_dequantised_cache(codec):
    g = torch.Generator().manual_seed(7)
    Hq, Hkv, D, T = 8, 2, 64, 150
    q = torch.randn(Hq, D, generator=g)
    k = torch.randn(T, Hkv, D, generator=g) * 0.4
    v = torch.randn(T, Hkv, D, generator=g)
    kr, vr = KQ.encode_rows(codec, k), KQ.encode_rows(codec, v, True)
    kd, vd = KQ.decode_rows(codec, kr, Hkv, D), KQ.decode_rows(codec, vr, Hkv, D, True)
    for window in (0, 40):
        got = KQ.attention_host(codec, q, kr, vr, Hkv, window=window)
        want = _ref_attention(q, kd, vd, Hkv, 1 / math.sqrt(D), window)
        torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
    # per-tensor scales of an fp8-style cache multiply scores and outputs
    got = KQ.attention_host(codec, q, kr, vr, Hkv, k_scale=0.5, v_scale=2.0)
    want = 2.0 * _ref_attention(q, 0.5 * kd, vd, Hkv, 1 / math.sqrt(D))
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)


def test_turbo3_sketch_brings_scores_closer_to_exact():
    g = torch.Generator().manual_seed(11)
    Hkv, D, T = 2, 128, 400
    k = (torch.randn(T, Hkv, D, generator=g) * 0.35).clamp(-1, 1)
    q = torch.randn(Hkv, D, generator=g)
    rows = KQ.encode_rows("turbo3", k)
    base = KQ.decode_rows("turbo3", rows, Hkv, D)
    exact = torch.einsum("hd,thd->th", q, k)
    s_base = torch.einsum("hd,thd->th", q, base)
    # residual term as the attention computes it: scale / 32 * sum_p sign_p(residual) * (signs_p . q)
    signs = KQ.random_signs(Hkv, D)
    pq = torch.einsum("hpd,hd->hp", signs, q)
    nb = KQ.row_bytes("turbo3", Hkv, D) - 4 * Hkv
    sk = rows[:, nb:].to(torch.int32)
    bits = torch.stack([(sk[:, i // 8] >> (i % 8)) & 1 for i in range(32 * Hkv)], 1).view(T, Hkv, 32)
    corr = KQ.RESIDUAL_SCALE / 32 * ((bits * 2 - 1).float() * pq[None]).sum(-1)
    err_base = (s_base - exact).pow(2).mean()
    err_corr = (s_base + corr - exact).pow(2).mean()
    assert float(err_corr) < float(err_base)
    # and the host attention uses exactly base + correction: a one-hot softmax check through the value path
    v = torch.randn(T, Hkv, D, generator=g)
    vr = KQ.encode_rows("turbo3", v, True)
    got = KQ.attention_host("turbo3", q, rows, vr, Hkv, scale=1.0)
    w = (s_base + corr).softmax(0)                            # [T, Hkv]
    want = torch.einsum("th,thd->hd", w, KQ.decode_rows("turbo3", vr, Hkv, D, True))
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("codec", ["fp8", "int4", "turbo3"])
def test_paged_quantised_cache_decode(codec):
    g = torch.Generator().manual_seed(3)
    B, Hq, Hkv, D, page, nblk = 3, 4, 2, 64, 16, 12
    cache = KQ.QuantizedPagedKV(codec, nblk, page, Hkv, D)
    lens = [5, 33, 48]
    perm = torch.randperm(nblk, generator=g)
    bt = torch.zeros((B, 3), dtype=torch.int32)
    ks, vs, off = [], [], 0
    for b, n in enumerate(lens):
        nb = (n + page - 1) // page
        bt[b, :nb] = perm[off: off + nb].int()
        off += nb
        k = torch.randn(n, Hkv, D, generator=g) * 0.4
        v = torch.randn(n, Hkv, D, generator=g)
        t = torch.arange(n)
        slots = bt[b, t // page].long() * page + t % page
        slots[0] = slots[0] if b else slots[0]
        cache.write(slots, k, v)
        ks.append(k), vs.append(v)
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16)
    out = cache.attend(q, bt, torch.tensor(lens, dtype=torch.int32))
    assert out.shape == (B, Hq, D) and out.dtype == torch.bfloat16
    for b in range(B):
        kr, vr = KQ.encode_rows_torch(codec, ks[b]), KQ.encode_rows_torch(codec, vs[b], True)
        want = KQ.attention_host(codec, q[b], kr, vr, Hkv)
        torch.testing.assert_close(out[b].float(), want, atol=1e-2, rtol=1e-2)
        # and the quantised result stays close to full-precision attention
        full = _ref_attention(q[b].float(), ks[b], vs[b], Hkv, 1 / math.sqrt(D))
        tol = {"fp8": 0.08, "int4": 0.2, "turbo3": 0.35}[codec]
        assert float((out[b].float() - full).abs().max()) < tol
    assert cache.bytes_per_token() < 2 * Hkv * D * 2
