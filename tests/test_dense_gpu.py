"""GPU numerics: tcgen05 bf16 GEMM, norms, embedding lookups and pooling against the fp32 oracles."""
import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize(
    "M,N,K,tile",
    [
        (128, 64, 64, 64), (128, 128, 128, 128), (128, 256, 64, 256), (256, 512, 256, 0), (300, 200, 72, 0),
        (1000, 2304, 768, 0), (1024, 768, 3072, 0), (77, 3072, 768, 128), (4096, 1024, 1024, 256),
        (5, 40, 8, 64), (129, 257, 520, 128),
    ],
)
def test_gemm_plain(M, N, K, tile):
    from antfly_b200.ops import dense

    a = _rand(M, K, scale=1.0, seed=1)
    w = _rand(N, K, scale=K ** -0.5, seed=2)
    y = dense.gemm_bf16(a, w, tile_n=tile)
    ref = R.linear(a, w)
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("act", ["gelu", "gelu_tanh", "relu", "silu", None])
def test_gemm_epilogues(act):
    from antfly_b200.ops import dense

    M, N, K = 513, 1000, 768
    a = _rand(M, K, seed=3)
    w = _rand(N, K, scale=K ** -0.5, seed=4)
    b = _rand(N, seed=5)
    r = _rand(M, N, seed=6)
    y = dense.gemm_bf16(a, w, bias=b, act=act, residual=r)
    ref = R.linear(a, w, b, act, r)
    torch.testing.assert_close(y.float(), ref, atol=4e-2, rtol=2e-2)
    y32 = dense.gemm_bf16(a, w, bias=b, act=act, out_dtype=torch.float32, alpha=0.5)
    ref32 = R.linear(a, w, b, act, alpha=0.5)
    torch.testing.assert_close(y32, ref32, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_gemm_split_k_and_norm_consumer(splits):
    from antfly_b200.ops import dense

    M, N, K = 64, 1024, 4096
    a = _rand(M, K, seed=7)
    w = _rand(N, K, scale=K ** -0.5, seed=8)
    parts = dense.gemm_bf16(a, w, split_k=splits)
    assert parts.dtype == torch.float32 and parts.dim() == 3
    ref = R.linear(a, w)
    torch.testing.assert_close(parts.sum(0), ref, atol=1e-2, rtol=1e-2)
    res = _rand(M, N, seed=9)
    g = _rand(N, seed=10)
    s, y = dense.norm(None, g, None, eps=1e-5, rms=True, residual=res, partials=parts, want_sum=True)
    rs, ry = R.norm(None, g, None, eps=1e-5, rms=True, residual=res, partials=parts)
    torch.testing.assert_close(s.float(), rs, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(y.float(), ry, atol=4e-2, rtol=3e-2)


@pytest.mark.parametrize("H", [384, 768, 1024, 4096, 8192])
@pytest.mark.parametrize("rms", [False, True])
def test_norm(H, rms):
    from antfly_b200.ops import dense

    rows = 333
    x = _rand(rows, H, seed=11)
    r = _rand(rows, H, seed=12)
    g = _rand(H, seed=13)
    b = None if rms else _rand(H, seed=14)
    y = dense.norm(x, g, b, eps=1e-6, rms=rms)
    torch.testing.assert_close(y.float(), R.norm(x, g, b, eps=1e-6, rms=rms)[1], atol=3e-2, rtol=2e-2)
    s, y2 = dense.norm(x, g, b, eps=1e-6, rms=rms, residual=r, want_sum=True)
    rs, ry = R.norm(x, g, b, eps=1e-6, rms=rms, residual=r)
    torch.testing.assert_close(s.float(), rs, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(y2.float(), ry, atol=4e-2, rtol=3e-2)


def test_bert_embed_ln_and_gather():
    from antfly_b200.ops import dense

    T, H, V = 700, 768, 30522
    g = torch.Generator(device="cuda").manual_seed(0)
    ids = torch.randint(0, V, (T,), generator=g, device="cuda", dtype=torch.int32)
    pos = torch.randint(0, 512, (T,), generator=g, device="cuda", dtype=torch.int32)
    ty = torch.randint(0, 2, (T,), generator=g, device="cuda", dtype=torch.int32)
    word, ptab, ttab = _rand(V, H, seed=1), _rand(512, H, seed=2), _rand(2, H, seed=3)
    gam, bet = _rand(H, seed=4), _rand(H, seed=5)
    y = dense.bert_embed_ln(ids, pos, ty, word, ptab, ttab, gam, bet)
    ref = R.bert_embed_ln(ids, pos, ty, word, ptab, ttab, gam, bet)
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)
    e = dense.embed_gather(ids, word)
    assert torch.equal(e, word[ids.long()])


@pytest.mark.parametrize("mode", ["mean", "cls", "max", "last"])
def test_pool(mode):
    from antfly_b200.ops import dense

    H = 768
    lens = torch.tensor([5, 1, 128, 77, 512, 33], dtype=torch.int32)
    starts = torch.cumsum(lens, 0) - lens
    T = int(lens.sum())
    h = _rand(T, H, seed=21)
    out = dense.pool(h, starts.int().cuda(), lens.cuda(), mode=mode)
    ref = R.pool(h, starts, lens, mode=mode)
    torch.testing.assert_close(out, ref, atol=2e-3, rtol=2e-3)
    mask = (torch.rand(T, device="cuda") > 0.3).int()
    out = dense.pool(h, starts.int().cuda(), lens.cuda(), mode=mode, mask=mask)
    ref = R.pool(h, starts, lens, mode=mode, mask=mask)
    torch.testing.assert_close(out, ref, atol=2e-3, rtol=2e-3)


def test_maxsim_and_splade():
    from antfly_b200.ops import dense

    D = 128
    lens = torch.tensor([7, 40, 180], dtype=torch.int32)
    starts = (torch.cumsum(lens, 0) - lens).int()
    q = _rand(12, D, seed=30)
    d = _rand(int(lens.sum()), D, seed=31)
    out = dense.maxsim(q, d, starts.cuda(), lens.cuda())
    torch.testing.assert_close(out, R.maxsim(q, d, starts, lens), atol=2e-3, rtol=2e-3)
    logits = _rand(int(lens.sum()), 1000, seed=32)
    sp = dense.splade_pool(logits, starts.cuda(), lens.cuda())
    torch.testing.assert_close(sp, R.splade_pool(logits, starts, lens), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("H", [256, 768, 1024])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_warp_per_row_path(H, rms):
    """Many short rows take the warp-per-row kernel."""
    from antfly_b200.ops import dense

    rows = 4099
    x, r, g = _rand(rows, H, seed=41), _rand(rows, H, seed=42), _rand(H, seed=43)
    b = None if rms else _rand(H, seed=44)
    bias = _rand(H, seed=45)
    s, y = dense.norm(x, g, b, eps=1e-6, rms=rms, residual=r, bias=bias, want_sum=True)
    rs, ry = R.norm(x, g, b, eps=1e-6, rms=rms, residual=r, bias=bias)
    torch.testing.assert_close(s.float(), rs, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(y.float(), ry, atol=4e-2, rtol=3e-2)
