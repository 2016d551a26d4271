"""GPU numerics: block-scaled fp8 weight GEMM (tcgen05, in-kernel dequant) against the fp32 oracle."""
import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize(
    "M,N,K", [(64, 128, 64), (64, 256, 4096), (1, 512, 1024), (16, 1024, 2048), (33, 384, 96), (100, 4096, 4096),
              (700, 512, 1024), (64, 1008, 14336)]
)
def test_w8a16_plain(M, N, K):
    from antfly_b200.ops import quant

    x = _rand(M, K, seed=1)
    w = _rand(N, K, scale=K ** -0.5, seed=2)
    pw = quant.pack_fp8(w)
    y = quant.gemm_w8a16(x, pw)
    ref = R.linear_w8(x, pw.q, pw.scales)
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)
    # the quantised weight itself is close to the original
    assert (R.dequantize_block_fp8(pw.q, pw.scales) - w.float()).abs().max() < 0.07 * w.float().abs().max()


def test_w8a16_epilogues_and_splitk():
    from antfly_b200.ops import quant

    M, N, K = 64, 1024, 4096
    x = _rand(M, K, seed=3)
    w = _rand(N, K, scale=K ** -0.5, seed=4)
    b = _rand(N, seed=5)
    r = _rand(M, N, seed=6)
    pw = quant.pack_fp8(w)
    y = quant.gemm_w8a16(x, pw, bias=b, act="silu", residual=r)
    torch.testing.assert_close(y.float(), R.linear_w8(x, pw.q, pw.scales, b, "silu", r), atol=4e-2, rtol=2e-2)
    for s in (1, 2, 4, 7):
        parts = quant.gemm_w8a16(x, pw, split_k=s, partials=True)
        torch.testing.assert_close(parts.sum(0), R.linear_w8(x, pw.q, pw.scales), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("M", [8, 64, 300])
def test_w8a16_swiglu(M):
    from antfly_b200.ops import quant

    K, F = 1024, 1536
    x = _rand(M, K, seed=7)
    gate = _rand(F, K, scale=K ** -0.5, seed=8)
    up = _rand(F, K, scale=K ** -0.5, seed=9)
    pw = quant.pack_fp8_swiglu(gate, up)
    y = quant.gemm_w8a16(x, pw, swiglu=True)
    ref = R.swiglu_interleaved(R.linear_w8(x, pw.q, pw.scales))
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=3e-2)


def test_random_fp8_weight_statistics():
    from antfly_b200.ops import quant

    pw = quant.random_fp8(256, 4096, "cuda", seed=1)
    w = R.dequantize_block_fp8(pw.q, pw.scales)
    assert torch.isfinite(w).all()
    assert 0.3 < float(w.std()) * 4096 ** 0.5 < 3.0
