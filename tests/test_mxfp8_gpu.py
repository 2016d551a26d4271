"""GPU numerics: MX-fp8 activation quantiser and the block-scaled tcgen05 GEMM against the fp32 oracle."""
import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("T,K", [(64, 4096), (5, 128), (130, 1024)])
def test_quantize_mx_matches_oracle_and_is_accurate(T, K):
    from antfly_b200.ops import quant

    x = _rand(T, K, seed=1) * torch.exp(_rand(T, 1, seed=2).float()).to(torch.bfloat16)
    g = quant.quantize_mx(x, terms=2)
    c = quant.quantize_mx(x.cpu(), terms=2)
    def rows(sf):  # scale bytes of the T real rows; the padding rows of the last atom are left undefined on the GPU
        tiles, chunks = sf.shape[0], sf.shape[1]
        return sf.cpu().view(tiles, chunks, 32, 4, 4).permute(1, 4, 0, 3, 2).reshape(chunks * 4, tiles * 128)[:, :T]

    assert torch.equal(g.q0.cpu(), c.q0) and torch.equal(rows(g.sf0), rows(c.sf0))
    d1 = quant.MxAct(g.q0, g.sf0).dequant()
    d2 = g.dequant()
    xf = x.float()
    rel1 = float((d1 - xf).norm() / xf.norm())
    rel2 = float((d2 - xf).norm() / xf.norm())
    assert rel1 < 0.04 and rel2 < 0.003, (rel1, rel2)


@pytest.mark.parametrize("M,N,K", [(64, 128, 128), (64, 256, 4096), (1, 512, 1024), (16, 1024, 2048),
                                   (33, 384, 256), (100, 4096, 4096), (64, 1008, 14336), (300, 512, 1024)])
@pytest.mark.parametrize("terms", [1, 2])
def test_gemm_mxfp8(M, N, K, terms):
    from antfly_b200.ops import quant

    x = _rand(M, K, seed=3)
    w = _rand(N, K, scale=K ** -0.5, seed=4)
    pw = quant.pack_fp8(w)
    xq = quant.quantize_mx(x, terms=terms)
    y = quant.gemm_mxfp8(xq, pw)
    ref = R.linear(xq.dequant(), R.dequantize_block_fp8(pw.q, pw.scales))
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)
    # and against the un-quantised activations: one term is fp8-accurate, two terms bf16-accurate
    exact = R.linear(x, R.dequantize_block_fp8(pw.q, pw.scales))
    err = float((y.float() - exact).norm() / exact.norm())
    assert err < (0.05 if terms == 1 else 0.012), err


def test_gemm_mxfp8_modes():
    from antfly_b200.ops import quant

    M, K, F = 64, 1024, 1536
    x = _rand(M, K, seed=5)
    xq = quant.quantize_mx(x, terms=2)
    gate, up = _rand(F, K, scale=K ** -0.5, seed=6), _rand(F, K, scale=K ** -0.5, seed=7)
    pw = quant.pack_fp8_swiglu(gate, up)
    y = quant.gemm_mxfp8(xq, pw, swiglu=True)
    ref = R.swiglu_interleaved(R.linear(xq.dequant(), R.dequantize_block_fp8(pw.q, pw.scales)))
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=3e-2)
    w = quant.pack_fp8(_rand(512, K, scale=K ** -0.5, seed=8))
    full = R.linear(xq.dequant(), R.dequantize_block_fp8(w.q, w.scales))
    for s in (1, 2, 4, 8):
        parts = quant.gemm_mxfp8(xq, w, split_k=s, partials=True)
        torch.testing.assert_close(parts.sum(0), full, atol=1e-2, rtol=1e-2)
    b, r = _rand(512, seed=9), _rand(M, 512, seed=10)
    y = quant.gemm_mxfp8(xq, w, bias=b, act="silu", residual=r)
    torch.testing.assert_close(y.float(), R.linear(xq.dequant(), R.dequantize_block_fp8(w.q, w.scales), b, "silu", r),
                               atol=4e-2, rtol=2e-2)


@pytest.mark.parametrize("T,F,S", [(64, 1792, 3), (5, 128, 1), (130, 1024, 8)])
@pytest.mark.parametrize("terms", [1, 2])
def test_swiglu_quantize_from_partials(T, F, S, terms):
    """SwiGLU + MX quantisation over split-K slices of an interleaved gate/up GEMM vs the fp32 reference."""
    from antfly_b200.ops import quant

    g = torch.Generator(device="cuda").manual_seed(3)
    parts = torch.randn(S, T, 2 * F, generator=g, device="cuda") * 0.7
    ref = R.swiglu_interleaved(parts.sum(0))
    mx, y = quant.swiglu_quantize_mx(parts, terms=terms, want_bf16=True)
    torch.testing.assert_close(y.float(), ref, atol=2e-2, rtol=1e-2)
    tol = 1e-2 if terms == 2 else 8e-2
    torch.testing.assert_close(mx.dequant(), ref, atol=tol, rtol=tol)
    # the CPU route of the same op agrees with the kernel's bf16 rows
    mx_cpu, y_cpu = quant.swiglu_quantize_mx(parts.cpu(), terms=terms, want_bf16=True)
    torch.testing.assert_close(y_cpu.float(), y.float().cpu(), atol=2e-2, rtol=1e-2)
