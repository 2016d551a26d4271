"""GPU numerics: gated MLP activation kernel and the quick-GELU epilogue of the bf16 GEMMs."""
import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_tanh", "relu", "quick_gelu", "relu2"])
@pytest.mark.parametrize("T,F,interleaved,limit", [(5, 256, False, 0.0), (130, 1024, True, 0.0), (33, 200, False, 7.0),
                                                   (7, 37, True, 0.0), (64, 4096, False, 0.0)])
def test_gated_activation_kernel_matches_fp32_reference(act, T, F, interleaved, limit):
    """afb_gated_act: both layouts, the vector and the scalar path (F = 37: odd width; a sliced input whose base is
    not 16-byte aligned), the clamp, against the fp32 formula."""
    import torch

    from antfly_b200.ops import dense as Dn
    from antfly_b200.ops import reference as R

    g = torch.Generator().manual_seed(T * 7 + F)
    gu = (torch.randn(T, 2 * F, generator=g) * 3).to(torch.bfloat16)
    want = R.gated_act(gu, act, interleaved, limit)
    got = Dn.gated_act(gu.cuda(), act, interleaved, limit)
    assert got.dtype == torch.bfloat16 and got.shape == (T, F)
    torch.testing.assert_close(got.float().cpu(), want, atol=2e-2, rtol=2e-2)
    if F % 8 == 0:
        # a view one column into a wider buffer: rows keep their pitch, the base address loses its alignment
        wide = torch.zeros(T, 2 * F + 8, dtype=torch.bfloat16)
        wide[:, 1: 2 * F + 1] = gu
        got2 = Dn.gated_act(wide.cuda()[:, 1: 2 * F + 1], act, interleaved, limit)
        torch.testing.assert_close(got2.float().cpu(), want, atol=2e-2, rtol=2e-2)


def test_quick_gelu_epilogue_of_both_bf16_gemms():
    """x * sigmoid(1.702 x) as an epilogue code of the per-tile GEMM and of the persistent GEMM."""
    from antfly_b200.ops import dense
    from antfly_b200.ops import index_ops as IX

    M, N, K = 513, 1000, 768
    a = _rand(M, K, seed=3)
    w = _rand(N, K, scale=K ** -0.5, seed=4)
    b = _rand(N, seed=5)
    r = _rand(M, N, seed=6)
    ref = R.linear(a, w, b, "quick_gelu", r)
    y = dense.gemm_bf16(a, w, bias=b, act="quick_gelu", residual=r)
    torch.testing.assert_close(y.float(), ref, atol=4e-2, rtol=2e-2)
    yp = IX.gemm_persistent(a, w, bias=b, act="quick_gelu", residual=r)
    torch.testing.assert_close(yp.float(), ref, atol=4e-2, rtol=2e-2)
