"""GPU expansion of GGUF block formats against the C++ block decoders, and the linear layer built on it."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("type_id,bv,bb", [(2, 32, 18), (8, 32, 34), (12, 256, 144), (13, 256, 176), (14, 256, 210),
                                           (39, 32, 17)])
def test_device_dequant_matches_host(type_id, bv, bb):
    from antfly_b200.ops import gguf_ops as G

    rng = np.random.default_rng(type_id)
    rows, cols = 96, 1024
    blocks = rows * cols // bv
    raw = rng.integers(0, 256, size=(blocks, bb), dtype=np.uint8)
    half_at = {2: [0], 8: [0], 12: [0, 2], 13: [0, 2], 14: [208], 39: []}[type_id]
    for off in half_at:
        raw[:, off:off + 2] = rng.uniform(-1.0, 1.0, size=blocks).astype(np.float16).view(np.uint8).reshape(blocks, 2)
    if type_id == 39:
        raw[:, 0] = rng.integers(118, 132, size=blocks)
    t = torch.from_numpy(raw.reshape(-1))
    want = G.dequantize(t, type_id, (rows, cols), torch.float32)
    got32 = G.dequantize(t.cuda(), type_id, (rows, cols), torch.float32)
    torch.testing.assert_close(got32.cpu(), want, atol=0, rtol=0)
    got16 = G.dequantize(t.cuda(), type_id, (rows, cols), torch.bfloat16)
    torch.testing.assert_close(got16.float().cpu(), want.to(torch.bfloat16).float(), atol=0, rtol=0)
    x = (torch.randn(40, cols, device="cuda") * 0.1).to(torch.bfloat16)
    y = G.linear_gguf(x, t.cuda(), type_id, rows, cols)
    ref = x.float() @ want.to(torch.bfloat16).float().cuda().T
    torch.testing.assert_close(y.float(), ref, atol=5e-2 * float(ref.abs().max()), rtol=2e-2)


@pytest.mark.parametrize("type_id,bv", [(2, 32), (8, 32), (12, 256), (13, 256), (14, 256), (39, 32)])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_fused_matvec_matches_fp32_reference(type_id, bv, M):
    """afb_gguf_mul_mv: quantised bytes expanded in registers, against fp32 matmul over the host-decoded weight;
    ragged N, K across several 1024-value chunks, bias + activation epilogue."""
    from antfly_b200 import _native as N_
    from antfly_b200.ops import gguf_ops as G

    rng = np.random.default_rng(type_id * 10 + M)
    rows, cols = 203, 2304
    bb = {2: 18, 8: 34, 12: 144, 13: 176, 14: 210, 39: 17}[type_id]
    blocks = rows * cols // bv
    raw = rng.integers(0, 256, size=(blocks, bb), dtype=np.uint8)
    for off in {2: [0], 8: [0], 12: [0, 2], 13: [0, 2], 14: [208], 39: []}[type_id]:
        raw[:, off:off + 2] = rng.uniform(-1.0, 1.0, size=blocks).astype(np.float16).view(np.uint8).reshape(blocks, 2)
    if type_id == 39:
        raw[:, 0] = rng.integers(118, 132, size=blocks)
    t = torch.from_numpy(raw.reshape(-1))
    w = G.dequantize(t, type_id, (rows, cols), torch.float32)
    x = (torch.randn(M, cols) * 0.1).to(torch.bfloat16)
    bias = torch.randn(rows).to(torch.bfloat16)
    got = G.linear_gguf(x.cuda(), t.cuda(), type_id, rows, cols, bias=bias.cuda(), act="silu")
    assert N_.status() == 0 and got.shape == (M, rows)
    ref = torch.nn.functional.silu(x.float() @ w.T + bias.float())
    torch.testing.assert_close(got.float().cpu(), ref, atol=2e-2 * float(ref.abs().max()) + 1e-2, rtol=2e-2)


def test_large_batches_expand_in_l2_sized_slabs(monkeypatch):
    from antfly_b200.ops import gguf_ops as G

    rng = np.random.default_rng(0)
    rows, cols = 1024, 512
    raw = rng.integers(0, 256, size=(rows * cols // 32, 34), dtype=np.uint8)
    raw[:, 0:2] = rng.uniform(-1, 1, size=raw.shape[0]).astype(np.float16).view(np.uint8).reshape(-1, 2)
    t = torch.from_numpy(raw.reshape(-1))
    w = G.dequantize(t, 8, (rows, cols), torch.float32)
    x = (torch.randn(64, cols) * 0.1).to(torch.bfloat16)
    whole = G.linear_gguf(x.cuda(), t.cuda(), 8, rows, cols)
    monkeypatch.setattr(G, "EXPAND_SLAB_BYTES", 256 * cols * 2)           # four slabs of 256 rows
    slabs = G.linear_gguf(x.cuda(), t.cuda(), 8, rows, cols)
    assert torch.equal(whole, slabs)
    ref = x.float() @ w.to(torch.bfloat16).float().T
    torch.testing.assert_close(slabs.float().cpu(), ref, atol=5e-2 * float(ref.abs().max()), rtol=2e-2)
