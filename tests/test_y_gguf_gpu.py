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
