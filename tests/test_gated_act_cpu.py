"""Gated MLP activation: the fp32 formula in both layouts, the clamp, and the dtype contract of the op on CPU."""
import torch

from antfly_b200.ops import dense as Dn
from antfly_b200.ops import reference as R


def test_layouts_agree_and_match_the_plain_formula():
    g = torch.Generator().manual_seed(0)
    gate, up = torch.randn(6, 40, generator=g) * 3, torch.randn(6, 40, generator=g) * 3
    halves = torch.cat([gate, up], 1)
    inter = torch.stack([gate, up], -1).reshape(6, 80)
    for act, fn in (("silu", torch.nn.functional.silu), ("gelu", torch.nn.functional.gelu),
                    ("gelu_tanh", lambda x: torch.nn.functional.gelu(x, approximate="tanh")),
                    ("relu2", lambda x: torch.relu(x) ** 2), ("quick_gelu", lambda x: x * torch.sigmoid(1.702 * x))):
        want = fn(gate) * up
        torch.testing.assert_close(R.gated_act(halves, act), want)
        torch.testing.assert_close(R.gated_act(inter, act, interleaved=True), want)
    lim = 1.5
    want = torch.nn.functional.silu(gate.clamp(max=lim)) * up.clamp(-lim, lim)
    torch.testing.assert_close(R.gated_act(halves, "silu", limit=lim), want)


def test_op_keeps_the_input_dtype_on_cpu_and_fills_out():
    x = torch.randn(4, 32)
    y = Dn.gated_act(x, "gelu")
    assert y.dtype == torch.float32 and y.shape == (4, 16)
    xb = x.to(torch.bfloat16)
    out = torch.empty(4, 16, dtype=torch.bfloat16)
    assert Dn.gated_act(xb, "silu", out=out) is out
    torch.testing.assert_close(out.float(), R.gated_act(xb, "silu"), atol=2e-2, rtol=2e-2)
    assert set(Dn.GATE_ACT.values()) == {1, 2, 3, 4, 5, 6}
