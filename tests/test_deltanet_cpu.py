"""Gated delta-rule layer against the Hugging Face Qwen3.5 module, and prefill / decode equivalence of its state."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models.deltanet import DeltaNetConfig, GatedDeltaNetLayer, gated_delta_rule


def _hf():
    from transformers.models.qwen3_5 import modeling_qwen3_5 as M

    torch.manual_seed(0)
    cfg = transformers.Qwen3_5TextConfig(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                                         num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                         linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                                         linear_value_head_dim=8, linear_conv_kernel_dim=4)
    layer = M.Qwen3_5GatedDeltaNet(cfg, layer_idx=0).eval().float()
    with torch.no_grad():
        layer.norm.weight.uniform_(0.5, 1.5)
        layer.dt_bias.uniform_(-1, 1)
    return M, cfg, layer


def test_layer_matches_transformers_and_state_carries_over():
    M, hf_cfg, hf = _hf()
    cfg = DeltaNetConfig.from_hf(hf_cfg.to_dict())
    assert cfg.linear_num_value_heads == 4 and cfg.linear_key_head_dim == 16
    mine = GatedDeltaNetLayer.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    x = torch.randn(37, 64, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(x[None])[0]
    got, state = mine.forward(x)
    assert float(torch.nn.functional.cosine_similarity(got.float().flatten(), want.flatten(), dim=0)) > 0.999
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=5e-2)
    # prefill 30 tokens, then 7 single-token steps: same outputs, same final state
    a, st = mine.forward(x[:30])
    outs = [a]
    for t in range(30, 37):
        y, st = mine.forward(x[t:t + 1], st)
        outs.append(y)
    torch.testing.assert_close(torch.cat(outs).float(), got.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(st[1], state[1], atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(st[0], state[0], atol=1e-2, rtol=1e-2)


def test_recurrence_matches_the_library_restatement():
    M, _, _ = _hf()
    g0 = torch.Generator().manual_seed(2)
    T, H, Dk, Dv = 11, 3, 8, 5
    q, k = torch.randn(T, H, Dk, generator=g0), torch.randn(T, H, Dk, generator=g0)
    v = torch.randn(T, H, Dv, generator=g0)
    g = -torch.rand(T, H, generator=g0)
    beta = torch.rand(T, H, generator=g0)
    s0 = torch.randn(H, Dk, Dv, generator=g0)
    want, ws = M.torch_recurrent_gated_delta_rule(q[None], k[None], v[None], g[None], beta[None], s0[None], True,
                                                  use_qk_l2norm_in_kernel=True)
    got, gs = gated_delta_rule(q, k, v, g, beta, s0)
    torch.testing.assert_close(got, want[0], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(gs, ws[0], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("T,chunk", [(64, 64), (150, 64), (37, 16), (5, 8), (1, 4)])
def test_chunked_delta_rule_equals_the_recurrence(T, chunk):
    from antfly_b200.models.deltanet import gated_delta_rule, gated_delta_rule_chunked

    g_ = torch.Generator().manual_seed(T)
    H, Dk, Dv = 3, 16, 24
    q, k = torch.randn(T, H, Dk, generator=g_), torch.randn(T, H, Dk, generator=g_)
    v = torch.randn(T, H, Dv, generator=g_)
    g = -torch.rand(T, H, generator=g_) * 1.5                       # log decays, some strong
    beta = torch.rand(T, H, generator=g_)
    s0 = torch.randn(H, Dk, Dv, generator=g_) * 0.5
    for state in (None, s0):
        want_o, want_s = gated_delta_rule(q, k, v, g, beta, state)
        got_o, got_s = gated_delta_rule_chunked(q, k, v, g, beta, state, chunk=chunk)
        torch.testing.assert_close(got_o, want_o, atol=2e-4, rtol=2e-4)
        torch.testing.assert_close(got_s, want_s, atol=2e-4, rtol=2e-4)
    # a long prompt in one chunked call, then recurrent decode steps, equals the recurrence throughout
    o1, s1 = gated_delta_rule_chunked(q, k, v, g, beta, None, chunk=chunk)
    o2, s2 = gated_delta_rule(q[-1:], k[-1:], v[-1:], g[-1:], beta[-1:], gated_delta_rule(q[:-1], k[:-1], v[:-1], g[:-1],
                                                                                       beta[:-1])[1]) if T > 1 else (o1, s1)
    torch.testing.assert_close(o1[-1:], o2, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(s1, s2, atol=2e-4, rtol=2e-4)
