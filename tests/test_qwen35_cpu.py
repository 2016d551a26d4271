"""Qwen3.5 hybrid decoder (delta-rule layers + gated attention layers) against transformers' Qwen3_5ForCausalLM."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf():
    torch.manual_seed(0)
    cfg = transformers.Qwen3_5TextConfig(
        vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
        linear_value_head_dim=16, linear_conv_kernel_dim=4, max_position_embeddings=256, tie_word_embeddings=False)
    m = transformers.Qwen3_5ForCausalLM(cfg).eval().float()
    with torch.no_grad():     # norms and gates away from their zero / one initial values
        for n, p in m.named_parameters():
            if "norm" in n or "A_log" in n or "dt_bias" in n:
                p.add_(torch.randn_like(p) * 0.1)
    return cfg, m


def test_hybrid_decoder_logits_and_cached_decoding_match_transformers():
    from antfly_b200.models.qwen35 import Qwen35Config, Qwen35Model

    hf_cfg, hf = _hf()
    cfg = Qwen35Config.from_hf(hf_cfg.to_dict())
    assert cfg.layer_types == ["linear_attention"] * 3 + ["full_attention"]
    model = Qwen35Model.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    ids = torch.randint(0, 160, (1, 23), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids).logits[0]
    got, st = model.forward(ids[0])
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-3)
    # the carried state (KV for the attention layer, conv tail + matrix state for the others) continues exactly
    more = torch.randint(0, 160, (1, 5), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want2 = hf(torch.cat([ids, more], 1)).logits[0, 23:]
    got2 = []
    for t in range(5):
        lg, st = model.forward(more[0, t:t + 1], st)
        got2.append(lg[0])
    torch.testing.assert_close(torch.stack(got2), want2, atol=3e-4, rtol=3e-3)
    assert st.length == 28


def test_greedy_generation_matches_transformers():
    from antfly_b200.models.qwen35 import Qwen35Config, Qwen35Model

    hf_cfg, hf = _hf()
    model = Qwen35Model.from_state_dict(Qwen35Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                        dtype=torch.float32)
    prompt = [5, 9, 33, 120, 7, 64, 2]
    seq = torch.tensor([prompt])
    want = []
    with torch.no_grad():
        for _ in range(8):
            nxt = int(hf(seq).logits[0, -1].argmax())
            want.append(nxt)
            seq = torch.cat([seq, torch.tensor([[nxt]])], 1)
    assert model.generate(prompt, 8) == want


def test_long_prompt_through_the_chunked_delta_rule_matches_transformers():
    """Prompts of 32 tokens and more take the chunked (matrix-product) form of the delta rule in the recurrent
    layers; a prompt split over two calls carries the state from the chunked form into the next call."""
    from antfly_b200.models import deltanet
    from antfly_b200.models.qwen35 import Qwen35Config, Qwen35Model

    hf_cfg, hf = _hf()
    model = Qwen35Model.from_state_dict(Qwen35Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                        dtype=torch.float32)
    ids = torch.randint(0, 160, (1, 150), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        want = hf(ids).logits[0]
    assert 150 >= deltanet.CHUNKED_FROM
    got, _ = model.forward(ids[0])
    torch.testing.assert_close(got, want, atol=5e-4, rtol=3e-3)
    a, st = model.forward(ids[0, :100])
    b, st = model.forward(ids[0, 100:], st)
    torch.testing.assert_close(torch.cat([a, b]), want, atol=5e-4, rtol=3e-3)
