"""Rotary frequency tables for llama3 / yarn / longrope scaling against transformers' own initialisers."""
import pytest
import torch
from transformers import LlamaConfig as HFLlamaConfig
from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

from antfly_b200.models.rope_scaling import rope_frequencies


def _hf(kind, rope, max_pos=8192, theta=500000.0, head_dim=64, seq_len=None):
    cfg = HFLlamaConfig(hidden_size=head_dim * 4, num_attention_heads=4, max_position_embeddings=max_pos,
                        rope_parameters=dict(rope, rope_type=kind, rope_theta=theta))
    inv, att = ROPE_INIT_FUNCTIONS[kind](cfg, "cpu", seq_len=seq_len)
    return inv.double(), float(att)


def test_llama3_table_matches_transformers():
    rope = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
    want, att = _hf("llama3", rope, max_pos=131072)
    got, a = rope_frequencies(dict(rope, rope_type="llama3"), 500000.0, 64, 131072)
    assert a == att == 1.0
    torch.testing.assert_close(torch.tensor(got, dtype=torch.float64), want, rtol=1e-5, atol=0)
    # the three bands are all present: untouched, blended, divided by the factor
    base = torch.tensor([500000.0 ** (-2 * j / 64) for j in range(32)], dtype=torch.float64)
    ratio = torch.tensor(got, dtype=torch.float64) / base
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8) < 1e-12 and bool(((ratio > 0.13) & (ratio < 0.99)).any())


@pytest.mark.parametrize("extra", [{}, {"beta_fast": 16.0, "beta_slow": 2.0}, {"mscale": 1.0, "mscale_all_dim": 0.707},
                                   {"attention_factor": 1.3}, {"truncate": False}])
def test_yarn_table_and_attention_factor_match_transformers(extra):
    rope = dict({"factor": 4.0, "original_max_position_embeddings": 4096}, **extra)
    want, att = _hf("yarn", rope, max_pos=16384, theta=10000.0, head_dim=128)
    got, a = rope_frequencies(dict(rope, rope_type="yarn"), 10000.0, 128, 16384)
    torch.testing.assert_close(torch.tensor(got, dtype=torch.float64), want, rtol=1e-5, atol=0)
    assert abs(a - att) < 1e-6


def test_longrope_short_and_long_factor_sets():
    g = torch.Generator().manual_seed(0)
    short = (1.0 + torch.rand(48, generator=g)).tolist()
    long_ = (2.0 + 6 * torch.rand(48, generator=g)).tolist()
    rope = {"short_factor": short, "long_factor": long_, "original_max_position_embeddings": 4096, "factor": 32.0}
    want_s, att = _hf("longrope", rope, max_pos=131072, theta=10000.0, head_dim=96, seq_len=100)
    want_l, _ = _hf("longrope", rope, max_pos=131072, theta=10000.0, head_dim=96, seq_len=5000)
    got_s, a = rope_frequencies(dict(rope, rope_type="longrope"), 10000.0, 96, 131072)
    got_l, _ = rope_frequencies(dict(rope, rope_type="longrope"), 10000.0, 96, 131072, serve_context=8192)
    torch.testing.assert_close(torch.tensor(got_s, dtype=torch.float64), want_s, rtol=1e-5, atol=0)
    torch.testing.assert_close(torch.tensor(got_l, dtype=torch.float64), want_l, rtol=1e-5, atol=0)
    assert abs(a - att) < 1e-6 and a > 1.0
    with pytest.raises(ValueError):
        rope_frequencies({"rope_type": "longrope", "short_factor": [1.0], "long_factor": [1.0],
                          "original_max_position_embeddings": 4096}, 10000.0, 96, 131072)


def test_plain_and_linear_schemes_keep_the_scalar_path():
    assert rope_frequencies(None, 10000.0, 64) == (None, 1.0)
    assert rope_frequencies({"rope_type": "default", "rope_theta": 1e4}, 10000.0, 64) == (None, 1.0)
    assert rope_frequencies({"rope_type": "linear", "factor": 2.0}, 10000.0, 64) == (None, 1.0)
