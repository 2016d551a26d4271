"""Attention with sink logits and soft-capped scores: the oracle against plain loops, and a Llama-family checkpoint
that carries ``self_attn.sinks`` through the paged engine path."""
import math

import pytest
import torch

from antfly_b200.ops import reference as R


def _loops(q, kc, vc, bt, q_starts, q_lens, kv_lens, scale, window, sinks, softcap):
    T, Hq, D = q.shape
    page, Hkv = kc.shape[1], kc.shape[2]
    out = torch.zeros(T, Hq, D)
    for b in range(bt.shape[0]):
        for i in range(int(q_lens[b])):
            tok = int(q_starts[b]) + i
            qpos = int(kv_lens[b]) - int(q_lens[b]) + i
            lo = max(0, qpos + 1 - window) if window > 0 else 0
            for h in range(Hq):
                hk = h // (Hq // Hkv)
                logits, vals = [], []
                for key in range(lo, qpos + 1):
                    blk = int(bt[b, key // page])
                    s = float(q[tok, h].float() @ kc[blk, key % page, hk].float()) * scale
                    if softcap > 0:
                        s = softcap * math.tanh(s / softcap)
                    logits.append(s)
                    vals.append(vc[blk, key % page, hk].float())
                m = max(logits + ([float(sinks[h])] if sinks is not None else []))
                e = [math.exp(s - m) for s in logits]
                den = sum(e) + (math.exp(float(sinks[h]) - m) if sinks is not None else 0.0)
                out[tok, h] = sum(w * v for w, v in zip(e, vals)) / den
    return out


@pytest.mark.parametrize("sinks,softcap,window", [(True, 0.0, 0), (False, 2.5, 0), (True, 3.0, 5)])
def test_reference_matches_plain_loops(sinks, softcap, window):
    g = torch.Generator().manual_seed(0)
    Hq, Hkv, D, page, nblk = 4, 2, 8, 4, 12
    kc, vc = torch.randn(nblk, page, Hkv, D, generator=g), torch.randn(nblk, page, Hkv, D, generator=g)
    bt = torch.tensor([[3, 7, 1, 0], [5, 2, 9, 11]], dtype=torch.int32)
    q_lens, kv_lens = torch.tensor([3, 1]), torch.tensor([11, 14])
    q_starts = torch.tensor([0, 3])
    q = torch.randn(4, Hq, D, generator=g)
    sk = torch.randn(Hq, generator=g) if sinks else None
    got = R.paged_attention(q, kc, vc, bt, q_starts, q_lens, kv_lens, 0.4, window, sinks=sk, softcap=softcap)
    want = _loops(q, kc, vc, bt, q_starts, q_lens, kv_lens, 0.4, window, sk, softcap)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    if sinks:     # the sink only takes probability mass away: rows shrink towards zero, never change direction
        plain = R.paged_attention(q, kc, vc, bt, q_starts, q_lens, kv_lens, 0.4, window, softcap=softcap)
        ratio = (got * plain).sum(-1) / (plain * plain).sum(-1)
        assert bool(((ratio > 0) & (ratio < 1)).all())
        torch.testing.assert_close(got / ratio[..., None], plain, atol=1e-4, rtol=1e-4)


def test_checkpoint_with_sinks_runs_through_the_paged_path():
    transformers = pytest.importorskip("transformers")
    from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch

    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                      tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval().float()
    base = {k: v.detach().clone() for k, v in hf.state_dict().items()}

    def run(sd, chunks):
        cfg = LlamaConfig.from_hf(hf_cfg.to_dict())
        model = LlamaModel.from_state_dict(cfg, sd, device="cpu")
        page, nblk = 16, 2
        kc = torch.zeros((2, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        table = torch.arange(nblk, dtype=torch.int32)[None]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32)
        ids = torch.arange(5, 25, dtype=torch.int32)
        outs, at = [], 0
        for n in chunks:
            pos = torch.arange(at, at + n, dtype=torch.int32)
            b = StepBatch(ids[at:at + n], pos, pos.clone(), i32([0]), i32([n]), i32([at + n]), table,
                          torch.arange(n, dtype=torch.int32), n, 1)
            outs.append(model.forward(b, kc, vc).float())
            at += n
        return cfg, torch.cat(outs)

    cfg0, plain = run(base, [20])
    assert not cfg0.attn_sinks
    far = dict(base, **{f"model.layers.{l}.self_attn.sinks": torch.full((4,), -40.0) for l in range(2)})
    cfg1, same = run(far, [20])
    assert cfg1.attn_sinks
    torch.testing.assert_close(same, plain, atol=2e-2, rtol=2e-2)       # a sink at -40 takes no mass
    near = dict(base, **{f"model.layers.{l}.self_attn.sinks": torch.tensor([0.5, -0.3, 1.0, 0.0]) for l in range(2)})
    _, whole = run(near, [20])
    assert float((whole - plain).abs().max()) > 0.05                     # a live sink changes the logits
    _, stepped = run(near, [7, 1, 1, 6, 5])
    torch.testing.assert_close(stepped, whole, atol=3e-2, rtol=3e-2)    # prefill chunks and decode steps agree
