"""GPU numerics: argmax, penalties, filtered sampling and speculative verify against the fp32 oracle."""
import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def test_argmax_matches_torch():
    from antfly_b200.ops import sampling as S

    g = torch.Generator(device="cuda").manual_seed(0)
    for dt in (torch.float32, torch.bfloat16):
        x = torch.randn(64, 128256, generator=g, device="cuda").to(dt)
        idx, val = S.argmax(x, want_val=True)
        assert torch.equal(idx.long(), x.float().argmax(-1))
        torch.testing.assert_close(val, x.float().max(-1).values)
    x = torch.zeros(3, 1000, device="cuda")
    x[1, 7] = x[1, 9] = 2.0
    assert S.argmax(x).tolist() == [0, 7, 0]
    assert S.argmax(x, vocab_offset=100).tolist() == [100, 107, 100]


def test_penalties_and_counts():
    from antfly_b200.ops import sampling as S

    B, V = 4, 5000
    logits = torch.randn(B, V, device="cuda")
    counts = torch.zeros(B, V, dtype=torch.int16, device="cuda")
    toks = torch.tensor([1, 1, 1, 7, 4999, 3], dtype=torch.int32, device="cuda")
    rows = torch.tensor([0, 0, 0, 1, 2, 3], dtype=torch.int32, device="cuda")
    S.count_tokens(counts, toks, rows)
    assert counts[0, 1] == 3 and counts[1, 7] == 1 and counts[2, 4999] == 1 and counts.sum() == 6
    rep = torch.tensor([1.3, 1.0, 2.0, 1.1], device="cuda")
    fr = torch.tensor([0.5, 0.0, 0.1, 0.0], device="cuda")
    pr = torch.tensor([0.2, 0.3, 0.0, 0.0], device="cuda")
    out = S.penalties(logits, counts, rep, fr, pr)
    ref = S.penalties(logits.cpu(), counts.cpu(), rep.cpu(), fr.cpu(), pr.cpu())
    torch.testing.assert_close(out.cpu(), ref)


@pytest.mark.parametrize("top_k,top_p,min_p", [(0, 1.0, 0.0), (50, 1.0, 0.0), (0, 0.9, 0.0), (0, 1.0, 0.05),
                                                (40, 0.8, 0.02)])
def test_sampler_support_and_distribution(top_k, top_p, min_p):
    from antfly_b200.ops import sampling as S

    V, n = 2000, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    base = torch.randn(V, generator=g, device="cuda") * 2.0
    logits = base[None].repeat(n, 1).contiguous()
    temp = torch.full((n,), 0.8, device="cuda")
    tk = torch.full((n,), top_k, dtype=torch.int32, device="cuda")
    tp = torch.full((n,), top_p, device="cuda")
    mp = torch.full((n,), min_p, device="cuda")
    u = torch.rand(n, generator=g, device="cuda")
    out, prob = S.sample(logits, temp, tk, tp, mp, u, want_prob=True)
    p = R.filtered_probs(base, 0.8, top_k, top_p, min_p)
    support = p > 0
    assert bool(support[out.long()].all()), "sampled a token outside the filtered support"
    torch.testing.assert_close(prob, p[out.long()], atol=1e-4, rtol=1e-3)
    emp = torch.bincount(out.long(), minlength=V).float() / n
    assert float((emp - p).abs().sum()) < 0.25  # total-variation style bound at n = 4096
    # the same uniform draws give the same tokens as inverse-CDF sampling on the oracle distribution
    cum = p.cumsum(-1)
    exp_idx = torch.searchsorted(cum, u * cum[-1], right=True).clamp_max(V - 1)
    assert float((exp_idx == out.long()).float().mean()) > 0.98


def test_sampler_greedy_rows_and_spec_verify():
    from antfly_b200.ops import sampling as S

    logits = torch.randn(5, 3000, device="cuda")
    temp = torch.tensor([0.0, 1.0, 0.0, 0.7, 0.0], device="cuda")
    z = torch.zeros(5, device="cuda")
    out = S.sample(logits, temp, z.int(), z + 1.0, z, torch.rand(5, device="cuda"))
    am = logits.argmax(-1)
    for b in (0, 2, 4):
        assert int(out[b]) == int(am[b])
    draft = torch.tensor([[1, 2, 3, 4], [1, 2, 9, 4], [7, 2, 3, 4], [1, 2, 3, 4]], dtype=torch.int32, device="cuda")
    target = torch.tensor([[1, 2, 3, 4, 5], [1, 2, 3, 4, 5], [1, 2, 3, 4, 5], [1, 2, 3, 8, 5]], dtype=torch.int32,
                          device="cuda")
    n, nxt = S.spec_verify(draft, target)
    assert n.tolist() == [4, 2, 0, 3] and nxt.tolist() == [5, 3, 1, 8]
