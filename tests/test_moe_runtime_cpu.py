"""MoE runtime: route batching, co-activation prediction, residency eviction order, and a MoE model running with its
experts offloaded to host memory giving the same logits as the fully resident model."""
import torch

from antfly_b200.runtime.moe import CoactivationPredictor, ExpertResidency, HostExpertStore, route_batches


def test_route_batches_groups_tokens_by_expert():
    topi = torch.tensor([[2, 0], [2, 3], [0, 2], [3, 1]])
    topw = torch.tensor([[.6, .4], [.7, .3], [.9, .1], [.5, .5]])
    b = route_batches(topi, topw, 5)
    assert b.active == [0, 1, 2, 3] and b.offsets == [0, 2, 3, 6, 8]
    got = {e: (rows.tolist(), [round(x, 2) for x in w.tolist()]) for e, rows, w in b}
    assert got == {0: ([0, 2], [.4, .9]), 1: ([3], [.5]), 2: ([0, 1, 2], [.6, .7, .1]), 3: ([1, 3], [.3, .5])}
    # scatter-add of per-expert results reproduces the dense mixture
    T, H, E = 4, 8, 5
    x = torch.randn(T, H)
    We = torch.randn(E, H, H)
    dense = sum(topw[:, j, None] * torch.einsum("th,thk->tk", x, We[topi[:, j]]) for j in range(2))
    out = torch.zeros(T, H)
    for e, rows, w in b:
        out.index_add_(0, rows, (x[rows] @ We[e]) * w[:, None])
    torch.testing.assert_close(out, dense)


def test_predictor_uses_coactivation_then_activity():
    p = CoactivationPredictor()
    p.note(0, 4, [1, 2])
    p.note(0, 4, [1, 2])
    assert p.predict(0, [1], 2) == ([2], [4])          # expert 2: co-active twice + active twice; 0 and 3 score 0
    p.note(0, 4, [0, 3])
    pred, scores = p.predict(0, [1], 3)
    assert pred == [2, 0, 3] and scores == [4, 1, 1]   # ties go to the lower index
    assert p.predict(1, [1], 2) == ([], []) and p.predict(0, [], 2) == ([], [])


def test_residency_evicts_cold_then_old_and_protects_the_current_step():
    loads = []
    r = ExpertResidency(lambda l, e: loads.append((l, e)) or f"w{l}.{e}", max_resident_per_layer=2)
    assert r.ensure(0, [0, 1]) == {0: "w0.0", 1: "w0.1"}
    r.ensure(0, [0])                                   # expert 0 is hotter than 1
    r.ensure(0, [2])                                   # over capacity: 1 (one touch, older) goes, not 0, not 2
    assert sorted(e for (_l, e) in r.resident) == [0, 2]
    r.ensure(0, [1, 2])                                # 1 comes back (a miss); 0 has 2 touches, 2 has 2, 1 has 2
    assert r.stats["misses"] == 4 and r.stats["hits"] == 2 and r.resident_count(0) == 2
    assert (0, 1) in r.resident and (0, 2) in r.resident            # the step's own experts are never evicted
    # a step needing more experts than the capacity keeps them all for that step
    r.ensure(1, [0, 1, 2])
    assert r.resident_count(1) == 3
    # prefetch fills up to the capacity without touching protected experts, and a later use counts as a hit
    r2 = ExpertResidency(lambda l, e: (l, e), max_resident_per_layer=3)
    r2.ensure(0, [0, 1])
    assert r2.prefetch(0, [2, 3], protect=[0, 1]) == 1 and r2.resident_count(0) == 3
    r2.ensure(0, [2])
    assert r2.stats["prefetch_hits"] == 1 and r2.stats["misses"] == 2


def test_moe_model_with_offloaded_experts_matches_resident_model():
    import pytest

    transformers = pytest.importorskip("transformers")
    from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch

    torch.manual_seed(0)
    hf_cfg = transformers.MixtralConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                        num_local_experts=6, num_experts_per_tok=2)
    hf = transformers.MixtralForCausalLM(hf_cfg)
    cfg = LlamaConfig.from_hf(hf_cfg.to_dict())
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}

    def run(model, steps=6):
        S, page, nblk = 20, 16, 3
        ids = torch.randint(0, 320, (S + steps,), generator=torch.Generator().manual_seed(1))
        kc = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        table = torch.arange(nblk, dtype=torch.int32)[None]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32)
        pos = torch.arange(S, dtype=torch.int32)
        outs = [model.forward(StepBatch(ids[:S].int(), pos, pos.clone(), i32([0]), i32([S]), i32([S]), table,
                                        pos.clone(), S, 1), kc, vc).float()]
        for t in range(S, S + steps):
            outs.append(model.forward(StepBatch(ids[t:t + 1].int(), i32([t]), i32([t]), i32([0]), i32([1]),
                                                i32([t + 1]), table, i32([0]), 1, 1), kc, vc).float())
        return torch.cat(outs)

    want = run(LlamaModel.from_state_dict(cfg, sd, device="cpu"))
    off = LlamaModel.from_state_dict(cfg, sd, device="cpu")
    rt = off.offload_experts(max_resident_per_layer=3, max_predicted=1)
    assert not any(".e0." in k for k in off.w) and rt.store.bytes() > 0
    got = run(off)
    torch.testing.assert_close(got, want, atol=0, rtol=0)      # same kernels, same weights: bitwise equal
    st = rt.residency.stats
    assert st["misses"] > 0 and st["evictions"] > 0 and st["hits"] > 0
    assert all(rt.residency.resident_count(l) <= 3 for l in range(cfg.num_hidden_layers))
    # third tier: the experts live in a file, a bounded host cache sits between it and the device
    import tempfile, os

    with tempfile.TemporaryDirectory() as d:
        disk = LlamaModel.from_state_dict(cfg, sd, device="cpu")
        one = sum(v.nbytes() for k, v in disk.w.items() if k.startswith("l0.e0."))
        rd = disk.offload_experts(max_resident_per_layer=2, max_predicted=1, spill_path=os.path.join(d, "experts.st"),
                                  host_budget_bytes=3 * one)
        assert os.path.getsize(os.path.join(d, "experts.st")) > cfg.num_hidden_layers * cfg.num_experts * one * 0.9
        torch.testing.assert_close(run(disk), want, atol=0, rtol=0)
        ts = rd.store.store.stats
        assert ts["disk_reads"] > 0 and ts["evictions"] > 0 and rd.store.bytes() <= 3 * one
