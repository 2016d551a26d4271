"""Placement planner, run budget and the tiered weight store (CPU: the backend tier collapses onto the host)."""
import pytest
import torch

from antfly_b200.runtime import tiering as T


def test_weight_classes_and_placement():
    # the reference's own expectations (zig/pkg/inference/src/runtime/tier/planner.zig tests)
    assert T.classify_weight("model.layers.0.block_sparse_moe.experts.1.w1.weight") is T.WeightClass.EXPERT
    assert T.classify_weight("model.layers.0.block_sparse_moe.gate.weight") is T.WeightClass.ROUTER
    assert T.classify_weight("model.layers.0.self_attn.q_proj.weight") is T.WeightClass.ATTENTION
    assert T.classify_weight("model.embed_tokens.weight") is T.WeightClass.EMBEDDING
    assert T.classify_weight("model.layers.3.input_layernorm.weight") is T.WeightClass.NORM
    assert T.classify_weight("lm_head.weight") is T.WeightClass.OUTPUT
    e = "model.layers.0.block_sparse_moe.experts.1.w1.weight"
    g, c = T.plan_placement(e, gpu=True), T.plan_placement(e, gpu=False)
    assert (g.preferred, g.spill) == (T.Tier.BACKEND, T.Tier.HOST) and (c.preferred, c.spill) == (T.Tier.HOST, T.Tier.DISK)
    mb = 1 << 20
    p = T.plan_placement("lm_head.weight", True, 128 * mb, 256 * mb, 256 * mb)
    assert p.preferred is T.Tier.DISK and p.spill is T.Tier.DISK
    p = T.plan_placement(e, True, 128 * mb, 0, 256 * mb)
    assert (p.preferred, p.spill) == (T.Tier.HOST, T.Tier.DISK)
    assert T.plan_placement("model.layers.0.self_attn.q_proj.weight", True, 128 * mb, 256 * mb, 256 * mb).preferred \
        is T.Tier.BACKEND


def test_run_budget_limits_and_denial_line():
    b = T.RunBudget(T.Limits(host=100, backend=80, combined=150, kv=60, scratch=30))
    r1 = b.reserve("weight", T.Tier.HOST, 50)
    with pytest.raises(T.MemoryBudgetExceeded) as ei:
        b.reserve("weight", T.Tier.HOST, 70)
    assert "limit=host_total reservation=weight/host current=50 request=70 next=120 limit=100" in str(ei.value)
    assert "totals(host=50 backend=0 kv=0 scratch=0)" in b.denial_line() and b.denials == 1
    b.reserve("kv", T.Tier.BACKEND, 60)
    with pytest.raises(T.MemoryBudgetExceeded) as ei:
        b.reserve("kv", T.Tier.HOST, 1)
    assert "limit=kv_total" in str(ei.value)
    with pytest.raises(T.MemoryBudgetExceeded) as ei:
        b.reserve("weight", T.Tier.BACKEND, 30)
    assert "limit=backend_total" in str(ei.value)
    b.reserve("scratch", T.Tier.BACKEND, 20)
    with pytest.raises(T.MemoryBudgetExceeded) as ei:
        b.reserve("weight", T.Tier.HOST, 30)            # host 80 <= 100, but host + backend = 160 > 150
    assert "limit=combined_total" in str(ei.value)
    with pytest.raises(T.MemoryBudgetExceeded) as ei:
        b.reserve("scratch", T.Tier.HOST, 11)
    assert "limit=scratch_total" in str(ei.value)
    assert b.reserve("weight", T.Tier.DISK, 10 ** 9).nbytes == 10 ** 9       # disk is not budgeted
    b.release(r1)
    assert b.host_total == 0 and b.backend_total == 80 and b.peak_host == 50 and b.denials == 5
    assert T.Limits.from_mb(kv_mb=2).kv == 2 << 20


def test_tiered_store_lru_eviction_prefetch_and_file_source(tmp_path):
    from antfly_b200.formats.safetensors_io import save_file

    tensors = {f"model.layers.0.block_sparse_moe.experts.{i}.w1.weight": torch.full((64,), float(i)) for i in range(5)}
    path = str(tmp_path / "w.safetensors")
    save_file(tensors, path)
    src = T.SafetensorsSource(path)
    names = sorted(src.names())
    assert src.nbytes(names[0]) == 256
    store = T.TieredStore(src, "cpu", T.RunBudget(T.Limits(host=600)), start_worker=False)   # room for two tensors
    a = store.get(names[0])
    assert torch.equal(a, tensors[names[0]]) and store.tier_of(names[0]) is T.Tier.HOST
    store.get(names[1])
    store.get(names[0])                                      # touch: names[1] is now the oldest
    store.get(names[2])
    assert store.tier_of(names[1]) is T.Tier.DISK and store.tier_of(names[0]) is T.Tier.HOST
    assert store.stats["evictions"] == 1 and store.stats["host_hits"] == 1 and store.stats["disk_reads"] == 3
    assert store.budget.host_total == 512
    # prefetch: repeated requests raise one entry's priority; the hotter tensor is promoted first
    assert store.prefetch(names[3]) == 1 and store.prefetch(names[4]) == 1 and store.prefetch(names[4]) == 2
    assert store.pending(names[4]) == 2
    assert store.drain(1) == 1 and store.tier_of(names[4]) is T.Tier.HOST and store.tier_of(names[3]) is T.Tier.DISK
    assert store.drain() == 1 and store.pending(names[3]) == 0 and store.stats["prefetch_done"] == 2
    # a tensor larger than the whole budget is served from disk without being cached
    big = T.TieredStore(T.DictSource({"lm_head.weight": torch.zeros(1000)}), "cpu", T.RunBudget(T.Limits(host=100)),
                        start_worker=False)
    assert big.get("lm_head.weight").numel() == 1000 and big.tier_of("lm_head.weight") is T.Tier.DISK
    store.drop(names[4])
    assert store.tier_of(names[4]) is T.Tier.DISK
    # with the worker thread
    bg = T.TieredStore(src, "cpu", T.RunBudget(T.Limits(host=2000)))
    for n in names:
        bg.prefetch(n)
    assert bg.wait_idle(5.0) and all(bg.tier_of(n) is T.Tier.HOST for n in names)
    bg.close()


def test_generate_cli_refuses_a_run_over_budget(capsys):
    from antfly_b200.cli import main

    base = ["generate", "--model", "random:tiny", "--device", "cpu", "--prompt", "hi", "--max-tokens", "2"]
    assert main(base + ["--host-budget-mb", "100000"]) == 0
    capsys.readouterr()
    assert main(base + ["--kv-budget-mb", "1"]) == 3
    err = capsys.readouterr().err
    assert "memory budget exceeded: limit=kv_total reservation=kv/host" in err and "totals(host=" in err
