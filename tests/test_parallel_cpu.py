"""Multi-rank host logic on CPU (gloo, world size 2): sharding rules, the baseline TP communicator, a
tensor-parallel decoder that reproduces the single-rank logits, rank-failure detection by timeout."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from antfly_b200.parallel import sharding


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _hf_llama_state(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    H, F, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    r = lambda n, k: (torch.randn(n, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    sd = {"model.embed_tokens.weight": (torch.randn(cfg.vocab_size, H, generator=g) * 0.02).to(torch.bfloat16),
          "model.norm.weight": torch.ones(H, dtype=torch.bfloat16), "lm_head.weight": r(cfg.vocab_size, H)}
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        sd[p + "input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        sd[p + "self_attn.q_proj.weight"] = r(cfg.num_attention_heads * D, H)
        sd[p + "self_attn.k_proj.weight"] = r(cfg.num_key_value_heads * D, H)
        sd[p + "self_attn.v_proj.weight"] = r(cfg.num_key_value_heads * D, H)
        sd[p + "self_attn.o_proj.weight"] = r(H, cfg.num_attention_heads * D)
        sd[p + "mlp.gate_proj.weight"] = r(F, H)
        sd[p + "mlp.up_proj.weight"] = r(F, H)
        sd[p + "mlp.down_proj.weight"] = r(H, F)
    return sd


def _forward_logits(model, cfg, device="cpu"):
    from antfly_b200.models.llama import StepBatch

    lens = [9, 4]
    T = sum(lens)
    ids = (torch.arange(T, dtype=torch.int32) * 7 + 3) % cfg.vocab_size
    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
    ql = torch.tensor(lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int()
    tables = torch.tensor([[0, 0], [1, 0]], dtype=torch.int32)
    slots = torch.tensor(list(range(9)) + list(range(16, 20)), dtype=torch.int32)
    b = StepBatch(ids, pos, slots, qs, ql, ql.clone(), tables, (qs + ql - 1).int(), max(lens), 1)
    kc = torch.zeros((cfg.num_hidden_layers, 2, 16, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
    return model.forward(b, kc, torch.zeros_like(kc)).float()


def _tp_cfg(world):
    from antfly_b200.models.llama import LlamaConfig

    if world <= 2:
        return LlamaConfig.tiny(num_hidden_layers=2)
    return LlamaConfig.tiny(num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=4, hidden_size=512,
                            intermediate_size=1024)


def _tp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.parallel.comm import DistributedConfig, TpComm, init_process_group

    cfg_d = init_process_group(backend="gloo", timeout_s=60)
    assert cfg_d.mode == "tensor_parallel" and cfg_d.world_size == world
    comm = TpComm(rank, world, torch.device("cpu"))
    t = torch.full((3,), float(rank + 1))
    comm.all_reduce(t)
    assert t.tolist() == [world * (world + 1) / 2.0] * 3
    # vocabulary-sharded arg-max merge: the last rank holds the winner of row 0, a tie in row 1 resolves to the
    # lower index
    idx = torch.tensor([5 + 100 * rank, 7 + 100 * rank], dtype=torch.int32)
    val = torch.tensor([1.0 + rank, 2.0])
    assert comm.argmax_merge(idx, val).tolist() == [5 + 100 * (world - 1), 7]
    cfg = _tp_cfg(world)
    sd = _hf_llama_state(cfg)
    model = LlamaModel.from_state_dict(cfg, sd, device="cpu", tp_rank=rank, tp_size=world, comm=comm)
    logits = _forward_logits(model, cfg)                    # [2, V / world]
    full = comm.all_gather(logits).permute(1, 0, 2).reshape(2, -1)
    tok = model.greedy_tokens(logits.to(torch.bfloat16))
    if rank == 0:
        q.put((full, tok))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_decoder_matches_single_rank(world):
    from antfly_b200.models.llama import LlamaConfig, LlamaModel

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    full, tok = q.get(timeout=240)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    cfg = _tp_cfg(world)
    single = LlamaModel.from_state_dict(cfg, _hf_llama_state(cfg), device="cpu")
    ref = _forward_logits(single, cfg)
    torch.testing.assert_close(full, ref, atol=6e-2, rtol=5e-2)
    assert tok.tolist() == ref.argmax(-1).tolist()


def test_sharding_rules():
    assert sharding.shard_dim("model.layers.0.self_attn.q_proj.weight") == 0
    assert sharding.shard_dim("model.layers.0.mlp.down_proj.weight") == 1
    assert sharding.shard_dim("encoder.layer.0.attention.output.dense.weight") == 1
    assert sharding.shard_dim("encoder.layer.0.intermediate.dense.bias") == 0
    assert sharding.shard_dim("model.norm.weight") == -1
    w = torch.arange(64 * 128).view(64, 128).float()
    assert torch.equal(torch.cat([sharding.shard_rows(w, r, 4) for r in range(4)], 0), w)
    assert torch.equal(torch.cat([sharding.shard_cols(w, r, 4) for r in range(4)], 1), w)
    with pytest.raises(AssertionError):
        sharding.shard_cols(w, 0, 8)  # 16 columns per rank is not a whole 32-element quantisation block


def _silent_peer_worker(rank, world, port, q):
    """Rank 1 never joins the collective; rank 0 must get an error after the short timeout, not hang."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from antfly_b200.parallel.comm import init_process_group
    from antfly_b200.parallel.health import HeartbeatMonitor

    init_process_group(backend="gloo", timeout_s=5)
    store = dist.distributed_c10d._get_default_store()
    mon = HeartbeatMonitor(store, rank, world, interval_s=0.2, dead_after_s=1.5)
    mon.beat()
    if rank == 1:
        # leaves between steps, with nothing in flight
        q.put(("left", rank))
        return
    import time

    time.sleep(2.5)
    mon.beat()
    dead = mon.dead_ranks()
    q.put(("dead", dead))


def test_rank_failure_is_detected_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_silent_peer_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert got["left"] == 1 and got["dead"] == [1]


def _pp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import datetime

    from antfly_b200.models.llama import LlamaConfig
    from antfly_b200.parallel.pipeline import build_stage
    from antfly_b200.parallel.strategy import plan_parallel
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    cfg = LlamaConfig.tiny(num_hidden_layers=5)
    plan = plan_parallel(cfg, world, "pipeline")
    model = build_stage(cfg, _hf_llama_state(cfg), plan, rank, device="cpu")
    assert model.n_layers == plan.ranks[rank].layers[1] - plan.ranks[rank].layers[0]
    assert not any(k.startswith(f"l{plan.ranks[(rank + 1) % world].layers[0]}.") for k in model.w)
    logits = _forward_logits_layers(model, cfg)
    # the same stages drive the serving engine in lockstep: every rank generates the same tokens
    eng = LLMEngine(model, num_blocks=16, page=16, max_batch=2, use_cuda_graph=False)
    out = eng.generate([[5, 6, 7, 8, 9], [11, 12]], SamplingParams(max_tokens=5, ignore_eos=True))
    q.put((rank, logits.numpy(), [o.token_ids for o in out], model.pp.sent_bytes, model.pp.received_bytes))
    dist.barrier()
    dist.destroy_process_group()


def _forward_logits_layers(model, cfg):
    from antfly_b200.models.llama import StepBatch

    lens = [9, 4]
    T = sum(lens)
    ids = (torch.arange(T, dtype=torch.int32) * 7 + 3) % cfg.vocab_size
    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
    ql = torch.tensor(lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int()
    tables = torch.tensor([[0, 0], [1, 0]], dtype=torch.int32)
    slots = torch.tensor(list(range(9)) + list(range(16, 20)), dtype=torch.int32)
    b = StepBatch(ids, pos, slots, qs, ql, ql.clone(), tables, (qs + ql - 1).int(), max(lens), 1)
    kc = torch.zeros((model.n_layers, 2, 16, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
    return model.forward(b, kc, torch.zeros_like(kc)).float()


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_parallel_stages_match_single_rank(world):
    """Layer ranges on separate ranks (each with only its layers' weights and KV cache), hidden states passed by
    point-to-point sends, logits shared with every stage; also through the serving engine."""
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=300) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    cfg = LlamaConfig.tiny(num_hidden_layers=5)
    single = LlamaModel.from_state_dict(cfg, _hf_llama_state(cfg), device="cpu")
    ref = _forward_logits_layers(single, cfg)
    eng = LLMEngine(single, num_blocks=16, page=16, max_batch=2, use_cuda_graph=False)
    want = [o.token_ids for o in eng.generate([[5, 6, 7, 8, 9], [11, 12]], SamplingParams(max_tokens=5,
                                                                                            ignore_eos=True))]
    for rank, logits, toks, sent, recv in got:
        torch.testing.assert_close(torch.from_numpy(logits), ref, atol=6e-2, rtol=5e-2)
        assert toks == want
        assert (sent > 0) == (rank < world - 1) and (recv > 0) == (rank > 0)


def _moe_state():
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    hf_cfg = transformers.MixtralConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                        num_local_experts=6, num_experts_per_tok=2)
    hf = transformers.MixtralForCausalLM(hf_cfg)
    return hf_cfg.to_dict(), {k: v.detach().clone() for k, v in hf.state_dict().items()}


def _ep_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime

    from antfly_b200.models.llama import LlamaConfig, LlamaModel

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    cfg_d, sd = _moe_state()
    cfg = LlamaConfig.from_hf(cfg_d)
    model = LlamaModel.from_state_dict(cfg, sd, device="cpu", experts=(rank, world))
    model.set_expert_parallel(rank, world)
    held = sorted({int(k.split(".e")[1].split(".")[0]) for k in model.w if ".e" in k and k.endswith(".gu")})
    assert held == [e for e in range(6) if e % world == rank]
    if rank == 1:
        model.offload_experts(max_resident_per_layer=1)          # expert parallelism composes with host offload
    logits = _forward_logits(model, cfg)
    q.put((rank, logits.numpy()))          # by value: the worker may exit before the parent reads
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_moe_matches_single_rank(world):
    from antfly_b200.models.llama import LlamaConfig, LlamaModel

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    cfg_d, sd = _moe_state()
    cfg = LlamaConfig.from_hf(cfg_d)
    ref = _forward_logits(LlamaModel.from_state_dict(cfg, sd, device="cpu"), cfg)
    for _rank, logits in got:
        logits = torch.from_numpy(logits)
        # same experts, same tokens; only the order of the fp32 sums over experts differs
        torch.testing.assert_close(logits, ref, atol=3e-2, rtol=3e-2)
        assert logits.argmax(-1).tolist() == ref.argmax(-1).tolist()


# ---------------------------------------------------------------------------------------------------------------
# Elastic recovery: a 4-rank tensor-parallel generation loses a rank between steps; the survivors detect it by
# heartbeat, re-form a 2-rank group, re-shard the weights from the checkpoint, re-prefill prompt + accepted tokens
# and finish with the tokens a fresh 2-rank run produces.
# ---------------------------------------------------------------------------------------------------------------
_EL_PROMPTS = [[5, 6, 7, 8, 9, 10, 11], [21, 22, 23]]
_EL_GEN = 8
_EL_FAIL_STEP = 4


def _elastic_engine_factory(cfg, sd):
    from antfly_b200.models.llama import LlamaModel
    from antfly_b200.parallel.comm import TpComm
    from antfly_b200.runtime.engine import LLMEngine

    def build(tp_rank, tp_size):
        comm = TpComm(tp_rank, tp_size, torch.device("cpu")) if tp_size > 1 else None
        model = LlamaModel.from_state_dict(cfg, sd, device="cpu", tp_rank=tp_rank, tp_size=tp_size, comm=comm)
        return LLMEngine(model, num_blocks=32, page=16, max_batch=4, use_cuda_graph=False)

    return build


def _elastic_worker(uid, world, store_port, fail_uid, q):
    from antfly_b200.parallel.health import ElasticGroup, GroupLost, elastic_generate
    from antfly_b200.runtime.sampling_params import SamplingParams

    store = dist.TCPStore("127.0.0.1", store_port, is_master=False, timeout=__import__("datetime").timedelta(seconds=60))
    group = ElasticGroup(store, uid, list(range(world)), backend="gloo", timeout_s=8.0, dead_after_s=1.5)
    group.form()
    cfg = _tp_cfg(4)
    build = _elastic_engine_factory(cfg, _hf_llama_state(cfg))

    def before_step(step_no, g):
        if fail_uid is not None and uid == fail_uid and step_no == _EL_FAIL_STEP and g.world == world:
            q.put(("left", uid, None))
            q.close()
            q.join_thread()   # the message is on its way before the process goes
            os._exit(0)   # leaves between steps: nothing in flight; the others learn of it on the host

    try:
        res = elastic_generate(group, build, _EL_PROMPTS, SamplingParams(max_tokens=_EL_GEN, ignore_eos=True),
                               before_step=before_step)
        q.put(("done", uid, res))
    except GroupLost:
        q.put(("spare", uid, None))
    if dist.is_initialized():
        dist.destroy_process_group()


def _run_elastic(world, fail_uid):
    import datetime

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    store = dist.TCPStore("127.0.0.1", port, is_master=True, timeout=datetime.timedelta(seconds=60),
                          wait_for_workers=False)  # outlives every rank: hosted by the launcher
    procs = [ctx.Process(target=_elastic_worker, args=(u, world, port, fail_uid, q)) for u in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    del store
    return got


def test_elastic_recovery_regroups_from_four_ranks_to_two_and_matches_a_fresh_two_rank_run():
    got = _run_elastic(4, fail_uid=3)
    kinds = sorted((k, u) for k, u, _ in got)
    assert ("left", 3) in kinds
    finished = {u: r for k, u, r in got if k == "done"}
    spares = [u for k, u, _ in got if k == "spare"]
    assert sorted(finished) == [0, 1] and spares == [2]          # three survivors: the group of two is ranks 0, 1
    for res in finished.values():
        assert res["regroups"] == 1 and res["world"] == 2 and res["members"] == [0, 1]
    fresh = _run_elastic(2, fail_uid=None)
    want = [r for k, u, r in fresh if k == "done"][0]["tokens"]
    assert all(len(t) == _EL_GEN for t in want)
    for res in finished.values():
        assert res["tokens"] == want


def test_largest_power_of_two_group_and_first_proposal_wins():
    from antfly_b200.parallel.health import ElasticGroup, largest_power_of_two_group

    assert largest_power_of_two_group([0, 1, 2, 4, 5, 6, 7]) == [0, 1, 2, 4]
    assert largest_power_of_two_group([3, 1, 6]) == [1, 3]
    assert largest_power_of_two_group([5]) == [5]

    class FakeStore(dict):
        def set(self, k, v): self[k] = v.encode() if isinstance(v, str) else v
        def get(self, k): return self[k]
        def check(self, ks): return all(k in self for k in ks)
        def compare_set(self, k, expect, new):
            if k not in self:
                self[k] = new.encode()
            return self[k]

    store = FakeStore()
    import time as _t
    now = repr(_t.time())
    for r in (0, 1, 2):
        store.set(f"afb/hb/{r}", now)
    a = ElasticGroup(store, 0, [0, 1, 2, 3], dead_after_s=5.0)
    assert a.check() == [3]
    store.set("afb/regroup/1", "1,2")       # another survivor's proposal got there first
    b = ElasticGroup(store, 1, [0, 1, 2, 3], dead_after_s=5.0)
    b.form = lambda: None
    assert b.regroup() == [1, 2] and b.rank == 0 and b.world == 2 and b.epoch == 1


# ---------------------------------------------------------------------------------------------------------------
# Tensor-parallel encoder / cross-encoder: the reference's one real tensor-parallel consumer; it verifies a 2-rank
# run against the single-rank scores within 5e-4 (zig/pkg/inference/docs/RERANKING.md:109-112,
# scripts/verify_cross_encoder_rerank.sh).
# ---------------------------------------------------------------------------------------------------------------
def _bert_pairs():
    from antfly_b200.models.bert import pack_sequences

    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(5, 500, (int(n),), generator=g).tolist() for n in (12, 30, 7, 19)]
    types = [[0] * (len(s) // 2) + [1] * (len(s) - len(s) // 2) for s in seqs]
    return pack_sequences(seqs, types)


def _bert_tp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from antfly_b200.models.bert import BertConfig, BertModel
    from antfly_b200.parallel.comm import TpComm, init_process_group

    init_process_group(backend="gloo", timeout_s=60)
    cfg = BertConfig(hidden_size=128, num_hidden_layers=3, num_attention_heads=4, intermediate_size=256,
                     vocab_size=512, num_labels=1)
    full = BertModel.random_init(cfg, device="cpu", seed=0, dtype=torch.float32)
    model = full.tensor_parallel(rank, world, TpComm(rank, world, torch.device("cpu")))
    assert model.w["l0.qkv.w"].shape == (3 * 128 // world, 128) and model.w["l0.ff2.w"].shape == (128, 256 // world)
    b = _bert_pairs()
    q.put((rank, torch.sigmoid(model.classify(b)).flatten().tolist(), model.embed(b).numpy()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_cross_encoder_matches_single_rank_within_reference_tolerance(world):
    from antfly_b200.models.bert import BertConfig, BertModel

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_bert_tp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    cfg = BertConfig(hidden_size=128, num_hidden_layers=3, num_attention_heads=4, intermediate_size=256,
                     vocab_size=512, num_labels=1)
    single = BertModel.random_init(cfg, device="cpu", seed=0, dtype=torch.float32)
    b = _bert_pairs()
    want = torch.sigmoid(single.classify(b)).flatten()
    want_emb = single.embed(b)
    for _rank, scores, emb in got:
        assert (torch.tensor(scores) - want).abs().max() <= 5e-4
        torch.testing.assert_close(torch.from_numpy(emb), want_emb, atol=5e-4, rtol=1e-3)
