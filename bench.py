#!/usr/bin/env python
"""Headline benchmark: greedy decode throughput of a Llama-3-8B-architecture generator.

Config: 32 layers, hidden 4096, 32 heads / 8 KV heads, FFN 14336 SwiGLU, vocab 128256,
RoPE theta 500000, random-init block-scaled fp8 weights, bf16 activations, 64 concurrent prompts of 2048
uniform-random token ids, paged KV (block 16), greedy decoding, tensor parallel over --gpus ranks.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torch.distributed.run)

A "step" is one decode step of the whole batch (64 new tokens).  The prompts are prefilled through the same
engine before the timed region (prefill is not part of the decode metric; its time is reported in `config`).
`value`   : tokens/s over K decode steps timed with CUDA events around a host-sync-free burst (graph replays).
`e2e`     : tokens/s over K steps of LLMEngine.step(), each with its pinned-memory H2D of the step's inputs and
            a D2H read of the sampled tokens (wall clock between synchronisations).
Other workloads: --workload embed | rerank | knn (--knn-index flat|ivf, --knn-storage bf16|fp8) | spec | cpu.
Other arms: --impl reference (the reference's CUDA kernels; embed and rerank) | torch_nccl (library stand-in).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


from antfly_b200.utils.benchlib import (barrier as _barrier, clock_sampler as _clock_sampler,  # noqa: E402
                                        clock_summary as _clock_summary, dist_setup as _dist_setup,
                                        finish as _finish, log as _log, max_over_ranks as _max_over_ranks)


def bench_decode(args):
    import torch

    from antfly_b200 import _native as N
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.runtime.engine import LLMEngine, decode_burst
    from antfly_b200.runtime.sampling_params import SamplingParams

    rank, world, local = _dist_setup(args.gpus)
    cfg = LlamaConfig.llama3_8b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    comm = None
    if world > 1:
        from antfly_b200.parallel.comm import TpComm

        comm = TpComm(rank, world, torch.device("cuda", local), hidden=cfg.hidden_size, max_tokens=8192)
    if args.emulate_tp > 1 and world == 1:
        # Debug: run rank 0's shard of a tp-way split alone, without any communication (results are not a model
        # output; the point is the per-GPU compute time of the sharded shapes).
        model = LlamaModel.random_init(cfg, device=torch.device("cuda", local), seed=0, tp_rank=0,
                                       tp_size=args.emulate_tp, comm=None)
    else:
        model = LlamaModel.random_init(cfg, device=torch.device("cuda", local), seed=0, tp_rank=rank, tp_size=world,
                                       comm=comm)
    if args.force_fused and world == 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29588")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", local))
    if (world > 1 or args.force_fused) and args.tp_path in ("fused", "fused2"):
        from antfly_b200.parallel.fused import FusedTp, SymmetricWorkspace

        model.fused = FusedTp(SymmetricWorkspace(rank, world, torch.device("cuda", local), cfg.hidden_size,
                                                 max_tokens=128), one_shot=args.tp_path == "fused")
        # Pre-flight: every fused hand-off once, checked against NCCL.  If it does not hold on this machine the run
        # continues on the NCCL path and says so in its output line.
        try:
            fused_ok = model.fused.self_check()
        except Exception:
            fused_ok = False
        if not fused_ok:
            model.fused = None
            args.tp_path = "nccl (fused path failed its pre-flight check)"
        _log(f"fused pre-flight: {fused_ok}")
    B, prompt_len, gen = args.batch, args.prompt_len, args.gen_len
    total = prompt_len + gen + 16
    blocks = B * ((total + 15) // 16) + 8
    eng = LLMEngine(model, num_blocks=blocks, page=16, max_batch=B, max_step_tokens=8192, prefill_chunk=2048,
                    max_seq_len=total, use_cuda_graph=not os.environ.get("ANTFLY_B200_NO_GRAPH"))
    _log("model and engine ready")
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (B, prompt_len), generator=g).tolist()
    sp = SamplingParams(max_tokens=gen, ignore_eos=True)
    _barrier(world)
    t0 = time.perf_counter()
    for p in prompts:
        eng.add_request(p, sp)
    while eng.sched.snapshot()["waiting"] + eng.sched.snapshot()["prefill"] > 0:
        eng.step()
        _log(f"prefill step done, {eng.sched.snapshot()}")
    _barrier(world)
    prefill_s = time.perf_counter() - t0
    _log(f"prefill done in {prefill_s:.2f}s")

    W, K = args.warmup, args.steps
    assert W >= 3, "at least 3 warm-up steps"
    assert W + 2 * K + 1 <= gen, "warm-up + timed steps exceed the generation length"
    clocks = _clock_sampler()
    for _ in range(W):
        eng.step()
    _log("warm-up done")
    # A bounded wait that expired during warm-up (a rank missing, a hand-off that never arrived) means the numbers
    # would be garbage and every further step would cost a wait limit: stop here instead of queueing more work.
    st0 = int(_max_over_ranks(float(N.status()), world))
    if st0 != 0:
        if rank == 0:
            print(json.dumps({"metric": "decode tok/s @8B TP", "error": "a kernel wait expired during warm-up",
                              "kernel_status": st0, "n_gpus": world}))
        _finish(world)
        return
    # ---- end-to-end: K engine steps, each with its H2D of inputs and D2H of tokens ----
    h2d0, d2h0 = eng.h2d_bytes, eng.d2h_bytes
    _barrier(world)
    t1 = time.perf_counter()
    for _ in range(K):
        eng.step()
    _barrier(world)
    e2e_s = _max_over_ranks(time.perf_counter() - t1, world)
    h2d_step = (eng.h2d_bytes - h2d0) / K
    d2h_step = (eng.d2h_bytes - d2h0) / K
    _log("e2e steps done")
    # ---- device-timed burst ----
    _barrier(world)
    import datetime

    tb = datetime.datetime.now()
    _, ms, launches = decode_burst(eng, K)
    _barrier(world)
    clk = _clock_summary(clocks, tb, datetime.datetime.now())
    ms = _max_over_ranks(ms, world)
    st = N.status()
    value = B * K / (ms / 1e3)
    e2e = B * K / e2e_s
    if rank == 0:
        out = {
            "metric": "decode tok/s @8B TP", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 activations, block-scaled fp8 (e4m3 + e8m0/32) weights",
            "data": "synthetic: uniform-random token ids, random-init weights",
            "config": {"model": "Llama-3-8B architecture" + (f" ({cfg.num_hidden_layers} layers)" if args.layers else ""),
                       "global_batch": B, "seq_len": prompt_len, "gen_len": gen, "parallelism": f"tp{world}" + (f" ({args.tp_path})" if world > 1 else "") +
                       (f" EMULATED shard of tp{args.emulate_tp}, no comm: not a headline number" if args.emulate_tp > 1 else ""),
                       "kv": "paged bf16, block 16", "l2": "inputs (weights + KV read per step) far exceed L2",
                       "prefill_s": round(prefill_s, 3), "kernel_status": st},
            "clocks": clk,
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d_step),
                    "d2h_bytes_per_step": int(d2h_step), "ms_per_step": round(e2e_s * 1e3 / K, 4)},
            "gpu_launches": int(launches),
        }
        print(json.dumps(out))
    _finish(world)


def bench_embed(args):
    import torch

    from antfly_b200 import _native as N
    from antfly_b200.models.bert import BertConfig, BertModel
    from antfly_b200.pipelines.embedding import Embedder, synthetic_batches

    rank, world, local = _dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    model = BertModel.random_init(BertConfig.base(), device=dev, seed=0)
    emb = Embedder(model)
    if world > 1:
        # Data parallel: every rank embeds its own 256 documents; the pooling kernel pushes the finished rows
        # into every rank's gathered buffer, so each step ends with all world * 256 embeddings on every rank.
        from antfly_b200.parallel.dp_embed import DpEmbedder

        dp = DpEmbedder(model, rank, world, max_local_batch=256)
        emb.embed_packed = lambda b: dp.embed(b, emb.pooling, emb.normalize)
    W, K = args.warmup, args.steps
    batches = synthetic_batches(W + 2 * K, batch=256, lo=32, hi=512, vocab=(1000, 30000), seed=rank)
    pinned = [b.pin() for b in batches]
    dev_batches = [b.to(dev) for b in pinned[W:W + K]]
    import datetime

    clocks = _clock_sampler()
    for b in pinned[:W]:
        emb.embed_packed(b.to(dev))
    _barrier(world)
    tb = datetime.datetime.now()
    n0 = N.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in dev_batches:
        emb.embed_packed(b)
    e1.record()
    _barrier(world)
    launches = N.launches() - n0
    clk = _clock_summary(clocks, tb, datetime.datetime.now())
    ms = _max_over_ranks(e0.elapsed_time(e1), world)
    # end to end: pinned host ids -> device -> embeddings -> host
    h2d = sum(b.nbytes() for b in pinned[W + K:W + 2 * K]) / K
    _barrier(world)
    t1 = time.perf_counter()
    d2h = 0
    for b in pinned[W + K:W + 2 * K]:
        out = emb.embed_host(b)
        d2h += out.numel() * out.element_size()
    _barrier(world)
    e2e_s = _max_over_ranks(time.perf_counter() - t1, world)
    if rank == 0:
        docs = 256 * K * world
        print(json.dumps({
            "metric": "embed docs/s", "value": round(docs / (ms / 1e3), 1), "unit": "docs/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: uniform token ids, lengths U[32,512], random-init",
            "config": {"model": "BERT-base (12L, 768, 12 heads, FFN 3072)", "global_batch": 256 * world,
                       "seq_len": "U[32,512] packed (no padding)", "parallelism": f"dp{world}",
                       "l2": "activations per batch (~69k tokens x 768..3072 bf16) exceed L2",
                       "kernel_status": N.status()},
            "clocks": clk,
            "e2e": {"value": round(docs / e2e_s, 1), "unit": "docs/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h / K)},
            "gpu_launches": int(launches)}))
    _finish(world)


def bench_rerank(args):
    """Cross-encoder reranking: BERT-base + 1-logit head, 64 (query 32, document 448) pairs per query; one step is
    one query's 64 pairs.  Data parallel over ranks (each rank scores its own queries)."""
    import datetime

    import torch

    from antfly_b200 import _native as N
    from antfly_b200.models.bert import BertConfig, BertModel
    from antfly_b200.pipelines.reranking import CrossEncoderReranker, synthetic_pairs

    rank, world, local = _dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    model = BertModel.random_init(BertConfig.base(num_labels=1), device=dev, seed=0)
    rr = CrossEncoderReranker(model)
    W, K = args.warmup, args.steps
    batches = synthetic_pairs(W + 2 * K, docs_per_query=64, q_len=32, d_len=448, seed=rank)
    pinned = [b.pin() for b in batches]
    dev_batches = [b.to(dev) for b in pinned[W:W + K]]
    clocks = _clock_sampler()
    for b in pinned[:W]:
        rr.score_packed(b.to(dev))
    _barrier(world)
    tb = datetime.datetime.now()
    n0 = N.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in dev_batches:
        rr.score_packed(b)
    e1.record()
    _barrier(world)
    launches = N.launches() - n0
    clk = _clock_summary(clocks, tb, datetime.datetime.now())
    ms = _max_over_ranks(e0.elapsed_time(e1), world)
    h2d = sum(b.nbytes() for b in pinned[W + K:W + 2 * K]) / K
    _barrier(world)
    t1 = time.perf_counter()
    d2h = 0
    for b in pinned[W + K:W + 2 * K]:
        out = rr.score_host(b)
        d2h += out.numel() * out.element_size()
    _barrier(world)
    e2e_s = _max_over_ranks(time.perf_counter() - t1, world)
    if rank == 0:
        pairs = 64 * K * world
        print(json.dumps({
            "metric": "rerank pairs/s", "value": round(pairs / (ms / 1e3), 1), "unit": "pairs/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: uniform token ids, random-init",
            "config": {"model": "BERT-base + 1-logit head (cross-encoder)", "global_batch": 64 * world,
                       "seq_len": "32 + 448 (+3 special) per pair, packed", "parallelism": f"dp{world}",
                       "l2": "activations per query (~31k tokens x 768..3072 bf16) exceed L2",
                       "kernel_status": N.status()},
            "clocks": clk,
            "e2e": {"value": round(pairs / e2e_s, 1), "unit": "pairs/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h / K)},
            "gpu_launches": int(launches)}))
    _finish(world)


def bench_spec(args):
    """Speculative decoding, RAG-style: Llama-3-70B architecture (80 layers, hidden 8192, 64 heads / 8 KV heads, FFN
    28672), block-fp8, tensor parallel over the ranks; the draft is the target's first 8 layers with the shared
    embedding and LM head, 4 draft tokens per round; 16 prompts of 8192 uniform-random token ids, 512 generated
    tokens each.  A step is one speculative round of the whole batch (draft x 4, one verify pass, accept).  Reports
    tokens/s over the timed rounds, the acceptance rate and the median time to first token."""
    import datetime

    import torch

    from antfly_b200 import _native as N
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    rank, world, local = _dist_setup(args.gpus)
    cfg = LlamaConfig.llama3_70b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    comm = None
    if world > 1:
        from antfly_b200.parallel.comm import TpComm

        comm = TpComm(rank, world, torch.device("cuda", local), hidden=cfg.hidden_size, max_tokens=8192)
    model = LlamaModel.random_init(cfg, device=torch.device("cuda", local), seed=0, tp_rank=rank, tp_size=world,
                                   comm=comm)
    B, P, G, Kd = args.spec_batch, args.spec_prompt_len, args.spec_gen_len, 4
    total = P + G + 32
    eng = LLMEngine(model, num_blocks=B * ((total + 15) // 16) + 8, page=16, max_batch=B, max_step_tokens=8192,
                    prefill_chunk=2048, max_seq_len=total, draft_layers=min(8, cfg.num_hidden_layers), spec_k=Kd)
    g = torch.Generator().manual_seed(4321)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g).tolist()
    sp = SamplingParams(max_tokens=G, ignore_eos=True)
    _barrier(world)
    rids = [eng.add_request(p, sp) for p in prompts]
    while eng.sched.snapshot()["waiting"] + eng.sched.snapshot()["prefill"] > 0:
        eng.step()
    _barrier(world)
    ttft = sorted((eng.reqs[r].t_first - eng.reqs[r].t_admit) for r in rids if eng.reqs[r].t_first)
    W, K = args.warmup, args.steps
    assert W >= 3
    clocks = _clock_sampler()
    for _ in range(W):
        eng.step()
    st0 = eng.spec
    a0, d0, m0 = st0.accepted, st0.drafted, st0.matched
    h2d0, d2h0, l0 = eng.h2d_bytes, eng.d2h_bytes, N.launches()
    _barrier(world)
    tb = datetime.datetime.now()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t1 = time.perf_counter()
    e0.record()
    for _ in range(K):
        if not eng.has_work():
            break
        eng.step()
    e1.record()
    _barrier(world)
    wall = _max_over_ranks(time.perf_counter() - t1, world)
    ms = _max_over_ranks(e0.elapsed_time(e1), world)
    clk = _clock_summary(clocks, tb, datetime.datetime.now())
    toks = eng.spec.accepted - a0
    drafted, matched = eng.spec.drafted - d0, eng.spec.matched - m0
    if rank == 0:
        print(json.dumps({
            "metric": "speculative decode tok/s @70B TP", "value": round(toks / (ms / 1e3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 activations, block-scaled fp8 (e4m3 + e8m0/32) weights",
            "data": "synthetic: uniform-random token ids, random-init weights",
            "config": {"model": "Llama-3-70B architecture" + (f" ({cfg.num_hidden_layers} layers)" if args.layers else ""),
                       "draft": "first 8 layers + shared embedding and LM head, 4 tokens per round",
                       "global_batch": B, "seq_len": P, "gen_len": G, "parallelism": f"tp{world}",
                       "acceptance_rate": round(matched / max(drafted, 1), 4),
                       "tokens_per_round_per_sequence": round(toks / max(K * B, 1), 3),
                       "ttft_p50_s": round(ttft[len(ttft) // 2], 4) if ttft else None,
                       "l2": "weights + KV read per round far exceed L2", "kernel_status": N.status()},
            "clocks": clk,
            "e2e": {"value": round(toks / wall, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": int((eng.h2d_bytes - h2d0) / max(K, 1)),
                    "d2h_bytes_per_step": int((eng.d2h_bytes - d2h0) / max(K, 1))},
            "gpu_launches": int(N.launches() - l0)}))
    _finish(world)


def bench_cpu(args):
    """The CPU fp32 plumbing config: 6-layer BERT-style bi-encoder (hidden 384, 12 heads, FFN 1536) on 32 x 128
    token ids, mean pool + L2 normalise, then exact cosine top-10 against 100k x 384 unit vectors; all in the
    C++ CPU path.  A step is one embed + search; no GPU is used, so there are no clocks or launches to report."""
    import torch

    from antfly_b200.models.bert import BertConfig, BertModel
    from antfly_b200.ops import cpu_oracle as O

    cfg = BertConfig(vocab_size=30522, hidden_size=384, num_hidden_layers=6, num_attention_heads=12,
                     intermediate_size=1536, max_position_embeddings=512)
    model = BertModel.random_init(cfg, device=torch.device("cpu"), seed=0)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(1000, 30000, (32, 128), generator=g)
    ids[:, 0], ids[:, -1] = 101, 102
    g1 = torch.Generator().manual_seed(1)
    db = torch.nn.functional.normalize(torch.randn(100_000, 384, generator=g1), dim=-1)
    W, K = args.warmup, min(args.steps, 8)
    mask = torch.ones_like(ids)

    def step():
        e = O.bert_embed(model, ids, None, mask)
        e = torch.nn.functional.normalize(e, dim=-1)
        return O.topk(e, db, 10, "cosine")

    for _ in range(min(W, 3)):
        idx, _ = step()
    t0 = time.perf_counter()
    for _ in range(K):
        idx, _ = step()
    dt = (time.perf_counter() - t0) / K
    ref = (torch.nn.functional.normalize(O.bert_embed(model, ids, None, mask), dim=-1) @ db.T).topk(10, -1).indices
    exact = bool(torch.equal(idx.long().sort(-1).values, ref.sort(-1).values))
    print(json.dumps({"metric": "cpu fp32 embed + exact top-10 wall time", "value": round(dt * 1e3, 2), "unit": "ms",
                      "n_gpus": 0, "steps": K, "warmup": min(W, 3), "ms_per_step": round(dt * 1e3, 2),
                      "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
                      "data": "synthetic: token ids uniform in [1000, 30000), database N(0,1) unit-normalised",
                      "config": {"model": "6-layer BERT-style (384 hidden, 12 heads, FFN 1536)", "global_batch": 32,
                                 "seq_len": 128, "database": "100000 x 384", "top10_ids_exact": exact,
                                 "parallelism": "cpu"}, "gpu_launches": 0}))
    return 0


def _reference_arm(args):
    """The reference itself.  What of it can exist on this machine is its CUDA kernel file, compiled unchanged and
    driven with its own launch geometry (baseline/ref_cuda.py): enough for the BERT-base embed and rerank
    configurations.  Its CUDA backend has no RoPE, grouped-query or paged attention
    (zig/pkg/inference/src/ops/cuda/cuda_compute.zig:1256-1267 return unsupportedCt()), no index code runs on a
    GPU at all, and its Zig / Go host code does not build here, so the decode and kNN workloads have no reference
    arm."""
    if args.workload in ("embed", "rerank"):
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import ref_bench

        return ref_bench.run(args, _clock_sampler, _clock_summary)
    why = {"decode": "the reference's CUDA backend has no RoPE / grouped-query / paged attention (cuda_compute.zig:1256-1267 "
                     "return unsupportedCt()) and admits no Llama-class model; its Zig and Go sources have no Python "
                     "package (pip: 'neither setup.py nor pyproject.toml found') and neither toolchain is installed. "
                     "--workload embed and rerank have a reference arm",
           "knn": "the reference's vector index is CPU-only Zig / Go code that cannot be built here (no zig, no go)",
           "cpu": "the reference's CPU backend is Zig and cannot be built here (no zig toolchain)"}
    print(json.dumps({"impl": "reference", "unavailable": why.get(args.workload, why["decode"])}))
    return 0


def _torch_nccl_arm(args):
    """A constructed stand-in, NOT the reference: the same models as plain PyTorch modules (cuBLAS matmul, SDPA)
    with torch.distributed NCCL collectives -- the path "that only calls libraries"."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import torch_nccl

    return torch_nccl.run(args, _clock_sampler, _clock_summary)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="decode", choices=["decode", "embed", "knn", "rerank", "cpu", "spec"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--gen-len", type=int, default=256)
    ap.add_argument("--tp-path", default="fused", choices=["fused", "fused2", "nccl"],
                    help="tensor-parallel collectives: fused into the kernels over peer memory as one-shot "
                         "all-reduces (fused) or as reduce-scatter + all-gather (fused2), or the NCCL baseline")
    ap.add_argument("--knn-rows", type=int, default=12_500_000,
                    help="database rows per GPU for --workload knn (100M rows over 8 GPUs = 12.5M each)")
    ap.add_argument("--knn-index", default="flat", choices=["flat", "ivf"])
    ap.add_argument("--knn-storage", default="bf16", choices=["bf16", "fp8"])
    ap.add_argument("--knn-lists", type=int, default=16384)
    ap.add_argument("--knn-nprobe", type=int, default=64)
    ap.add_argument("--spec-batch", type=int, default=16)
    ap.add_argument("--spec-prompt-len", type=int, default=8192)
    ap.add_argument("--spec-gen-len", type=int, default=512)
    ap.add_argument("--emulate-tp", type=int, default=0,
                    help="debug: time one rank's shard of a tp-way split on a single GPU with no communication")
    ap.add_argument("--force-fused", action="store_true",
                    help="debug: run the peer-memory fused path with a single rank (pushes to itself)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (the result is then not the headline config)")
    args = ap.parse_args()
    if args.impl == "reference":
        return _reference_arm(args)
    if args.impl == "torch_nccl":
        return _torch_nccl_arm(args)
    if args.workload == "decode":
        bench_decode(args)
    elif args.workload == "embed":
        bench_embed(args)
    elif args.workload == "rerank":
        bench_rerank(args)
    elif args.workload == "cpu":
        return bench_cpu(args)
    elif args.workload == "spec":
        bench_spec(args)
    else:
        from antfly_b200.index.bench_knn import bench_knn

        bench_knn(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
