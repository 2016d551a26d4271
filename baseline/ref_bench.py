"""Benchmark lines of the reference arm (``bench.py --impl reference --workload embed | rerank``).

Same metric, same configuration and the same JSON fields as this repository's own arm; the work runs through
``baseline/ref_cuda.py`` only (the reference's CUDA kernels, the reference's launch geometry and op sequence).
With several ranks every rank serves its own stream of batches on its own GPU -- the reference has no
data-parallel collective, several server processes are how it scales out -- and the slowest rank's time counts.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def _ranks():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def _max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def unavailable(reason: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


def run(args, clock_sampler, clock_summary) -> int:
    import datetime

    import torch

    if not torch.cuda.is_available():
        return unavailable("no CUDA device on this machine (the reference arm runs the reference's CUDA kernels)")
    import ref_cuda as R

    if not os.path.exists(R.CUBIN):
        try:
            import build_ref

            build_ref.build()
        except Exception as e:  # no reference checkout and nothing installed
            return unavailable(f"reference kernels not installed: {e}".replace("\n", " ")[:300])
    rank, world, local = _ranks()
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rerank = args.workload == "rerank"
    model = R.RefBert(R.RefBertConfig(num_labels=1 if rerank else 0), seed=0)
    W, K = args.warmup, args.steps
    per_step = 64 if rerank else 256

    def make(seed):
        if rerank:  # 64 pairs of query (32) + document (448) (+3 special tokens), padded to 512
            g = torch.Generator().manual_seed(seed)
            n = 32 + 448 + 3
            ids = torch.zeros((64, R.MAX_LENGTH), dtype=torch.int64)
            ids[:, :n] = torch.randint(1000, 30000, (64, n), generator=g)
            mask = torch.zeros_like(ids)
            mask[:, :n] = 1
            typ = torch.zeros_like(ids)
            typ[:, 34:n] = 1
            return ids.pin_memory(), mask.pin_memory(), typ.pin_memory()
        ids, mask, _ = R.synthetic_docs(256, 32, 512, seed=seed)
        return ids, mask, None

    batches = [make(1000 * rank + i) for i in range(W + 2 * K)]
    h2d = sum(b[0].numel() * 8 * (3 if rerank else 2) for b in batches[:1])  # ids, mask (, types) int64 per step

    def step_device(b):
        for lo, hi in R.request_chunks(per_step):
            model.forward(b[0][lo:hi], b[1][lo:hi], b[2][lo:hi] if b[2] is not None else None)

    def step_e2e(b):
        n = 0
        for lo, hi in R.request_chunks(per_step):
            out = (model.rerank_request(b[0][lo:hi], b[1][lo:hi], b[2][lo:hi]) if rerank
                   else model.embed_request(b[0][lo:hi], b[1][lo:hi]))
            n += out.numel() * out.element_size()
        return n

    clocks = clock_sampler()
    for b in batches[:W]:
        step_device(b)
    torch.cuda.synchronize()
    tb = datetime.datetime.now()
    l0 = model.mod.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in batches[W:W + K]:
        step_device(b)
    e1.record()
    torch.cuda.synchronize()
    launches = model.mod.launches - l0
    clk = clock_summary(clocks, tb, datetime.datetime.now())
    ms = _max_over_ranks(e0.elapsed_time(e1), world)
    t1 = time.perf_counter()
    d2h_user = 0
    for b in batches[W + K:W + 2 * K]:
        d2h_user += step_e2e(b)
    torch.cuda.synchronize()
    e2e_s = _max_over_ranks(time.perf_counter() - t1, world)
    # the reference's stock path downloads the whole hidden-state tensor and pools on the host
    d2h_hidden = per_step * R.MAX_LENGTH * model.cfg.hidden * 4
    if rank == 0:
        n = per_step * K * world
        unit = "pairs/s" if rerank else "docs/s"
        print(json.dumps({
            "impl": "reference", "metric": "rerank pairs/s" if rerank else "embed docs/s",
            "value": round(n / (ms / 1e3), 2), "unit": unit, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(ms / K, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp32 (the reference's CUDA kernels are fp32-only)",
            "data": "synthetic: uniform token ids, lengths U[32,512], random-init" if not rerank
                    else "synthetic: uniform token ids, random-init",
            "config": {"model": "BERT-base (12L, 768, 12 heads, FFN 3072)" + (" + 1-logit head" if rerank else ""),
                       "global_batch": per_step * world,
                       "seq_len": "padded to max_length 512, requests of 32 sequences (the reference pipelines' "
                                  "defaults; one 256 x 512 call exceeds its launcher's grid.y limit)",
                       "parallelism": f"dp{world} (independent ranks)",
                       "what": "unmodified inference_cuda_kernels.cu of the reference (nvcc, sm_100a) driven with "
                               "the launch geometry of ops/cuda/kernels.zig and the op sequence of "
                               "architectures/bert.zig; its Zig host code cannot be built here",
                       "l2": "activations per request (16384 tokens x 768..3072 fp32) exceed L2"},
            "clocks": clk,
            "e2e": {"value": round(n / e2e_s, 2), "unit": unit, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h_hidden if not rerank else d2h_user / K)},
            "gpu_launches": int(launches)}))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0
