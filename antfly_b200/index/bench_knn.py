"""kNN throughput workload of bench.py: sharded brute-force or IVF search over a synthetic mixture-of-Gaussians
database (bf16 rows, or block-scaled fp8 rows with an exact re-score of a short list), queries drawn the same way.

Recall@10 is measured against exact fp32 search over the WHOLE database -- every rank's shard, scored in chunks so
no chunk's fp32 copy exceeds a few hundred MB -- on a sample of the timed queries, at any number of ranks: each
rank computes the exact top-10 of the sample over its own shard, the per-rank lists are gathered and merged.

Database size is a parameter: the headline config is 100M x 768 over 8 GPUs (12.5M rows per GPU = 19.2 GB bf16);
``--knn-rows`` is the number of rows per GPU.
"""
from __future__ import annotations

import json
import time

import torch


def mixture(n, d, centers, sigma, gen, device, chunk=1 << 20, dtype=torch.bfloat16):
    out = torch.empty((n, d), dtype=dtype, device=device)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        lab = torch.randint(0, centers.shape[0], (hi - lo,), generator=gen, device=device)
        x = centers[lab] + sigma * torch.randn(hi - lo, d, generator=gen, device=device)
        out[lo:hi] = torch.nn.functional.normalize(x, dim=-1).to(dtype)
    return out


def exact_topk_chunked(queries: torch.Tensor, x: torch.Tensor, k: int, id_offset: int, chunk: int = 1 << 18):
    """Exact cosine top-k of fp32 queries over bf16 rows, fp32 arithmetic, ``chunk`` rows at a time."""
    q = torch.nn.functional.normalize(queries.float(), dim=-1)
    best_v = torch.full((q.shape[0], k), float("inf"), device=x.device)
    best_i = torch.full((q.shape[0], k), -1, dtype=torch.long, device=x.device)
    for lo in range(0, x.shape[0], chunk):
        d = 1.0 - q @ x[lo:lo + chunk].float().t()
        v, i = d.topk(min(k, d.shape[1]), dim=-1, largest=False)
        cv, ci = torch.cat([best_v, v], 1), torch.cat([best_i, i + lo + id_offset], 1)
        best_v, j = cv.topk(k, dim=-1, largest=False)
        best_i = ci.gather(1, j)
    return best_v, best_i


def global_truth(sample: torch.Tensor, x: torch.Tensor, k: int, rank: int, world: int, rows: int):
    """Exact top-k ids of ``sample`` over all ranks' shards (identical on every rank)."""
    v, i = exact_topk_chunked(sample, x, k, rank * rows)
    if world > 1:
        import torch.distributed as dist

        vs = [torch.empty_like(v) for _ in range(world)]
        is_ = [torch.empty_like(i) for _ in range(world)]
        dist.all_gather(vs, v.contiguous())
        dist.all_gather(is_, i.contiguous())
        cv, ci = torch.cat(vs, 1), torch.cat(is_, 1)
        v, j = cv.topk(k, dim=-1, largest=False)
        i = ci.gather(1, j)
    return i


def bench_knn(args) -> None:
    import datetime

    from .. import _native as N
    from ..utils import benchlib as B
    from .flat import recall_at_k
    from .sharded import ShardedFlatIndex, ShardedIVFIndex

    rank, world, local = B.dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    d, nq, k = 768, 1024, 100
    rows = args.knn_rows
    g = torch.Generator(device=dev).manual_seed(1)
    centers = torch.randn(10000, d, generator=g, device=dev)
    gs = torch.Generator(device=dev).manual_seed(100 + rank)
    x = mixture(rows, d, centers, 0.3, gs, dev)
    kind, storage = args.knn_index, args.knn_storage
    t_build = time.perf_counter()
    if kind == "ivf":
        if storage != "bf16":
            raise SystemExit("--knn-index ivf stores its lists as bf16 rows")
        index = ShardedIVFIndex(x, args.knn_lists, "cosine", rank, world, rows, train_sample=min(rows, 1 << 21))
        search = lambda b: index.search(b, k, nprobe=args.knn_nprobe)
        what = f"IVF, {args.knn_lists} lists, nprobe {args.knn_nprobe}, cosine top-100"
    else:
        index = ShardedFlatIndex(x, "cosine", rank, world, rows, storage=storage)
        search = lambda b: index.search(b, k)
        what = "brute-force cosine top-100" + (" over block-fp8 rows" if storage == "fp8" else "")
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t_build
    gq = torch.Generator(device=dev).manual_seed(7)
    W, K = args.warmup, args.steps
    batches = [mixture(nq, d, centers, 0.3, gq, dev, dtype=torch.float32) for _ in range(W + 2 * K)]
    pinned = [b.cpu().pin_memory() for b in batches[W + K:]]
    clocks = B.clock_sampler()
    for b in batches[:W]:
        search(b)
    B.barrier(world)
    tb = datetime.datetime.now()
    n0 = N.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in batches[W:W + K]:
        search(b)
    e1.record()
    B.barrier(world)
    launches = N.launches() - n0
    clk = B.clock_summary(clocks, tb, datetime.datetime.now())
    ms = B.max_over_ranks(e0.elapsed_time(e1), world)
    # end to end: pinned host queries in, ids + distances back on the host
    B.barrier(world)
    t1 = time.perf_counter()
    d2h = 0
    for b in pinned:
        r = search(b.to(dev, non_blocking=True))
        ids, dist_ = r.ids.cpu(), r.distances.cpu()
        d2h += ids.numel() * ids.element_size() + dist_.numel() * 4
    B.barrier(world)
    e2e_s = B.max_over_ranks(time.perf_counter() - t1, world)
    # recall@10 of the first timed batch's first 64 queries against exact fp32 over every shard
    sample = batches[W][:64]
    truth = global_truth(sample, x, 10, rank, world, rows)
    found = search(batches[W]).ids[:64]
    recall = recall_at_k(found.long(), truth, 10)
    st = N.status()
    if rank == 0:
        print(json.dumps({
            "metric": "kNN queries/s at recall@10>=0.95", "value": round(nq * K / (ms / 1e3), 1), "unit": "queries/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if storage == "bf16" else "block-scaled fp8 (e4m3 + e8m0/32) rows, bf16 queries",
            "data": "synthetic: 10k-centre Gaussian mixture (sigma 0.3), unit-normalised",
            "config": {"model": what, "global_batch": nq, "seq_len": d, "database_rows": rows * world,
                       "parallelism": f"shard{world}", "recall_at_10": round(recall, 4),
                       "recall_sample": "64 queries vs exact fp32 over all shards", "build_s": round(build_s, 2),
                       "l2": "database shard far exceeds L2", "kernel_status": st},
            "clocks": clk,
            "e2e": {"value": round(nq * K / e2e_s, 1), "unit": "queries/s", "h2d_bytes_per_step": nq * d * 4,
                    "d2h_bytes_per_step": int(d2h / K)},
            "gpu_launches": int(launches)}))
    B.finish(world)
