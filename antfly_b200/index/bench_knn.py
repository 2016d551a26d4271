"""kNN throughput workload of bench.py: sharded brute-force (and IVF) search over a synthetic mixture-of-Gaussians
database, queries drawn the same way, recall@10 measured against exact fp32 on a query subset.

Database size is a parameter: the headline config is 100M x 768 over 8 GPUs (12.5M rows per GPU = 19.2 GB bf16);
``--knn-rows`` sets the rows per GPU so a single-GPU run can use the per-GPU share of that config.
"""
from __future__ import annotations

import json
import os
import time

import torch


def _mixture(n, d, centers, sigma, gen, device, chunk=1 << 20, dtype=torch.bfloat16):
    out = torch.empty((n, d), dtype=dtype, device=device)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        lab = torch.randint(0, centers.shape[0], (hi - lo,), generator=gen, device=device)
        x = centers[lab] + sigma * torch.randn(hi - lo, d, generator=gen, device=device)
        out[lo:hi] = torch.nn.functional.normalize(x, dim=-1).to(dtype)
    return out


def bench_knn(args) -> None:
    import bench as B
    from .. import _native as N
    from .flat import exact_search_fp32, recall_at_k
    from .sharded import ShardedFlatIndex

    rank, world, local = B._dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    d, nq, k = 768, 1024, 100
    rows = args.knn_rows
    g = torch.Generator(device=dev).manual_seed(1)
    centers = torch.randn(10000, d, generator=g, device=dev)
    gs = torch.Generator(device=dev).manual_seed(100 + rank)
    x = _mixture(rows, d, centers, 0.3, gs, dev)
    index = ShardedFlatIndex(x, "cosine", rank, world, rows, storage="bf16")
    gq = torch.Generator(device=dev).manual_seed(7)
    W, K = args.warmup, args.steps
    batches = [_mixture(nq, d, centers, 0.3, gq, dev, dtype=torch.float32) for _ in range(W + 2 * K)]
    pinned = [b.cpu().pin_memory() for b in batches[W + K:]]
    import datetime

    clocks = B._clock_sampler()
    for b in batches[:W]:
        index.search(b, k)
    B._barrier(world)
    tb = datetime.datetime.now()
    n0 = N.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in batches[W:W + K]:
        res = index.search(b, k)
    e1.record()
    B._barrier(world)
    launches = N.launches() - n0
    clk = B._clock_summary(clocks, tb, datetime.datetime.now())
    ms = B._max_over_ranks(e0.elapsed_time(e1), world)
    # end to end: pinned host queries in, ids + distances back on the host
    B._barrier(world)
    t1 = time.perf_counter()
    d2h = 0
    for b in pinned:
        r = index.search(b.to(dev, non_blocking=True), k)
        ids, dist_ = r.ids.cpu(), r.distances.cpu()
        d2h += ids.numel() * 4 + dist_.numel() * 4
    B._barrier(world)
    e2e_s = B._max_over_ranks(time.perf_counter() - t1, world)
    # recall@10 against exact fp32 on a subset of queries (single rank: whole shard; multi-rank: rank 0's shard
    # is what it can check locally, so recall is reported for world == 1 only)
    recall = None
    if world == 1:
        sub = batches[W][:64]
        truth = exact_search_fp32(sub, x.float() if rows <= 2_000_000 else x, 10, "cosine") if rows <= 2_000_000 else None
        if truth is not None:
            recall = recall_at_k(index.search(sub, k).ids, truth.ids, 10)
    if rank == 0:
        total_rows = rows * world
        print(json.dumps({
            "metric": "kNN queries/s at recall@10>=0.95", "value": round(nq * K / (ms / 1e3), 1), "unit": "queries/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: 10k-centre Gaussian mixture (sigma 0.3), unit-normalised",
            "config": {"model": "brute-force cosine top-100", "global_batch": nq, "seq_len": d,
                       "database_rows": total_rows, "parallelism": f"shard{world}", "recall_at_10": recall,
                       "l2": "database shard far exceeds L2", "kernel_status": N.status()},
            "clocks": clk,
            "e2e": {"value": round(nq * K / e2e_s, 1), "unit": "queries/s", "h2d_bytes_per_step": nq * d * 4,
                    "d2h_bytes_per_step": int(d2h / K)},
            "gpu_launches": int(launches)}))
    B._finish(world)
