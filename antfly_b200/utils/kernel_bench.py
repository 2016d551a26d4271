"""Micro-benchmarks of single kernels (the counterpart of the reference's cuda_microbench,
zig/pkg/inference/src/bench/cuda_microbench.zig): one kernel, fixed shape, event-timed under CUDA-graph replay so
host launch cost is excluded, rotating through several weight copies so every launch reads cold data.

    python -m antfly_b200.utils.kernel_bench w8a16 --m 64 --n 4096 --k 4096 --split 4
    python -m antfly_b200.utils.kernel_bench gemm  --m 8192 --n 8192 --k 8192
    python -m antfly_b200.utils.kernel_bench attn  --batch 64 --ctx 2048
    python -m antfly_b200.utils.kernel_bench gguf  --type q4_k --m 1 --n 14336 --k 4096   (the reference's Q4_K shapes)
    python -m antfly_b200.utils.kernel_bench sinkattn --batch 64 --ctx 2048
    ... --plain N : no graph, N eager launches (the form to put under ncu)
"""
from __future__ import annotations

import argparse
import json

import torch


def _graph_time(fns, reps: int = 10) -> float:
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps / len(fns) * 1e3  # us per call


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["w8a16", "mxfp8", "gemm", "pgemm", "attn", "sinkattn", "norm", "encattn", "gguf"])
    ap.add_argument("--type", default="q4_k", help="gguf: tensor type of the weight (q4_0, q8_0, q4_k, q6_k, ...)")
    ap.add_argument("--m", type=int, default=64)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--split", type=int, default=1)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--plain", type=int, default=0)
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--terms", type=int, default=2)
    args = ap.parse_args()
    from ..ops import attention as A
    from ..ops import dense as Dn
    from ..ops import quant as Q

    dev = "cuda"
    res = {"kernel": args.kernel}
    if args.kernel == "w8a16":
        M, Nn, K = args.m, args.n, args.k
        copies = args.copies or max(2, min(16, (300 << 20) // (Nn * K) + 1))
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        ws = [Q.random_fp8(Nn, K, dev, seed=i, interleaved_swiglu=args.swiglu) for i in range(copies)]
        if args.swiglu:
            fns = [(lambda w=w: Q.gemm_w8a16(x, w, swiglu=True)) for w in ws]
        else:
            fns = [(lambda w=w: Q.gemm_w8a16(x, w, split_k=args.split, partials=True)) for w in ws]
        nbytes, flops = Nn * K + Nn * K // 32, 2.0 * M * Nn * K
    elif args.kernel == "mxfp8":
        M, Nn, K = args.m, args.n, args.k
        copies = args.copies or max(2, min(16, (300 << 20) // (Nn * K) + 1))
        x = Q.quantize_mx(torch.randn(M, K, device=dev).to(torch.bfloat16), terms=args.terms)
        ws = [Q.random_fp8(Nn, K, dev, seed=i, interleaved_swiglu=args.swiglu) for i in range(copies)]
        for w in ws:
            Q.weight_sf_atoms(w)
        if args.swiglu:
            fns = [(lambda w=w: Q.gemm_mxfp8(x, w, swiglu=True)) for w in ws]
        else:
            fns = [(lambda w=w: Q.gemm_mxfp8(x, w, split_k=args.split, partials=True)) for w in ws]
        nbytes, flops = Nn * K + Nn * K // 32, 2.0 * M * Nn * K
    elif args.kernel in ("gemm", "pgemm"):
        M, Nn, K = args.m, args.n, args.k
        copies = args.copies or max(2, min(8, (300 << 20) // (2 * (M * K + Nn * K)) + 1))
        a = [torch.randn(M, K, device=dev).to(torch.bfloat16) for _ in range(copies)]
        w = [torch.randn(Nn, K, device=dev).to(torch.bfloat16) for _ in range(copies)]
        out = torch.empty(M, Nn, device=dev, dtype=torch.bfloat16)
        if args.kernel == "pgemm":
            from ..ops import index_ops as IX

            fns = [(lambda i=i: IX.gemm_persistent(a[i], w[i], out=out)) for i in range(copies)]
        else:
            fns = [(lambda i=i: Dn.gemm_bf16(a[i], w[i], out=out, tile_n=args.tile_n)) for i in range(copies)]
        nbytes, flops = 2 * (M * K + Nn * K + M * Nn), 2.0 * M * Nn * K
    elif args.kernel == "attn":
        B, ctx, Hq, Hkv, D, page = args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim, 16
        nblk = (ctx + page - 1) // page
        copies = args.copies or 4
        kcs = [torch.randn(B * nblk, page, Hkv, D, device=dev).to(torch.bfloat16) for _ in range(copies)]
        vcs = [torch.randn(B * nblk, page, Hkv, D, device=dev).to(torch.bfloat16) for _ in range(copies)]
        tables = torch.arange(B * nblk, dtype=torch.int32, device=dev).view(B, nblk)
        q = torch.randn(B, Hq, D, device=dev).to(torch.bfloat16)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        ones = torch.ones_like(ar)
        kvl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        scratch = A.PagedAttnScratch(B, Hq, D, max(args.splits, 1), dev) if args.splits > 1 else None
        fns = [(lambda i=i: A.paged_attention(q, kcs[i], vcs[i], tables, ar, ones, kvl, 1, num_splits=args.splits,
                                               scratch=scratch)) for i in range(copies)]
        nbytes, flops = 2 * B * ctx * Hkv * D * 2, 4.0 * B * Hq * ctx * D
    elif args.kernel == "sinkattn":
        B, ctx, Hq, Hkv, D, page = args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim, 16
        nblk = (ctx + page - 1) // page
        copies = args.copies or 4
        kcs = [torch.randn(B * nblk, page, Hkv, D, device=dev).to(torch.bfloat16) for _ in range(copies)]
        vcs = [torch.randn(B * nblk, page, Hkv, D, device=dev).to(torch.bfloat16) for _ in range(copies)]
        tables = torch.arange(B * nblk, dtype=torch.int32, device=dev).view(B, nblk)
        q = torch.randn(B, Hq, D, device=dev).to(torch.bfloat16)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        ones = torch.ones_like(ar)
        kvl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        sinks = torch.zeros(Hq, device=dev)
        out = torch.empty_like(q)
        fns = [(lambda i=i: A.paged_attention_sink(q, kcs[i], vcs[i], tables, ar, ones, kvl, sinks=sinks, out=out))
               for i in range(copies)]
        nbytes, flops = 2 * B * ctx * Hkv * D * 2, 4.0 * B * Hq * ctx * D
    elif args.kernel == "gguf":
        from ..formats import gguf as GF
        from ..ops import gguf_ops as GO

        M, Nn, K = args.m, args.n, args.k
        ids = {v.lower(): k for k, v in GF.TYPE_NAMES.items()}
        tid = int(args.type) if args.type.isdigit() else ids[args.type.lower()]
        bv, bb = GO.block_geometry(tid)
        wbytes = Nn * (K // bv) * bb
        copies = args.copies or max(2, min(16, (300 << 20) // wbytes + 1))
        # timing only: zero bytes decode to finite values in every format, so the outputs stay finite
        ws = [torch.zeros(wbytes, dtype=torch.uint8, device=dev) for _ in range(copies)]
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        fns = [(lambda w=w: GO.linear_gguf(x, w, tid, Nn, K)) for w in ws]
        nbytes, flops = wbytes + 2 * M * (K + Nn), 2.0 * M * Nn * K
    elif args.kernel == "encattn":
        B, L, Hq, D = args.batch, args.ctx, args.heads, args.head_dim
        T = B * L
        qkv = torch.randn(T, 3 * Hq * D, device=dev).to(torch.bfloat16)
        q, k, v = (qkv[:, i * Hq * D:(i + 1) * Hq * D].view(T, Hq, D) for i in range(3))
        lens = torch.full((B,), L, dtype=torch.int32, device=dev)
        starts = (torch.arange(B, dtype=torch.int32, device=dev) * L).int()
        fns = [lambda: A.varlen_attention(q, k, v, starts, lens, L)]
        nbytes, flops = 4 * T * Hq * D * 2, 4.0 * B * Hq * L * L * D
    else:
        rows, H = args.m, args.n
        x = torch.randn(rows, H, device=dev).to(torch.bfloat16)
        g = torch.ones(H, device=dev, dtype=torch.bfloat16)
        fns = [lambda: Dn.norm(x, g, eps=1e-5, rms=True, residual=x, want_sum=True)]
        nbytes, flops = 4 * rows * H * 2, 0.0
    if args.plain:
        for i in range(args.plain):
            fns[i % len(fns)]()
        torch.cuda.synchronize()
        print(json.dumps({"kernel": args.kernel, "plain_launches": args.plain}))
        return
    us = _graph_time(fns)
    res.update({"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 1),
                "args": {k: v for k, v in vars(args).items() if k != "kernel"}})
    print(json.dumps(res))


if __name__ == "__main__":
    main()
