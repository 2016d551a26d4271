"""Per-op device timing of one decode step (the analogue of the reference CLI's ``--print-timing`` /
``gpt_timing_ms`` lines, zig/pkg/inference/PERF.md:151-166), measured with CUDA events around every kernel
wrapper call in eager mode.

    python -m antfly_b200.utils.op_timing --layers 2 --batch 64 --ctx 2048 --iters 20

Prints one line per (op, shape): calls per step, mean microseconds, share of the step, and for the weight GEMMs
and attention the achieved HBM bandwidth.
"""
from __future__ import annotations

import argparse
import collections
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()

    from ..models import llama as L
    from ..ops import attention as A
    from ..ops import dense as Dn
    from ..ops import quant as Q
    from ..ops import sampling as S

    cfg = L.LlamaConfig.llama3_8b()
    cfg.num_hidden_layers = args.layers
    model = L.LlamaModel.random_init(cfg, device="cuda", seed=0)
    B, ctx, page = args.batch, args.ctx, 16
    nblk = (ctx + page) // page + 1
    kc = torch.randn((args.layers, B * nblk, page, cfg.num_key_value_heads, cfg.head_dim), device="cuda").to(
        torch.bfloat16)
    vc = torch.randn_like(kc)
    tables = torch.arange(B * nblk, dtype=torch.int32, device="cuda").view(B, nblk)
    ar = torch.arange(B, dtype=torch.int32, device="cuda")
    kvl = torch.full((B,), ctx + 1, dtype=torch.int32, device="cuda")
    slots = (tables[:, ctx // page] * page + ctx % page).int()
    batch = L.StepBatch(torch.randint(0, 1000, (B,), dtype=torch.int32, device="cuda"), kvl - 1, slots, ar,
                        torch.ones_like(ar), kvl, tables, ar, 1, 1)

    records = collections.OrderedDict()
    pending = []

    def wrap(mod, name, label, bytes_fn=None):
        orig = getattr(mod, name)

        def f(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = orig(*a, **k)
            e1.record()
            key = label(*a, **k)
            pending.append((key, e0, e1, bytes_fn(*a, **k) if bytes_fn else 0))
            return out

        setattr(mod, name, f)

    wrap(Q, "gemm_w8a16", lambda x, w, **k: f"gemm_w8a16 M={x.shape[0]} N={w.out_features} K={w.in_features}"
         + (" swiglu" if k.get("swiglu") else f" split={k.get('split_k', 1)}"), lambda x, w, **k: w.nbytes())
    wrap(Q, "gemm_mxfp8", lambda x, w, **k: f"gemm_mxfp8 M={x.q0.shape[0]} N={w.out_features} K={w.in_features}"
         + (" swiglu" if k.get("swiglu") else f" split={k.get('split_k', 1)}"), lambda x, w, **k: w.nbytes())
    wrap(Q, "quantize_mx", lambda x, **k: f"quantize_mx K={x.shape[1]}")
    wrap(A, "rope_kv_write", lambda *a, **k: "rope_kv_write")
    wrap(A, "paged_attention", lambda q, kcache, *a, **k: f"paged_attention ctx={ctx}",
         lambda q, kcache, *a, **k: 2 * B * ctx * kcache.shape[2] * kcache.shape[3] * 2)
    wrap(Dn, "norm", lambda *a, **k: "norm(+residual+partials)" if k.get("partials") is not None else "norm")
    wrap(Dn, "embed_gather", lambda *a, **k: "embed_gather")
    wrap(S, "argmax", lambda *a, **k: "argmax")

    for it in range(args.iters + 3):
        if it == 3:
            pending.clear()
        lg = model.forward(batch, kc, vc)
        model.greedy_tokens(lg)
    torch.cuda.synchronize()
    for key, e0, e1, nb in pending:
        r = records.setdefault(key, [0, 0.0, nb])
        r[0] += 1
        r[1] += e0.elapsed_time(e1) * 1e3
    total = sum(r[1] for r in records.values()) / args.iters
    rows = []
    for key, (n, us, nb) in records.items():
        mean = us / n
        rows.append({"op": key, "calls_per_step": n / args.iters, "mean_us": round(mean, 2),
                     "share": round(us / args.iters / total, 4),
                     "gbps": round(nb / mean / 1e3, 1) if nb else None})
    if args.json:
        print(json.dumps({"total_us_per_step": total, "rows": rows}))
        return
    print(f"decode step, {args.layers} layers, batch {B}, ctx {ctx}: {total:.1f} us of kernels (event-timed, eager)")
    for r in rows:
        bw = f"{r['gbps']:8.1f} GB/s" if r["gbps"] else ""
        print(f"  {r['op']:<52} x{r['calls_per_step']:<5.1f} {r['mean_us']:9.2f} us  {100 * r['share']:5.1f}%  {bw}")


if __name__ == "__main__":
    main()
