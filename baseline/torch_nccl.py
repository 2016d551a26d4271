"""Constructed library baseline (``bench.py --impl torch_nccl``): NOT the reference.

The reference ships neither an NCCL nor a cuBLAS build, and its own CUDA backend cannot run a Llama-class decoder.
This arm is the "path that only calls libraries" the fused kernels of the package are compared against: the same
architectures as plain PyTorch modules -- ``torch.matmul`` / ``F.linear`` (cuBLAS), ``scaled_dot_product_attention``
-- with ``torch.distributed`` NCCL collectives (all-reduce after row-parallel linears, all-gather of vocabulary
shards, embeddings and top-k candidates); decode steps run eagerly over the exact KV prefix.  Weights are bf16 (the libraries
have no block-scaled fp8 GEMM with 32-element e8m0 scales to call), the KV cache is contiguous rather than paged.
Nothing of the package is imported.  Every function also runs on CPU tensors (fp32) with tiny shapes for tests.
"""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass

import torch
import torch.nn.functional as F


def _ranks():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


# ------------------------------------------------------------------------------------------------------------------
# Llama-architecture decoder, Megatron tensor parallel
# ------------------------------------------------------------------------------------------------------------------
@dataclass
class LlamaShape:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    theta: float = 500000.0
    eps: float = 1e-5


class TorchLlama:
    def __init__(self, s: LlamaShape, rank: int, world: int, device, dtype, seed: int = 0, group=None):
        self.s, self.rank, self.world, self.dev, self.dt, self.group = s, rank, world, device, dtype, group
        self.hd = s.hidden // s.heads
        self.hq, self.hkv = s.heads // world, max(1, s.kv_heads // world)
        g = torch.Generator(device=device).manual_seed(seed + 17 * rank)

        def w(o, i):
            return (torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * i ** -0.5).to(dtype)

        gr = torch.Generator(device=device).manual_seed(seed)  # replicated tensors: same on every rank
        self.embed = (torch.randn(s.vocab, s.hidden, generator=gr, device=device, dtype=torch.float32) * 0.02).to(dtype)
        self.layers = []
        for _ in range(s.layers):
            self.layers.append({
                "qkv": w((self.hq + 2 * self.hkv) * self.hd, s.hidden), "o": w(s.hidden, self.hq * self.hd),
                "gu": w(2 * s.ffn // world, s.hidden), "d": w(s.hidden, s.ffn // world),
                "n1": torch.ones(s.hidden, device=device, dtype=dtype), "n2": torch.ones(s.hidden, device=device, dtype=dtype)})
        self.norm = torch.ones(s.hidden, device=device, dtype=dtype)
        self.head = w(s.vocab // world, s.hidden)
        inv = 1.0 / (s.theta ** (torch.arange(0, self.hd, 2, device=device, dtype=torch.float32) / self.hd))
        self.inv_freq = inv

    def _reduce(self, x):
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(x, group=self.group)
        return x

    def _rope(self, x, pos):  # x [B, T, H, D], pos [B, T]
        ang = pos[..., None].float() * self.inv_freq  # [B, T, D/2]
        cos, sin = ang.cos()[:, :, None, :], ang.sin()[:, :, None, :]
        x1, x2 = x[..., : self.hd // 2].float(), x[..., self.hd // 2:].float()
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)

    def new_cache(self, batch: int, max_len: int):
        shape = (self.s.layers, batch, self.hkv, max_len, self.hd)
        return torch.zeros(shape, device=self.dev, dtype=self.dt), torch.zeros(shape, device=self.dev, dtype=self.dt)

    def forward(self, ids, pos, kc, vc, batch_slice, kv_len_after: int, causal_chunk: bool):
        """ids / pos [B, T]; writes K/V at pos into the cache rows of `batch_slice`; attends to [0, kv_len_after).
        causal_chunk: T > 1 rows are causal inside the chunk (prefill); decode (T = 1) sees the whole prefix."""
        s = self.s
        B, T = ids.shape
        x = self.embed[ids]
        for li, L in enumerate(self.layers):
            h = F.rms_norm(x, (s.hidden,), L["n1"], s.eps)
            qkv = F.linear(h, L["qkv"]).view(B, T, self.hq + 2 * self.hkv, self.hd)
            q, k, v = qkv.split([self.hq, self.hkv, self.hkv], dim=2)
            q, k = self._rope(q, pos), self._rope(k, pos)
            idx = pos[:, None, :, None].expand(B, self.hkv, T, self.hd)
            kc[li, batch_slice].scatter_(2, idx, k.transpose(1, 2))
            vc[li, batch_slice].scatter_(2, idx, v.transpose(1, 2))
            kk, vv = kc[li, batch_slice, :, :kv_len_after], vc[li, batch_slice, :, :kv_len_after]
            mask = None
            if causal_chunk and T > 1:
                keys = torch.arange(kv_len_after, device=x.device)
                mask = keys[None, None, None, :] <= pos[:, None, :, None]
            a = F.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, attn_mask=mask, enable_gqa=True)
            x = x + self._reduce(F.linear(a.transpose(1, 2).reshape(B, T, self.hq * self.hd), L["o"]))
            h = F.rms_norm(x, (s.hidden,), L["n2"], s.eps)
            g, u = F.linear(h, L["gu"]).chunk(2, -1)
            x = x + self._reduce(F.linear(F.silu(g) * u, L["d"]))
        return F.rms_norm(x[:, -1], (s.hidden,), self.norm, s.eps)

    def greedy(self, last_hidden):
        logits = F.linear(last_hidden, self.head).float()
        val, idx = logits.max(-1)
        idx = idx + self.rank * (self.s.vocab // self.world)
        if self.world > 1:
            import torch.distributed as dist

            vals = [torch.empty_like(val) for _ in range(self.world)]
            idxs = [torch.empty_like(idx) for _ in range(self.world)]
            dist.all_gather(vals, val, group=self.group)
            dist.all_gather(idxs, idx, group=self.group)
            vals, idxs = torch.stack(vals), torch.stack(idxs)
            best = vals.max(0).values
            idx = torch.where(vals == best[None], idxs, torch.full_like(idxs, 2 ** 62)).min(0).values
        return idx


def decode_tokens(model: TorchLlama, prompts, gen: int, prefill_batch: int = 8):
    """Greedy generation (un-timed helper used by the CPU test): returns [B, gen] tokens."""
    B, P = prompts.shape
    kc, vc = model.new_cache(B, P + gen + 1)
    last = torch.empty((B, model.s.hidden), device=model.dev, dtype=model.dt)
    pos = torch.arange(P, device=model.dev)[None].expand(prefill_batch, P)
    for lo in range(0, B, prefill_batch):
        sl = slice(lo, min(B, lo + prefill_batch))
        n = sl.stop - sl.start
        last[sl] = model.forward(prompts[sl], pos[:n], kc, vc, sl, P, True)
    out = []
    tok = model.greedy(last)
    for t in range(gen):
        out.append(tok)
        p = torch.full((B, 1), P + t, device=model.dev, dtype=torch.long)
        tok = model.greedy(model.forward(tok[:, None], p, kc, vc, slice(0, B), P + t + 1, False))
    return torch.stack(out, 1)


# ------------------------------------------------------------------------------------------------------------------
# BERT-base encoder (padded to the batch maximum, key-padding mask)
# ------------------------------------------------------------------------------------------------------------------
class TorchBert:
    def __init__(self, device, dtype, layers=12, hidden=768, heads=12, ffn=3072, vocab=30522, num_labels=0, seed=0):
        g = torch.Generator(device=device).manual_seed(seed)
        r = lambda *s: (torch.randn(*s, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
        one, zero = (lambda n: torch.ones(n, device=device, dtype=dtype)), (lambda n: torch.zeros(n, device=device, dtype=dtype))
        self.heads, self.hidden = heads, hidden
        self.word, self.pos, self.typ = r(vocab, hidden), r(512, hidden), r(2, hidden)
        self.eg, self.eb = one(hidden), zero(hidden)
        self.layers = [{"qkv": (r(3 * hidden, hidden), r(3 * hidden)), "o": (r(hidden, hidden), r(hidden)),
                        "ln1": (one(hidden), zero(hidden)), "i": (r(ffn, hidden), r(ffn)), "d": (r(hidden, ffn), r(hidden)),
                        "ln2": (one(hidden), zero(hidden))} for _ in range(layers)]
        self.cls = (r(num_labels, hidden), r(num_labels)) if num_labels else None

    def forward(self, ids, mask, types=None):
        B, S = ids.shape
        H, nh = self.hidden, self.heads
        x = self.word[ids] + self.pos[:S][None] + self.typ[types if types is not None else torch.zeros_like(ids)]
        x = F.layer_norm(x, (H,), self.eg, self.eb, 1e-12)
        key_mask = mask[:, None, None, :].bool()
        for L in self.layers:
            q, k, v = F.linear(x, *L["qkv"]).view(B, S, 3, nh, H // nh).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=key_mask)
            x = F.layer_norm(x + F.linear(a.transpose(1, 2).reshape(B, S, H), *L["o"]), (H,), *L["ln1"], 1e-12)
            x = F.layer_norm(x + F.linear(F.gelu(F.linear(x, *L["i"])), *L["d"]), (H,), *L["ln2"], 1e-12)
        return x

    def embed(self, ids, mask):
        h = self.forward(ids, mask).float()
        m = mask[:, :, None].float()
        return F.normalize((h * m).sum(1) / m.sum(1).clamp_min(1), dim=-1)

    def score(self, ids, mask, types):
        return torch.sigmoid(F.linear(self.forward(ids, mask, types)[:, 0], *self.cls).float())


def padded_batch(n, lo, hi, seed, device):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n,), generator=g)
    S = int(lens.max())
    ids = torch.zeros((n, S), dtype=torch.long)
    for i, L in enumerate(lens.tolist()):
        ids[i, :L] = torch.randint(1000, 30000, (L,), generator=g)
    mask = (torch.arange(S)[None] < lens[:, None]).long()
    return ids.pin_memory() if device.type == "cuda" else ids, mask.pin_memory() if device.type == "cuda" else mask


# ------------------------------------------------------------------------------------------------------------------
# exact top-k over a sharded database
# ------------------------------------------------------------------------------------------------------------------
def knn_search(db, queries, k, id_offset, world, chunk=262144, group=None):
    best_v = torch.full((queries.shape[0], k), -float("inf"), device=db.device)
    best_i = torch.full((queries.shape[0], k), -1, device=db.device, dtype=torch.long)
    for lo in range(0, db.shape[0], chunk):
        s = (queries @ db[lo:lo + chunk].t()).float()
        v, i = s.topk(min(k, s.shape[1]), -1)
        cv, ci = torch.cat([best_v, v], 1), torch.cat([best_i, i + lo + id_offset], 1)
        best_v, j = cv.topk(k, -1)
        best_i = ci.gather(1, j)
    if world > 1:
        import torch.distributed as dist

        vs = [torch.empty_like(best_v) for _ in range(world)]
        is_ = [torch.empty_like(best_i) for _ in range(world)]
        dist.all_gather(vs, best_v, group=group)
        dist.all_gather(is_, best_i, group=group)
        cv, ci = torch.cat(vs, 1), torch.cat(is_, 1)
        best_v, j = cv.topk(k, -1)
        best_i = ci.gather(1, j)
    return 1 - best_v, best_i


# ------------------------------------------------------------------------------------------------------------------
def run(args, clock_sampler, clock_summary) -> int:
    import datetime

    if not torch.cuda.is_available():
        print(json.dumps({"impl": "torch_nccl", "unavailable": "no CUDA device on this machine"}))
        return 0
    rank, world, local = _ranks()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    def mx(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    W, K = args.warmup, args.steps
    clocks = clock_sampler()
    out = {"impl": "torch_nccl", "n_gpus": world, "steps": K, "warmup": W, "higher_is_better": True, "vs_baseline": None,
           "note": "constructed torch + cuBLAS + NCCL stand-in; not the reference"}
    if args.workload == "decode":
        B, P, G = args.batch, args.prompt_len, args.gen_len
        model = TorchLlama(LlamaShape(), rank, world, dev, torch.bfloat16)
        kc, vc = model.new_cache(B, P + G + 1)
        prompts = torch.randint(0, model.s.vocab, (B, P), generator=torch.Generator().manual_seed(1234)).to(dev)
        last = torch.empty((B, model.s.hidden), device=dev, dtype=torch.bfloat16)
        pos = torch.arange(P, device=dev)[None].expand(8, P)
        with torch.no_grad():
            for lo in range(0, B, 8):
                last[lo:lo + 8] = model.forward(prompts[lo:lo + 8], pos, kc, vc, slice(lo, lo + 8), P, True)
            tok = model.greedy(last)
            step = [0]

            def one():
                t = step[0]
                p = torch.full((B, 1), P + t, device=dev, dtype=torch.long)
                nonlocal_tok[0] = model.greedy(model.forward(nonlocal_tok[0][:, None], p, kc, vc, slice(0, B), P + t + 1, False))
                step[0] += 1

            nonlocal_tok = [tok]
            for _ in range(W):
                one()
            torch.cuda.synchronize()
            tb = datetime.datetime.now()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(K):
                one()
            e1.record()
            torch.cuda.synchronize()
            ms = mx(e0.elapsed_time(e1))
            t1 = time.perf_counter()
            for _ in range(K):
                one()
                _ = nonlocal_tok[0].cpu()
            e2e = mx(time.perf_counter() - t1)
        out.update({"metric": "decode tok/s @8B TP", "value": round(B * K / (ms / 1e3), 1), "unit": "tokens/s",
                    "ms_per_step": round(ms / K, 4), "scaling": "strong", "dtype": "bf16 (weights and activations)",
                    "data": "synthetic: uniform-random token ids, random-init weights",
                    "config": {"model": "Llama-3-8B architecture", "global_batch": B, "seq_len": P, "gen_len": G,
                               "parallelism": f"tp{world} (NCCL all-reduce)", "kv": "contiguous bf16",
                               "l2": "weights + KV read per step far exceed L2"},
                    "e2e": {"value": round(B * K / e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                            "d2h_bytes_per_step": B * 8}})
    elif args.workload in ("embed", "rerank"):
        rr = args.workload == "rerank"
        model = TorchBert(dev, torch.bfloat16, num_labels=1 if rr else 0)
        n = 64 if rr else 256

        def batch(i):
            if rr:
                L = 32 + 448 + 3
                ids = torch.randint(1000, 30000, (64, L), generator=torch.Generator().manual_seed(1000 * rank + i))
                typ = torch.zeros_like(ids)
                typ[:, 34:] = 1
                return ids.pin_memory(), torch.ones_like(ids).pin_memory(), typ.pin_memory()
            return padded_batch(256, 32, 512, 1000 * rank + i, dev) + (None,)

        bs = [batch(i) for i in range(W + 2 * K)]

        def step(b, to_host):
            ids, mask = b[0].to(dev, non_blocking=True), b[1].to(dev, non_blocking=True)
            with torch.no_grad():
                r = model.score(ids, mask, b[2].to(dev, non_blocking=True)) if rr else model.embed(ids, mask)
                if world > 1 and not rr:
                    g = torch.empty((world * r.shape[0], r.shape[1]), device=dev, dtype=r.dtype)
                    dist.all_gather_into_tensor(g, r.contiguous())
                    r = g
            return r.cpu() if to_host else r

        for b in bs[:W]:
            step(b, False)
        torch.cuda.synchronize()
        tb = datetime.datetime.now()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for b in bs[W:W + K]:
            step(b, False)
        e1.record()
        torch.cuda.synchronize()
        ms = mx(e0.elapsed_time(e1))
        t1 = time.perf_counter()
        d2h = 0
        for b in bs[W + K:]:
            r = step(b, True)
            d2h += r.numel() * r.element_size()
        e2e = mx(time.perf_counter() - t1)
        tot = n * K * world
        unit = "pairs/s" if rr else "docs/s"
        out.update({"metric": "rerank pairs/s" if rr else "embed docs/s", "value": round(tot / (ms / 1e3), 1), "unit": unit,
                    "ms_per_step": round(ms / K, 4), "scaling": "weak", "dtype": "bf16",
                    "data": "synthetic: uniform token ids, random-init",
                    "config": {"model": "BERT-base", "global_batch": n * world, "seq_len": "padded to the batch maximum",
                               "parallelism": f"dp{world} (NCCL all-gather)", "l2": "activations per batch exceed L2"},
                    "e2e": {"value": round(tot / e2e, 1), "unit": unit,
                            "h2d_bytes_per_step": int(sum(t.numel() * 8 for t in bs[0] if t is not None)),
                            "d2h_bytes_per_step": int(d2h / K)}})
    else:  # knn
        rows, dim, nq, k = args.knn_rows, 768, 1024, 100
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        db = F.normalize(torch.randn(rows, dim, generator=g, device=dev), dim=-1).bfloat16()
        q = F.normalize(torch.randn(nq, dim, generator=torch.Generator(device=dev).manual_seed(3), device=dev), dim=-1).bfloat16()
        for _ in range(W):
            knn_search(db, q, k, rank * rows, world)
        torch.cuda.synchronize()
        tb = datetime.datetime.now()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            knn_search(db, q, k, rank * rows, world)
        e1.record()
        torch.cuda.synchronize()
        ms = mx(e0.elapsed_time(e1))
        qh = q.cpu().pin_memory()
        t1 = time.perf_counter()
        for _ in range(K):
            v, i = knn_search(db, qh.to(dev, non_blocking=True), k, rank * rows, world)
            i.cpu()
        e2e = mx(time.perf_counter() - t1)
        out.update({"metric": "kNN queries/s at recall@10>=0.95", "value": round(nq * K / (ms / 1e3), 1), "unit": "queries/s",
                    "ms_per_step": round(ms / K, 4), "scaling": "weak", "dtype": "bf16",
                    "data": "synthetic: unit-normalised Gaussian rows",
                    "config": {"model": "exact cosine top-100", "global_batch": nq, "seq_len": dim,
                               "database_rows": rows * world, "parallelism": f"{world} shards (NCCL all-gather merge)",
                               "l2": "the database shard far exceeds L2"},
                    "e2e": {"value": round(nq * K / e2e, 1), "unit": "queries/s", "h2d_bytes_per_step": nq * dim * 2,
                            "d2h_bytes_per_step": nq * k * 8}})
    out["clocks"] = clock_summary(clocks, tb, datetime.datetime.now())
    out["gpu_launches"] = 0  # library kernels only: none of them is this repository's
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0
