"""Score distortion of the quantised KV-cache key codecs: how far q.k computed against the codes is from the exact
dot product.

The reference ships this as a standalone bench (zig/pkg/inference/src/bench/turboquant_distortion.zig: uniform
[-1, 1) keys and queries from a splitmix64 stream, MAE / RMSE / max error of the polar4 and turbo3 scores, and a sweep
of the multiplier of the turbo3 residual-sketch correction that reports the scale with the lowest RMSE).  This one
covers every key codec of :mod:`antfly_b200.ops.kv_quant`, uses the same sample stream, and runs anywhere: the
encoders are the tensor-op ones, so ``--device cuda`` measures the bytes the GPU cache would hold.

    python -m antfly_b200.utils.kv_distortion --samples 4096 --num-kv-heads 8 --head-dim 128
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List

import numpy as np
import torch

from ..ops import kv_quant as KQ

_M64 = (1 << 64) - 1


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def sample_values(samples: np.ndarray, n: int, seed: int) -> np.ndarray:
    """[len(samples), n] floats in [-1, 1): value i of sample s is a 24-bit fraction of
    splitmix64(seed ^ (s + 1) * a ^ (i + 1) * b)."""
    with np.errstate(over="ignore"):
        s = (samples.astype(np.uint64) + np.uint64(1))[:, None] * np.uint64(0x9E3779B97F4A7C15)
        i = (np.arange(n, dtype=np.uint64) + np.uint64(1))[None, :] * np.uint64(0xBF58476D1CE4E5B9)
        mixed = _splitmix64(np.uint64(seed) ^ s ^ i)
    u = (mixed >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)
    return u * 2.0 - 1.0


def _metrics(exact: torch.Tensor, est: torch.Tensor) -> Dict[str, float]:
    diff = (exact.double() - est.double()).abs()
    return {"mae": float(diff.mean()), "rmse": float(diff.pow(2).mean().sqrt()), "max_abs": float(diff.max())}


def sketch_signs(rows: torch.Tensor, heads: int, D: int) -> torch.Tensor:
    """The residual sketch of turbo3 key rows as [T, heads, 32] of +-1 (the bits follow the 3-bit base codes)."""
    base = (heads * D * 3 + 7) // 8
    sk = rows[:, base:].to(torch.int32)
    bits = (sk[..., None] >> torch.arange(8, device=rows.device)) & 1
    bits = bits.reshape(rows.shape[0], -1)[:, : heads * KQ.SKETCH_BITS]
    return (bits.view(-1, heads, KQ.SKETCH_BITS) * 2 - 1).float()


def measure(samples: int = 4096, heads: int = 8, D: int = 128, codecs=("fp8", "int8", "int4", "polar4", "turbo3"),
            scale_min: float = -2.0, scale_max: float = 2.0, scale_step: float = 0.125, device: str = "cpu",
            block: int = 1024) -> Dict[str, object]:
    """Per codec: MAE / RMSE / max error of the head-wise scores over ``samples`` keys x ``heads`` queries.  For
    turbo3 the base (3-bit only) error, the error with the built-in correction, and the sweep over multipliers of
    the unit correction (mean of sign x query projection) with its best scale."""
    if samples <= 0 or heads <= 0:
        raise ValueError("samples and heads must be positive")
    if scale_step <= 0 or scale_max < scale_min:
        raise ValueError("bad scale sweep")
    for c in codecs:
        KQ.row_bytes(c, heads, D)
    scales = np.arange(scale_min, scale_max + 1e-5, scale_step, dtype=np.float64)
    exact_all, est = [], {c: [] for c in codecs}
    unit_all, base_all = [], []
    for s0 in range(0, samples, block):
        ids = np.arange(s0, min(samples, s0 + block))
        key = torch.from_numpy(sample_values(ids, heads * D, 0x1234ABCD)).view(-1, heads, D).to(device)
        q = torch.stack([torch.from_numpy(sample_values(ids + h * 131, D, 0xFEEDFACE)) for h in range(heads)], 1)
        q = q.to(device)
        exact_all.append((q * key).sum(-1).cpu())
        for c in codecs:
            rows = KQ.encode_rows_torch(c, key)
            dec = KQ.decode_rows(c, rows.cpu(), heads, D).to(device)
            score = (q * dec).sum(-1)
            if c == "turbo3":
                pq = torch.einsum("thd,hpd->thp", q, KQ.random_signs(heads, D, device))
                unit = (sketch_signs(rows, heads, D) * pq).mean(-1)
                base_all.append(score.cpu())
                unit_all.append(unit.cpu())
                score = score + KQ.RESIDUAL_SCALE * unit
            est[c].append(score.cpu())
    exact = torch.cat(exact_all)
    out: Dict[str, object] = {"samples": samples, "num_kv_heads": heads, "head_dim": D, "dots": int(exact.numel()),
                              "codecs": {}}
    for c in codecs:
        out["codecs"][c] = dict(_metrics(exact, torch.cat(est[c])), key_bytes_per_token=KQ.row_bytes(c, heads, D))
    if "turbo3" in codecs:
        base, unit = torch.cat(base_all), torch.cat(unit_all)
        sweep: List[Dict[str, float]] = []
        for sc in scales:
            sweep.append(dict(_metrics(exact, base + float(sc) * unit), scale=float(sc)))
        best = min(sweep, key=lambda r: r["rmse"])
        out["turbo3_base"] = _metrics(exact, base)
        out["turbo3_residual_best"] = best
        out["turbo3_residual_builtin_scale"] = KQ.RESIDUAL_SCALE
        out["scale_sweep"] = sweep
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--samples", type=int, default=4096)
    ap.add_argument("--num-kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--scale-min", type=float, default=-2.0)
    ap.add_argument("--scale-max", type=float, default=2.0)
    ap.add_argument("--scale-step", type=float, default=0.125)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--sweep", action="store_true", help="print every row of the scale sweep")
    args = ap.parse_args(argv)
    rep = measure(args.samples, args.num_kv_heads, args.head_dim, scale_min=args.scale_min,
                  scale_max=args.scale_max, scale_step=args.scale_step, device=args.device)
    if not args.sweep:
        rep.pop("scale_sweep", None)
    print(json.dumps(rep))


if __name__ == "__main__":
    main()
