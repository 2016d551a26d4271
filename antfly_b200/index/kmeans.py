"""Lloyd k-means on the GPU.

Rules kept from the reference (zig/lib/vectorindex/src/kmeans.zig:71-142, 179-296; zig/KMEANS.md:7-13):
deterministic farthest-first seeding from ``first_index`` (for large K a strided sample is used instead, the
farthest-first scan being O(N K) sequential), centroids re-normalised for cosine, at most ``max_iter`` (16)
iterations, stop when the summed squared centroid shift is <= 1e-6, an empty cluster keeps its old centroid,
results can be returned sorted by (cluster, distance).

Assignment is one persistent tcgen05 GEMM with an arg-min epilogue (``||c||^2 - 2 x.c``, or ``-x.c`` for
inner-product / cosine); the update is a vectorised atomic accumulation plus a finalise kernel.  With several
ranks each holds a shard of the points and the per-cluster sums and counts are all-reduced between the two.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import index_ops as IX


@dataclass
class KMeansResult:
    centroids: torch.Tensor      # [K, D] fp32
    assignments: torch.Tensor    # [N] int32
    distances: torch.Tensor      # [N] fp32 distance to the assigned centroid
    iterations: int
    shift: float


def _seed(x: torch.Tensor, k: int, first_index: int, metric: str, farthest_first_max_k: int = 256) -> torch.Tensor:
    n = x.shape[0]
    if k > farthest_first_max_k or k >= n:
        idx = (torch.arange(k, device=x.device) * max(n // max(k, 1), 1) + first_index) % n
        return x[idx].float()
    xf = x.float()
    chosen = [first_index % n]
    d = (xf - xf[chosen[0]]).pow(2).sum(-1)
    for _ in range(1, k):
        nxt = int(torch.argmax(d))
        chosen.append(nxt)
        d = torch.minimum(d, (xf - xf[nxt]).pow(2).sum(-1))
    return xf[torch.tensor(chosen, device=x.device)]


def kmeans(x: torch.Tensor, k: int, metric: str = "l2_squared", max_iter: int = 16, tol: float = 1e-6,
           first_index: int = 0, init: Optional[torch.Tensor] = None, all_reduce=None,
           chunk: int = 1 << 22) -> KMeansResult:
    """x: [N, D] bf16 (this rank's shard).  ``all_reduce(tensor)`` sums a tensor over ranks in place."""
    dev = x.device
    n, dim = x.shape
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    normalize = metric == "cosine"
    cent = (init.float().clone() if init is not None else _seed(xb, k, first_index, metric)).to(dev)
    if normalize:
        cent = torch.nn.functional.normalize(cent, dim=-1)
    cent = cent.contiguous()
    cent_b = cent.to(torch.bfloat16).contiguous()
    sq = cent_b.float().pow(2).sum(-1).contiguous()
    l2 = metric == "l2_squared"
    assign = torch.empty((n,), dtype=torch.int32, device=dev)
    best = torch.empty((n,), dtype=torch.float32, device=dev)
    sums = torch.zeros((k, dim), dtype=torch.float32, device=dev)
    counts = torch.zeros((k,), dtype=torch.int32, device=dev)
    shift = torch.zeros((1,), dtype=torch.float32, device=dev)
    xn = IX.row_sqnorm(xb) if l2 else None
    it, sh = 0, float("inf")

    def assign_all():
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            a, b = IX.assign_argmin(xb[lo:hi], cent_b, sq if l2 else None, -2.0 if l2 else -1.0,
                                    row_term=xn[lo:hi] if l2 else None)
            assign[lo:hi] = a
            best[lo:hi] = b

    for it in range(1, max_iter + 1):
        assign_all()
        sums.zero_(); counts.zero_(); shift.zero_()
        IX.kmeans_accumulate(xb, assign, sums, counts)
        if all_reduce is not None:
            all_reduce(sums); all_reduce(counts)
        IX.kmeans_finalize(sums, counts, cent, cent_b, sq, shift, normalize)
        sh = float(shift.item())
        if sh <= tol:
            break
    assign_all()
    if l2:
        best.clamp_(min=0)
    elif metric == "cosine":
        best.add_(1.0)
    return KMeansResult(cent, assign, best, it, sh)


def sorted_by_cluster(res: KMeansResult):
    """Point order sorted by (cluster, distance) and the cluster offsets [K+1] (posting lists)."""
    k = res.centroids.shape[0]
    key = res.assignments.long() * 4 + 0  # stable two-key sort: first by distance, then stably by cluster
    order = torch.argsort(res.distances, stable=True)
    order = order[torch.argsort(res.assignments[order].long(), stable=True)]
    counts = torch.bincount(res.assignments.long(), minlength=k)
    offsets = torch.zeros(k + 1, dtype=torch.int64, device=counts.device)
    offsets[1:] = torch.cumsum(counts, 0)
    return order, offsets
