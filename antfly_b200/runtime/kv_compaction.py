"""KV-cache compaction by attention matching: keep the keys that carry the attention mass and re-fit their values
so that attention over the small cache reproduces attention over the full one.

Per KV head (reference: zig/pkg/inference/src/runtime/kv/compaction.zig:14-26, after "Fast KV Compaction via
Attention Matching"):

1. reference queries are drawn from the cached keys themselves (evenly spaced),
2. every key is scored by the total soft-max attention mass the reference queries give it,
3. the top M = ceil(N * ratio) keys are kept (in their original order; the most recent ``keep_recent`` tokens are
   always kept),
4. new values solve the ridge-regularised least squares  softmax(Q K_hat^T) V_hat ~= softmax(Q K^T) V
   through a Cholesky factorisation of the M x M normal matrix.

Keys are stored with their rotary embedding applied, so the surviving keys stay valid at their original positions;
the engine keeps counting logical positions for new tokens while attention runs over the shorter physical cache.
All of it is plain tensor algebra (it runs once per request, after prefill), on whatever device the cache lives on.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch


def compact_head(K: torch.Tensor, V: torch.Tensor, ratio: float, n_ref: int = 64, keep_recent: int = 0,
                 ridge: float = 1e-4) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """K, V: [N, D] fp32.  Returns (kept indices [M], K_hat [M, D], V_hat [M, D])."""
    N, D = K.shape
    M = max(1, min(N, int(math.ceil(N * ratio))))
    if M >= N:
        idx = torch.arange(N, device=K.device)
        return idx, K.clone(), V.clone()
    scale = 1.0 / math.sqrt(D)
    n_ref = min(n_ref, N)
    ref_idx = torch.linspace(0, N - 1, n_ref, device=K.device).round().long()
    Q = K.index_select(0, ref_idx)                                   # [R, D]
    A = torch.softmax(Q @ K.T * scale, dim=-1)                       # [R, N]
    mass = A.sum(0)
    if keep_recent > 0:
        mass[-min(keep_recent, N):] = float("inf")
    idx = torch.topk(mass, M).indices.sort().values
    K_hat = K.index_select(0, idx)
    Y = A @ V                                                        # what full attention returns for the probes
    A_hat = torch.softmax(Q @ K_hat.T * scale, dim=-1)               # [R, M]
    # Least squares for the correction to the kept tokens' own values (so the ridge term pulls towards them):
    #   (A_hat^T A_hat + lambda I) dV = A_hat^T (Y - A_hat V_kept),   V_hat = V_kept + dV
    V_kept = V.index_select(0, idx)
    G = A_hat.T @ A_hat
    G = G + ridge * (G.diagonal().mean() + 1e-12) * torch.eye(M, device=K.device, dtype=K.dtype)
    dV = torch.cholesky_solve(A_hat.T @ (Y - A_hat @ V_kept), torch.linalg.cholesky(G))
    return idx, K_hat, V_kept + dV


def compact_layer(K: torch.Tensor, V: torch.Tensor, ratio: float, n_ref: int = 64, keep_recent: int = 0):
    """K, V: [N, Hkv, D] (any float dtype).  Every head keeps the same count M, its own choice of keys.
    Returns K_hat, V_hat [M, Hkv, D] fp32."""
    N, H, D = K.shape
    outs_k, outs_v = [], []
    for h in range(H):
        _, kh, vh = compact_head(K[:, h].float(), V[:, h].float(), ratio, n_ref, keep_recent)
        outs_k.append(kh)
        outs_v.append(vh)
    return torch.stack(outs_k, 1), torch.stack(outs_v, 1)


def attention_output(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
    """softmax(Q K^T / sqrt(D)) V for [*, D] operands (test helper and documentation of what is preserved)."""
    return torch.softmax(Q @ K.T / math.sqrt(K.shape[-1]), -1) @ V
