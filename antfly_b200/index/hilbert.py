"""Hilbert-curve ordering of vectors and the random orthogonal transform.

``hilbert_keys`` gives every vector a byte key that sorts in Hilbert-curve order (C++: ``csrc/host/hilbert.cpp``;
the reference's ``Hilbert`` encoder, zig/lib/vector/src/vector.zig:42-140); ``hilbert_order`` is the permutation that
sorts by it -- contiguous runs of the sorted order are spatially compact, which is what the Hilbert bulk build of
the HBC tree cuts into leaves.  ``random_orthogonal`` is a seeded rotation (QR of a Gaussian matrix, sign-fixed) used
to decorrelate dimensions before 1-bit quantisation (the reference's rand_ortho transform,
go/pkg/antfly/lib/vector/rand_ortho.go)."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _native as N


def hilbert_keys(vectors: torch.Tensor) -> np.ndarray:
    """[n, dims] float -> uint8 [n, 4 * dims] keys (lexicographic order = curve order)."""
    v = np.ascontiguousarray(vectors.detach().float().cpu().numpy())
    n, d = v.shape
    keys = np.empty((n, 4 * d), dtype=np.uint8)
    rc = N.host().afb_hilbert_keys(v.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(n), ctypes.c_int(d),
                                   keys.ctypes.data_as(ctypes.c_void_p))
    assert rc == 0
    return keys


def hilbert_order(vectors: torch.Tensor) -> torch.Tensor:
    """Permutation (int64 [n]) that sorts the vectors along the Hilbert curve."""
    keys = hilbert_keys(vectors)
    # lexicographic sort of byte rows: view each row as one fixed-width bytes object
    as_void = keys.view(np.dtype((np.void, keys.shape[1]))).reshape(-1)
    return torch.from_numpy(np.argsort(as_void, kind="stable").astype(np.int64))


def random_orthogonal(dims: int, seed: int = 42, dtype=torch.float32) -> torch.Tensor:
    """A dims x dims orthogonal matrix drawn from the Haar measure, reproducible from ``seed``."""
    g = torch.Generator().manual_seed(seed)
    q, r = torch.linalg.qr(torch.randn(dims, dims, generator=g, dtype=torch.float64))
    q = q * torch.sign(torch.diagonal(r))[None]  # fix the sign ambiguity of the factorisation
    return q.to(dtype)
