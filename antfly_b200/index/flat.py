"""Exact (brute-force) vector search on the GPU.

The database shard stays resident in HBM as bf16 rows (optionally block-scaled fp8 storage that is expanded to
bf16 a chunk at a time).  A query batch is scored by the persistent tcgen05 GEMM whose epilogue never writes the
score matrix: it only appends pairs that beat the query's current k-th best distance to a small candidate list.
The database is walked in geometrically growing chunks; after each chunk a select kernel merges the candidates
into the running top-k and tightens the thresholds, so the expected number of appended pairs per query per
chunk stays around k.  Results are exact (every true top-k pair beats every threshold it meets).

Replaces the reference's CPU exact scoring + heap (zig/lib/vector/src/vector.zig:267-500,
zig/lib/vectorindex/src/search_results.zig).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from ..ops import index_ops as IX
from ..ops import quant as Q
from ..ops import reference as R
from .distance import score_form


@dataclass
class SearchResult:
    distances: torch.Tensor  # [Q, k] ascending, +inf padded
    ids: torch.Tensor        # [Q, k] int32 (or int64 after id mapping), -1 padded
    # set by the searches that do not synchronise with the host: a device int32 [1] that is non-zero when a
    # candidate buffer overflowed and the result may miss neighbours (the caller repeats on the safe path)
    overflow: Optional[torch.Tensor] = None


class FlatIndex:
    def __init__(self, vectors: torch.Tensor, metric: str = "cosine", ids: Optional[torch.Tensor] = None,
                 storage: str = "bf16", id_offset: int = 0, device=None, keep_rerank_copy: bool = False):
        """vectors: [N, D] (any float dtype).  storage 'bf16' or 'fp8' (block-scaled e4m3 + e8m0 per 32).
        keep_rerank_copy: with fp8 storage also keep a bf16 copy in pinned host memory (or on the device when the
        input already lives there) used only to re-score the short list exactly."""
        self.metric = metric
        self.form = score_form(metric)
        dev = torch.device(device) if device is not None else vectors.device
        self.device = dev
        self.n, self.dim = vectors.shape
        self.id_offset = id_offset
        self.ids = ids.to(dev) if ids is not None else None
        self.storage = storage
        x = vectors.to(dev)
        if self.form.normalize:
            x = torch.nn.functional.normalize(x.float(), dim=-1)
        self.rerank_store = None
        if storage == "fp8" and keep_rerank_copy:
            self.rerank_store = x.to(torch.bfloat16).contiguous()
        if storage == "fp8":
            assert self.dim % 32 == 0, "fp8 storage needs a dimension that is a multiple of 32"
            q, e8 = R.quantize_block_fp8(x.float())
            self.q, self.e8 = q.contiguous(), e8.contiguous()
            self.x = None
            self.col_norm = None
            if self.form.use_col_norm:
                self.col_norm = R.dequantize_block_fp8(self.q, self.e8).pow(2).sum(-1)
        else:
            self.x = x.to(torch.bfloat16).contiguous()
            self.col_norm = IX.row_sqnorm(self.x) if self.form.use_col_norm else None
        self.seed_cols = 4096
        self.cand_cap = 4096

    def nbytes(self) -> int:
        if self.x is not None:
            return self.x.numel() * 2
        return self.q.numel() + self.e8.numel()

    def _rows(self, lo: int, hi: int) -> torch.Tensor:
        if self.x is not None:
            return self.x[lo:hi]
        # fp8 storage: expand the chunk to bf16 (exact: power-of-two scales).
        return R.dequantize_block_fp8(self.q[lo:hi], self.e8[:, lo:hi].contiguous()).to(torch.bfloat16)

    def prepare_queries(self, queries: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        q = queries.to(self.device)
        if self.form.normalize:
            q = torch.nn.functional.normalize(q.float(), dim=-1)
        qb = q.to(torch.bfloat16).contiguous()
        row = None
        if self.form.use_row_norm:
            row = IX.row_sqnorm(qb)
        elif self.form.row_const:
            row = torch.full((qb.shape[0],), self.form.row_const, dtype=torch.float32, device=self.device)
        return qb, row

    def search(self, queries: torch.Tensor, k: int, rerank_factor: int = 4) -> SearchResult:
        """Top-k; ids are row numbers + id_offset (or the user ids given at construction).  Exact for bf16
        storage; fp8 storage with a rerank copy fetches k * rerank_factor candidates and re-scores them."""
        if self.rerank_store is not None and rerank_factor > 1:
            return self._search_rerank(queries, k, rerank_factor)
        return self._search(queries, k)

    def _search_rerank(self, queries, k: int, factor: int) -> SearchResult:
        short = self._search(queries, min(self.n, k * factor), map_ids=False)
        rows = (short.ids - self.id_offset).clamp_min(0)
        nq, R_ = rows.shape
        cand = IX.gather_rows(self.rerank_store, rows.reshape(-1).contiguous()).view(nq, R_, self.dim).float()
        q = queries.to(self.device).float()
        if self.form.normalize:
            q = torch.nn.functional.normalize(q, dim=-1)
        dot = torch.einsum("qd,qrd->qr", q, cand)
        if self.metric == "l2_squared":
            d = (q.pow(2).sum(-1, keepdim=True) + cand.pow(2).sum(-1) - 2 * dot).clamp_min(0)
        elif self.metric == "inner_product":
            d = -dot
        else:
            d = 1 - dot
        d = torch.where(short.ids >= 0, d, torch.full_like(d, float("inf")))
        top_v, top_i, _, _ = IX.topk_select([(d.contiguous(), short.ids.contiguous(), None, R_)], nq, k, R_)
        return SearchResult(top_v, self._map_ids(top_i))

    def _map_ids(self, top_i: torch.Tensor) -> torch.Tensor:
        if self.ids is None:
            return top_i
        return torch.where(top_i >= 0, self.ids[(top_i - self.id_offset).clamp_min(0).long()],
                           torch.full_like(top_i, -1).to(self.ids.dtype))

    def search_nosync(self, queries: torch.Tensor, k: int) -> SearchResult:
        """As ``search`` on the fast path, without looking at the overflow flag on the host: the flag comes back in
        ``SearchResult.overflow`` for the caller to check when it reads the results anyway."""
        return self._search(queries, k, nosync=True)

    def _search(self, queries: torch.Tensor, k: int, map_ids: bool = True, push=None,
                safe: bool = False, nosync: bool = False) -> SearchResult:
        """push: peer targets of a sharded search (``MergeWorkspace.push_targets``); the select that ends the walk
        then also stores the result into every rank's merge buffer.  In that mode a candidate-buffer overflow is
        not repaired here: it travels with the pushed rows and the caller repeats the search with safe=True on
        all ranks."""
        qb, row = self.prepare_queries(queries)
        if push is not None:
            assert self.ids is None, "sharded search pushes row ids; user id maps are applied after the merge"
            map_ids = False
        if safe:
            return self._search_safe(qb, row, k, map_ids, push)
        nq = qb.shape[0]
        dev = self.device
        cap = max(self.cand_cap, 2 * k)
        cand_val = torch.empty((nq, cap), dtype=torch.float32, device=dev)
        cand_idx = torch.empty((nq, cap), dtype=torch.int32, device=dev)
        count = torch.zeros((nq,), dtype=torch.int32, device=dev)
        thr = torch.full((nq,), float("inf"), dtype=torch.float32, device=dev)
        top_v = torch.full((nq, k), float("inf"), dtype=torch.float32, device=dev)
        top_i = torch.full((nq, k), -1, dtype=torch.int32, device=dev)
        lo = 0
        chunk = min(self.n, min(self.seed_cols, cap))
        # One sticky overflow word for the whole walk (set by any chunk's select, never cleared).
        ovf = torch.zeros((1,), dtype=torch.int32, device=dev) if dev.type == "cuda" else None
        any_ovf = 0
        while lo < self.n:
            hi = min(self.n, lo + chunk)
            count.zero_()
            cn = self.col_norm[lo:hi] if self.col_norm is not None else None
            IX.score_filter(qb, self._rows(lo, hi), row, cn, self.form.scale, self.form.clamp_zero, thr, cand_val,
                            cand_idx, count, col_offset=lo + self.id_offset)
            top_v, top_i, thr, o = IX.topk_select([(top_v, top_i, None, k), (cand_val, cand_idx, count, cap)], nq, k,
                                                  k + cap, overflow=ovf, push=push if hi == self.n else None)
            if isinstance(o, int):
                any_ovf |= o
            lo = hi
            chunk = max(chunk, lo)  # geometric growth: expected appends per query per chunk stay ~k
        if nosync:
            flag = ovf if ovf is not None else torch.tensor([any_ovf], dtype=torch.int32)
            return SearchResult(top_v, self._map_ids(top_i) if map_ids else top_i, overflow=flag)
        if push is None and (any_ovf or (ovf is not None and int(ovf))):
            return self._search_safe(qb, row, k, map_ids)
        return SearchResult(top_v, self._map_ids(top_i) if map_ids else top_i)

    def _search_safe(self, qb, row, k, map_ids: bool = True, push=None) -> SearchResult:
        """Fallback when a candidate buffer overflowed (adversarially ordered data): fixed small chunks whose
        full score set fits the buffer."""
        nq = qb.shape[0]
        dev = self.device
        cap = self.cand_cap
        cand_val = torch.empty((nq, cap), dtype=torch.float32, device=dev)
        cand_idx = torch.empty((nq, cap), dtype=torch.int32, device=dev)
        count = torch.zeros((nq,), dtype=torch.int32, device=dev)
        thr = torch.full((nq,), float("inf"), dtype=torch.float32, device=dev)
        top_v = torch.full((nq, k), float("inf"), dtype=torch.float32, device=dev)
        top_i = torch.full((nq, k), -1, dtype=torch.int32, device=dev)
        for lo in range(0, self.n, cap):
            hi = min(self.n, lo + cap)
            count.zero_()
            cn = self.col_norm[lo:hi] if self.col_norm is not None else None
            IX.score_filter(qb, self._rows(lo, hi), row, cn, self.form.scale, self.form.clamp_zero, thr, cand_val,
                            cand_idx, count, col_offset=lo + self.id_offset)
            top_v, top_i, thr, _ = IX.topk_select([(top_v, top_i, None, k), (cand_val, cand_idx, count, cap)], nq, k,
                                                  k + cap, push=push if hi == self.n else None)
        return SearchResult(top_v, self._map_ids(top_i) if map_ids else top_i)


def exact_search_fp32(queries: torch.Tensor, vectors: torch.Tensor, k: int, metric: str) -> SearchResult:
    """fp32 oracle (the recall ground truth)."""
    d = R.distances(queries, vectors, metric)
    v, i = torch.topk(d, min(k, vectors.shape[0]), dim=-1, largest=False)
    return SearchResult(v, i.int())


def recall_at_k(found: torch.Tensor, truth: torch.Tensor, k: int) -> float:
    f, t = found[:, :k].cpu().tolist(), truth[:, :k].cpu().tolist()
    hit = sum(len(set(a) & set(b)) for a, b in zip(f, t))
    return hit / (len(t) * k)


class GrowableFlatIndex:
    """Exact index that accepts new vectors: rows are appended to a staging list and the searchable
    :class:`FlatIndex` is rebuilt on the first search after a change (a re-upload of the bf16 matrix; exact search
    has no structure to maintain).  Re-adding an id replaces its vector."""

    def __init__(self, dim: int, metric: str = "cosine", device=None, storage: str = "bf16"):
        self.dim, self.metric, self.device, self.storage = dim, metric, device, storage
        self._rows: List[torch.Tensor] = []
        self._ids: List[int] = []
        self._pos: dict = {}
        self._index: Optional[FlatIndex] = None

    def __len__(self) -> int:
        return len(self._ids)

    def add(self, vectors: torch.Tensor, ids: torch.Tensor) -> None:
        assert vectors.shape[1] == self.dim
        for v, i in zip(vectors.float().cpu(), ids.tolist()):
            if i in self._pos:
                self._rows[self._pos[i]] = v
            else:
                self._pos[i] = len(self._ids)
                self._ids.append(int(i))
                self._rows.append(v)
        self._index = None

    def search(self, queries: torch.Tensor, k: int, **_kw) -> SearchResult:
        if not self._ids:
            q = queries.shape[0]
            return SearchResult(torch.full((q, k), float("inf")), torch.full((q, k), -1, dtype=torch.int64))
        if self._index is None:
            self._index = FlatIndex(torch.stack(self._rows), self.metric, ids=torch.tensor(self._ids),
                                    storage=self.storage, device=self.device)
        return self._index.search(queries, min(k, len(self._ids)))
