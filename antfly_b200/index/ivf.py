"""IVF index: k-means centroids + posting lists, probed nprobe lists per query.

The counterpart of the reference's flat centroid directory mode (``centroid_directory_mode = flat_rabitq``:
score all leaf centroids, take the top probe_count postings, score their members, exact re-rank;
zig/lib/vectorindex/src/hbc_index.zig:1720-1775, spfresh_index.zig:200-390).  On the GPU the centroid scan is
one filter GEMM + select, and member scoring runs list-major: vectors are stored sorted by list, each probed list
is scored once against the (few) queries that probe it, and candidates go through the same threshold-filter /
select machinery as the flat index.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import index_ops as IX
from .distance import score_form
from .flat import FlatIndex, SearchResult
from .kmeans import kmeans, sorted_by_cluster


class IVFIndex:
    def __init__(self, vectors: torch.Tensor, n_lists: int, metric: str = "cosine", max_iter: int = 16,
                 train_sample: int = 0, id_offset: int = 0, seed: int = 0, all_reduce=None,
                 init_centroids: Optional[torch.Tensor] = None):
        """``all_reduce`` + ``init_centroids`` train one set of centroids jointly over the shards of several ranks:
        every rank must start from the same ``init_centroids`` (then every rank's centroids, and so its stopping
        decision, stay identical from the first update on)."""
        dev = vectors.device
        self.metric, self.form = metric, score_form(metric)
        self.id_offset = id_offset
        x = vectors
        if self.form.normalize:
            x = torch.nn.functional.normalize(x.float(), dim=-1)
        xb = x.to(torch.bfloat16).contiguous()
        n = xb.shape[0]
        train = xb
        if train_sample and train_sample < n:
            g = torch.Generator(device=dev).manual_seed(seed)
            train = xb[torch.randperm(n, generator=g, device=dev)[:train_sample]]
        km = kmeans(train, n_lists, metric=metric, max_iter=max_iter, all_reduce=all_reduce, init=init_centroids)
        if train is not xb:
            l2 = metric == "l2_squared"
            cb = km.centroids.to(torch.bfloat16)
            sq = cb.float().pow(2).sum(-1)
            a, b = IX.assign_argmin(xb, cb, sq if l2 else None, -2.0 if l2 else -1.0,
                                    row_term=IX.row_sqnorm(xb) if l2 else None)
            km.assignments, km.distances = a, b
        order, offsets = sorted_by_cluster(km)
        self.centroids = km.centroids
        self.order = order.int()                  # sorted position -> original row
        self.offsets = offsets                    # [L+1]
        self.x = xb[order]                        # vectors sorted by list
        self.col_norm = IX.row_sqnorm(self.x) if self.form.use_col_norm else None
        self.n_lists, self.n, self.dim = n_lists, n, xb.shape[1]
        self.centroid_index = FlatIndex(self.centroids, metric=metric)
        self.list_sizes = (offsets[1:] - offsets[:-1])
        self.offsets_dev = offsets.to(dev).long().contiguous()
        self.max_list_len = int(self.list_sizes.max()) if n_lists > 0 else 0
        self.kmeans_iterations = km.iterations

    # Candidate capacity of the thresholded pass, and the largest list the seed pass can take whole (the select
    # kernel sorts at most 16384 candidates per query in shared memory).
    cand_cap = 4096
    max_seed_list = 16384 - 512

    def _pairs(self, probes: torch.Tensor):
        """(query, list) pairs of a [Q, P] probe table, sorted by list, as fixed-shape device arrays: pair_query
        [Q * P] and pair_off [n_lists + 1].  Unused probe slots (-1) sort behind the last list.  No host sync."""
        nq, P = probes.shape
        dev = probes.device
        pl = probes.reshape(-1).long()
        pl = torch.where(pl >= 0, pl, torch.full_like(pl, self.n_lists))
        pq = torch.arange(nq, device=dev, dtype=torch.int32)[:, None].expand(nq, P).reshape(-1)
        pl_sorted, order = torch.sort(pl, stable=True)
        pair_query = pq[order].contiguous()
        pair_off = torch.searchsorted(pl_sorted, torch.arange(self.n_lists + 1, device=dev)).int()
        return pair_query, pair_off

    def search(self, queries: torch.Tensor, k: int, nprobe: int = 64, check: bool = True, push=None) -> SearchResult:
        """Top-k over the ``nprobe`` nearest lists of every query.  A fixed launch sequence with no host
        synchronisation inside: centroid scan (filter GEMM + select), pair sort, a seed list-scan of every query's
        nearest list (all members -> first top-k and a threshold), one thresholded list-scan over all other probed
        lists, a final select.  ``check=True`` reads the overflow flag afterwards and repeats on the host-driven
        path if a candidate buffer overflowed; ``check=False`` leaves the flag in ``SearchResult.overflow``.
        ``push``: peer targets of a sharded search (the final select also pushes, see index/sharded.py)."""
        nprobe = min(nprobe, self.n_lists)
        if self.max_list_len > self.max_seed_list or self.max_list_len + k > 16384:
            return self._search_host(queries, k, nprobe, push=push)
        dev = self.x.device
        cres = self.centroid_index.search_nosync(queries, nprobe)
        probes = cres.ids                                                      # [Q, nprobe]
        qb, row = self.centroid_index.prepare_queries(queries)
        nq = qb.shape[0]
        ovf = cres.overflow.to(dev) if cres.overflow is not None else torch.zeros(1, dtype=torch.int32, device=dev)
        ovf = ovf.clone()
        list_off = self.offsets_dev
        # seed: every query's nearest list, all members
        cap0 = max(16, self.max_list_len)
        cv = torch.empty((nq, cap0), dtype=torch.float32, device=dev)
        ci = torch.empty((nq, cap0), dtype=torch.int32, device=dev)
        cc = torch.zeros((nq,), dtype=torch.int32, device=dev)
        pq0, po0 = self._pairs(probes[:, :1])
        IX.ivf_scan(self.x, self.col_norm, qb, row, None, list_off, po0, pq0, cv, ci, cc, self.form.scale,
                    self.form.clamp_zero)
        last = nprobe == 1
        top_v, top_i, thr, _ = IX.topk_select([(cv, ci, cc, cap0)], nq, k, cap0, overflow=ovf,
                                              push=push if last else None)
        if not last:
            cap = self.cand_cap
            cv = torch.empty((nq, cap), dtype=torch.float32, device=dev)
            ci = torch.empty((nq, cap), dtype=torch.int32, device=dev)
            cc = torch.zeros((nq,), dtype=torch.int32, device=dev)
            pq1, po1 = self._pairs(probes[:, 1:])
            IX.ivf_scan(self.x, self.col_norm, qb, row, thr, list_off, po1, pq1, cv, ci, cc, self.form.scale,
                        self.form.clamp_zero)
            top_v, top_i, thr, _ = IX.topk_select([(top_v, top_i, None, k), (cv, ci, cc, cap)], nq, k, k + cap,
                                                  overflow=ovf, push=push)
        if push is not None:
            return SearchResult(top_v, top_i, overflow=ovf)     # sorted-row ids; the sharded caller maps them
        if check and int(ovf):
            return self._search_host(queries, k, nprobe)
        return SearchResult(top_v, self._ids_of(top_i), overflow=None if check else ovf)

    def _ids_of(self, top_i: torch.Tensor) -> torch.Tensor:
        return torch.where(top_i >= 0, self.order[top_i.clamp_min(0).long()] + self.id_offset,
                           torch.full_like(top_i, -1))

    def _search_host(self, queries: torch.Tensor, k: int, nprobe: int = 64, push=None) -> SearchResult:
        """Host-driven walk over the probed lists in bounded spans (each span's scores fit the candidate buffer, so
        nothing can overflow): the safe path behind ``search``, and the path for indexes with very long lists."""
        dev = self.x.device
        probes = self.centroid_index.search(queries, min(nprobe, self.n_lists)).ids  # [Q, nprobe]
        qb, row = self.centroid_index.prepare_queries(queries)
        nq = qb.shape[0]
        # (list, query) pairs grouped by list: every probed list is scored once.
        pq = torch.arange(nq, device=dev, dtype=torch.int64)[:, None].expand_as(probes).reshape(-1)
        pl = probes.reshape(-1).long()
        keep = pl >= 0
        pq, pl = pq[keep], pl[keep]
        order = torch.argsort(pl, stable=True)
        pq, pl = pq[order], pl[order]
        lists, starts = torch.unique_consecutive(pl, return_counts=True)
        ends = torch.cumsum(starts, 0)
        begins = ends - starts
        cap = 4096
        top_v = torch.full((nq, k), float("inf"), device=dev)
        top_i = torch.full((nq, k), -1, dtype=torch.int32, device=dev)
        thr = torch.full((nq,), float("inf"), device=dev)
        # Group lists into segments so that one filter launch covers a contiguous span of sorted vectors and a
        # gathered subset of queries; spans are bounded so candidate buffers cannot overflow before a select.
        lists_h, b_h, e_h = lists.tolist(), begins.tolist(), ends.tolist()
        off_h = self.offsets.tolist()
        for li, b, e in zip(lists_h, b_h, e_h):
            lo, hi = off_h[li], off_h[li + 1]
            if hi <= lo:
                continue
            qsel = pq[b:e]
            for s in range(lo, hi, cap):
                t = min(hi, s + cap)
                sub_q = qb[qsel]
                sub_row = row[qsel] if row is not None else None
                cv = torch.empty((qsel.numel(), cap), device=dev)
                ci = torch.empty((qsel.numel(), cap), dtype=torch.int32, device=dev)
                cc = torch.zeros((qsel.numel(),), dtype=torch.int32, device=dev)
                IX.score_filter(sub_q, self.x[s:t], sub_row, self.col_norm[s:t] if self.col_norm is not None else None,
                                self.form.scale, self.form.clamp_zero, thr[qsel].contiguous(), cv, ci, cc, col_offset=s)
                v, i, th, _ = IX.topk_select([(top_v[qsel].contiguous(), top_i[qsel].contiguous(), None, k),
                                              (cv, ci, cc, cap)], qsel.numel(), k, k + cap)
                top_v[qsel], top_i[qsel], thr[qsel] = v, i, th
        if push is not None:
            top_v, top_i, _, _ = IX.topk_select([(top_v.contiguous(), top_i.contiguous(), None, k)], nq, k, k, push=push)
            return SearchResult(top_v, top_i)
        return SearchResult(top_v, self._ids_of(top_i))
