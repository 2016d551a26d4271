"""HBC: hierarchical balanced clustering tree with RaBitQ-quantised nodes and exact re-ranking.

A compact restatement of the reference's main vector index (zig/lib/vectorindex/src/hbc_index.zig, hbc.zig,
search.zig; defaults zig/lib/vectorindex/src/types.zig:44-77): leaves hold up to ``leaf_size`` vectors, internal
nodes up to ``branching_factor`` children, the tree is bulk-built bottom-up with k-means (K ~ N / leaf_size per
level, parents clustered by branching factor), every node's members are RaBitQ-quantised once against the node
centroid, search is a best-first beam over a priority queue of (estimated distance - error bound) that stops after
``search_width`` leaves, skips subtrees whose lower bound exceeds ``d_min * (1 + epsilon)`` once the result set is
full (not for inner-product), and re-ranks ``k * ceil(1 + epsilon)`` candidates with exact distances.  On-disk
layout (four key namespaces, 50-byte metadata record, ``HBN1`` packed nodes) is implemented in
:mod:`antfly_b200.index.artifact`.
"""
from __future__ import annotations

import heapq
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import reference as R
from .kmeans import kmeans
from .rabitq import RaBitQSet, RaBitQuantizer


@dataclass
class HBCConfig:
    dims: int
    metric: str = "l2_squared"
    branching_factor: int = 16
    leaf_size: int = 100
    search_width: int = 32
    epsilon: float = 0.1
    kmeans_max_iter: int = 16
    use_quantization: bool = True
    quantizer_seed: int = 42
    # kmeans: cluster every level (farthest-first seeding); hilbert_seeded: k-means seeded with the means of
    # Hilbert-curve runs (the reference's default bulk build); hilbert: cut the curve order into runs, no clustering;
    # recursive: split the set in two with 2-means until the pieces fit a leaf (top-down)
    bulk_build: str = "kmeans"
    # hbc: beam search down the tree; flat_rabitq: score every leaf centroid with one quantised pass (blocks of
    # flat_centroid_block_size), open the best flat_centroid_probe_count leaves (0: the search width) -- IVF-style
    centroid_directory_mode: str = "hbc"
    flat_centroid_block_size: int = 8192
    flat_centroid_probe_count: int = 0
    merge_below: float = 0.25           # a leaf that shrinks below this fraction of leaf_size is merged away


@dataclass
class Node:
    id: int
    is_leaf: bool
    level: int
    parent: int
    centroid: torch.Tensor
    children: List[int] = field(default_factory=list)  # child node ids (internal) or vector ids (leaf)
    quant: Optional[RaBitQSet] = None


class HBCIndex:
    def __init__(self, cfg: HBCConfig):
        self.cfg = cfg
        self.nodes: Dict[int, Node] = {}
        self.root = 0
        self.vectors: Optional[torch.Tensor] = None  # [N, D] fp32 (exact re-rank store)
        self.ids: Optional[torch.Tensor] = None
        self.quantizer = RaBitQuantizer(cfg.dims, cfg.metric, cfg.quantizer_seed)
        self.leaf_of: Dict[int, int] = {}

    # -- build --------------------------------------------------------------------------------------------
    @classmethod
    def bulk_build(cls, vectors: torch.Tensor, cfg: HBCConfig, ids: Optional[torch.Tensor] = None) -> "HBCIndex":
        self = cls(cfg)
        x = vectors.float()
        if cfg.metric == "cosine":
            x = torch.nn.functional.normalize(x, dim=-1)
        self.vectors = x
        n = x.shape[0]
        self.ids = ids if ids is not None else torch.arange(n)
        next_id = [1]

        def new_node(is_leaf, level, centroid, children) -> Node:
            nd = Node(next_id[0], is_leaf, level, 0, centroid, children)
            next_id[0] += 1
            self.nodes[nd.id] = nd
            return nd

        # level 0: leaves
        k = max(1, math.ceil(n / cfg.leaf_size))
        members: List[torch.Tensor]
        if k == 1:
            cents = x.mean(0, keepdim=True)
            members = [torch.arange(n)]
        elif cfg.bulk_build in ("hilbert", "hilbert_seeded"):
            # Sort along the Hilbert curve and cut into leaf-sized runs (the reference's hilbert bulk builds,
            # zig/HBC.md).  "hilbert" keeps the runs as leaves: no clustering pass over the data, but a space-filling
            # curve preserves little locality in many dimensions, so leaves are loose.  "hilbert_seeded" uses the
            # runs' means as the starting centroids of the usual Lloyd iterations.
            from .hilbert import hilbert_order

            order = hilbert_order(x).to(x.device)
            members = [order[i:i + cfg.leaf_size] for i in range(0, n, cfg.leaf_size)]
            cents = torch.stack([x[m].mean(0) for m in members])
            if cfg.metric == "cosine":
                cents = torch.nn.functional.normalize(cents, dim=-1)
            if cfg.bulk_build == "hilbert_seeded":
                km = kmeans(x.to(torch.bfloat16), len(members), metric=cfg.metric, max_iter=cfg.kmeans_max_iter,
                            init=cents)
                cents = km.centroids.float().cpu() if not x.is_cuda else km.centroids.float()
                a = km.assignments.long()
                members = [torch.nonzero(a == c).flatten() for c in range(cents.shape[0])]
        elif cfg.bulk_build == "recursive":
            members, work = [], [torch.arange(n)]
            while work:
                m = work.pop()
                if m.numel() <= cfg.leaf_size:
                    members.append(m)
                    continue
                km = kmeans(x[m].to(torch.bfloat16), 2, metric=cfg.metric, max_iter=cfg.kmeans_max_iter)
                a = km.assignments.long()
                left, right = m[a == 0], m[a == 1]
                if left.numel() == 0 or right.numel() == 0:      # identical points: cut in the middle
                    left, right = m[: m.numel() // 2], m[m.numel() // 2:]
                work += [left, right]
            cents = torch.stack([x[m].mean(0) for m in members])
            if cfg.metric == "cosine":
                cents = torch.nn.functional.normalize(cents, dim=-1)
        else:
            km = kmeans(x.to(torch.bfloat16), k, metric=cfg.metric, max_iter=cfg.kmeans_max_iter)
            cents = km.centroids.float().cpu() if not x.is_cuda else km.centroids.float()
            a = km.assignments.long()
            members = [torch.nonzero(a == c).flatten() for c in range(k)]
        level_nodes: List[Node] = []
        for c, mem in enumerate(members):
            if mem.numel() == 0:
                continue
            nd = new_node(True, 0, cents[c].to(x.device), mem.tolist())
            for v in nd.children:
                self.leaf_of[v] = nd.id
            level_nodes.append(nd)
        level = 0
        while len(level_nodes) > 1:
            level += 1
            cm = torch.stack([nd.centroid for nd in level_nodes])
            kk = max(1, math.ceil(len(level_nodes) / cfg.branching_factor))
            if kk == 1:
                groups = [list(range(len(level_nodes)))]
                pc = cm.mean(0, keepdim=True)
            elif cfg.bulk_build == "hilbert":
                # leaves were created in curve order, so consecutive nodes are neighbours: group them in runs
                bf = cfg.branching_factor
                groups = [list(range(i, min(i + bf, len(level_nodes)))) for i in range(0, len(level_nodes), bf)]
                pc = torch.stack([cm[g].mean(0) for g in groups])
                if cfg.metric == "cosine":
                    pc = torch.nn.functional.normalize(pc, dim=-1)
            else:
                km = kmeans(cm.to(torch.bfloat16), kk, metric=cfg.metric, max_iter=cfg.kmeans_max_iter)
                a = km.assignments.long()
                groups = [torch.nonzero(a == c).flatten().tolist() for c in range(kk)]
                pc = km.centroids.float()
            parents = []
            for c, grp in enumerate(groups):
                if not grp:
                    continue
                p = new_node(False, level, pc[c].to(x.device), [level_nodes[i].id for i in grp])
                for i in grp:
                    level_nodes[i].parent = p.id
                parents.append(p)
            level_nodes = parents
        self.root = level_nodes[0].id
        if cfg.use_quantization:
            for nd in self.nodes.values():
                pts = x[torch.tensor(nd.children)] if nd.is_leaf else torch.stack(
                    [self.nodes[c].centroid for c in nd.children])
                nd.quant = self.quantizer.quantize(nd.centroid, pts)
        return self

    # -- search -------------------------------------------------------------------------------------------
    def _score(self, nd: Node, q: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if nd.quant is not None:
            return self.quantizer.estimate(nd.quant, q)
        pts = self.vectors[torch.tensor(nd.children)] if nd.is_leaf else torch.stack(
            [self.nodes[c].centroid for c in nd.children])
        d = R.distances(q[None], pts, self.cfg.metric)[0]
        return d, torch.zeros_like(d)

    def search(self, query: torch.Tensor, k: int, search_width: Optional[int] = None,
               epsilon: Optional[float] = None, profile: Optional[dict] = None) -> Tuple[List[int], List[float]]:
        """Beam search.  When ``profile`` is a dict it is filled with the per-query breakdown the reference's
        SearchProfile reports (zig/lib/vectorindex/src/hbc_index.zig:1652 searchProfiledRequest): nodes expanded,
        leaves scored, candidates kept, vectors re-ranked exactly, pruned queue pops, and nanoseconds spent scoring
        internal nodes, scoring leaves and re-ranking."""
        import time as _time

        t_start = _time.perf_counter_ns()
        prof = {"internal_nodes": 0, "leaves": 0, "pruned": 0, "candidates": 0, "reranked": 0,
                "internal_ns": 0, "leaf_ns": 0, "rerank_ns": 0, "total_ns": 0}
        cfg = self.cfg
        width = search_width or cfg.search_width
        eps = cfg.epsilon if epsilon is None else epsilon
        q = query.float().to(self.vectors.device)
        if cfg.metric == "cosine":
            q = torch.nn.functional.normalize(q, dim=-1)
        rerank_n = k * math.ceil(1 + eps)
        cap = min(max(4 * width, 2 * cfg.branching_factor, 1), 1024) * max(cfg.leaf_size, 1)
        pq: List[Tuple[float, int, int]] = [(0.0, 0, self.root)]
        cands: List[Tuple[float, int]] = []
        leaves, counter = 0, 1
        dmin = float("inf")
        if cfg.centroid_directory_mode == "flat_rabitq":
            # One quantised pass over every leaf centroid instead of walking the tree; the best leaves are then
            # opened in order by the loop below (internal nodes are never pushed).
            t0 = _time.perf_counter_ns()
            probe = cfg.flat_centroid_probe_count or width
            width = min(width, probe) if cfg.flat_centroid_probe_count else width
            leaf_ids, est = self._directory(q)
            top = torch.topk(est, min(probe, est.numel()), largest=False)
            pq = [(float(d), i, leaf_ids[j]) for i, (d, j) in enumerate(zip(top.values.tolist(), top.indices.tolist()))]
            heapq.heapify(pq)
            prof["internal_ns"] += _time.perf_counter_ns() - t0
            prof["internal_nodes"] = -(-len(leaf_ids) // cfg.flat_centroid_block_size)      # blocks scored
        while pq and leaves < width:
            bound, _, nid = heapq.heappop(pq)
            nd = self.nodes[nid]
            # Dynamic pruning compares like with like (zig/lib/vectorindex/src/search.zig:56-79): the bound of a
            # node's centroid against the smallest leaf-centroid bound met once enough candidates are held -- never
            # against a member distance, which a centroid distance does not bound from below.
            if cfg.metric != "inner_product" and len(cands) >= rerank_n:
                if nd.is_leaf and bound < dmin:
                    dmin = bound
                elif dmin < float("inf") and (abs(bound) > abs(dmin * (1 + eps)) if nd.is_leaf
                                              else bound > dmin * (1 + eps)):
                    prof["pruned"] += 1
                    continue
            t0 = _time.perf_counter_ns()
            d, e = self._score(nd, q)
            d, e = d.tolist(), e.tolist()
            prof["leaf_ns" if nd.is_leaf else "internal_ns"] += _time.perf_counter_ns() - t0
            prof["leaves" if nd.is_leaf else "internal_nodes"] += 1
            if nd.is_leaf:
                leaves += 1
                for vid, dist in zip(nd.children, d):
                    cands.append((dist, vid))
                if len(cands) > cap:
                    cands = heapq.nsmallest(cap, cands)
            else:
                for cid, dist, err in zip(nd.children, d, e):
                    heapq.heappush(pq, (dist - err, counter, cid))
                    counter += 1
        # Exact re-rank of the best estimated candidates, up to the reference's candidate capacity.
        capacity = min(max(4 * width, 2 * cfg.branching_factor, 1), 1024)
        short = [vid for _, vid in heapq.nsmallest(max(rerank_n, k, capacity), cands)]
        prof["candidates"], prof["reranked"] = len(cands), len(short)
        if not short:
            if profile is not None:
                prof["total_ns"] = _time.perf_counter_ns() - t_start
                profile.update(prof)
            return [], []
        t0 = _time.perf_counter_ns()
        exact = R.distances(q[None], self.vectors[torch.tensor(short)], cfg.metric)[0]
        order = torch.argsort(exact)[:k]
        out = [int(self.ids[short[i]]) for i in order.tolist()], exact[order].tolist()
        if profile is not None:
            prof["rerank_ns"] = _time.perf_counter_ns() - t0
            prof["total_ns"] = _time.perf_counter_ns() - t_start
            profile.update(prof)
        return out

    def _directory(self, q: torch.Tensor) -> Tuple[List[int], torch.Tensor]:
        """Flat directory of the leaf centroids: quantised once (lazily, rebuilt after inserts / deletes), scored
        for a query in blocks.  Returns (leaf node ids, estimated distance lower bounds)."""
        d = getattr(self, "_dir", None)
        if d is None:
            leaf_ids = [nd.id for nd in self.nodes.values() if nd.is_leaf and nd.children]
            blocks = []
            bs = self.cfg.flat_centroid_block_size
            for lo in range(0, len(leaf_ids), bs):
                cents = torch.stack([self.nodes[i].centroid for i in leaf_ids[lo:lo + bs]])
                mean = cents.mean(0)
                if self.cfg.metric == "cosine":
                    mean = torch.nn.functional.normalize(mean, dim=-1)
                blocks.append(self.quantizer.quantize(mean, cents) if self.cfg.use_quantization else cents)
            d = self._dir = (leaf_ids, blocks)
        leaf_ids, blocks = d
        est = []
        for b in blocks:
            if isinstance(b, RaBitQSet):
                d_, e_ = self.quantizer.estimate(b, q)
                est.append(d_ - e_)                      # lower bound, the beam's priority for internal nodes too
            else:
                est.append(R.distances(q[None], b, self.cfg.metric)[0])
        return leaf_ids, torch.cat(est) if est else torch.zeros(0)

    # -- online maintenance -------------------------------------------------------------------------------
    def _requantize(self, nd: Node) -> None:
        if not self.cfg.use_quantization:
            return
        pts = self.vectors[torch.tensor(nd.children)] if nd.is_leaf else torch.stack(
            [self.nodes[c].centroid for c in nd.children])
        nd.quant = self.quantizer.quantize(nd.centroid, pts)

    def _recentre(self, nd: Node) -> None:
        pts = self.vectors[torch.tensor(nd.children)] if nd.is_leaf else torch.stack(
            [self.nodes[c].centroid for c in nd.children])
        c = pts.mean(0)
        nd.centroid = torch.nn.functional.normalize(c, dim=-1) if self.cfg.metric == "cosine" else c

    def _new_node(self, is_leaf: bool, level: int, parent: int, children: List[int]) -> Node:
        nid = max(self.nodes) + 1
        nd = Node(nid, is_leaf, level, parent, torch.zeros(self.cfg.dims), children)
        self.nodes[nid] = nd
        return nd

    def _split(self, nd: Node) -> None:
        """Split an over-full node in two with 2-means over its members (SPFresh-style posting split); the new
        sibling joins the parent, which may split in turn; a split root grows the tree by one level."""
        pts = self.vectors[torch.tensor(nd.children)] if nd.is_leaf else torch.stack(
            [self.nodes[c].centroid for c in nd.children])
        km = kmeans(pts.to(torch.bfloat16), 2, metric=self.cfg.metric, max_iter=self.cfg.kmeans_max_iter)
        a = km.assignments.long().tolist()
        left = [c for c, g in zip(nd.children, a) if g == 0]
        right = [c for c, g in zip(nd.children, a) if g == 1]
        if not left or not right:  # degenerate (identical points): cut in the middle
            half = len(nd.children) // 2
            left, right = nd.children[:half], nd.children[half:]
        sib = self._new_node(nd.is_leaf, nd.level, nd.parent, right)
        nd.children = left
        for node in (nd, sib):
            if node.is_leaf:
                for v in node.children:
                    self.leaf_of[v] = node.id
            else:
                for c in node.children:
                    self.nodes[c].parent = node.id
            self._recentre(node)
            self._requantize(node)
        limit = 2 * (self.cfg.leaf_size if nd.is_leaf else self.cfg.branching_factor)
        self._attach_sibling(nd, sib)
        for node in (nd, sib):  # a large batch can leave a half that is still over-full
            if len(node.children) > limit:
                self._split(node)

    def _attach_sibling(self, nd: Node, sib: Node) -> None:
        if nd.id == self.root:
            root = self._new_node(False, nd.level + 1, 0, [nd.id, sib.id])
            nd.parent = sib.parent = root.id
            self.root = root.id
            self._recentre(root)
            self._requantize(root)
            return
        parent = self.nodes[nd.parent]
        parent.children.append(sib.id)
        self._recentre(parent)
        self._requantize(parent)
        if len(parent.children) > 2 * self.cfg.branching_factor:
            self._split(parent)

    def insert(self, vectors: torch.Tensor, ids: Optional[torch.Tensor] = None) -> None:
        """Online batch insert: every vector descends greedily to its nearest leaf (exact centroid distances),
        leaves that grow past twice the leaf size are split, splits propagate upwards.  Mirrors the reference's
        online insert path (zig/lib/vectorindex/src/hbc_index.zig, spfresh_index.zig)."""
        self._dir = None
        x = vectors.float().to(self.vectors.device)
        if self.cfg.metric == "cosine":
            x = torch.nn.functional.normalize(x, dim=-1)
        base = self.vectors.shape[0]
        self.vectors = torch.cat([self.vectors, x], 0)
        new_ids = ids if ids is not None else torch.arange(int(self.ids.max()) + 1, int(self.ids.max()) + 1 + x.shape[0])
        self.ids = torch.cat([self.ids, new_ids.to(self.ids.dtype)])
        touched = set()
        for i in range(x.shape[0]):
            nd = self.nodes[self.root]
            while not nd.is_leaf:
                cents = torch.stack([self.nodes[c].centroid for c in nd.children])
                nd = self.nodes[nd.children[int(torch.argmin(R.distances(x[i][None], cents, self.cfg.metric)[0]))]]
            nd.children.append(base + i)
            self.leaf_of[base + i] = nd.id
            touched.add(nd.id)
        for nid in sorted(touched):
            nd = self.nodes[nid]
            self._recentre(nd)
            if len(nd.children) > 2 * self.cfg.leaf_size:
                self._split(nd)
            else:
                self._requantize(nd)
                p = nd.parent
                if p in self.nodes:
                    self._requantize(self.nodes[p])  # the parent's payload encodes its children's centroids

    def delete(self, vector_ids: List[int]) -> int:
        """Remove vectors by external id from their leaves (leaves may become small; they are not merged).
        Returns how many were found."""
        pos = {int(v): i for i, v in enumerate(self.ids.tolist())}
        n, touched = 0, set()
        for vid in vector_ids:
            i = pos.get(int(vid))
            if i is None or i not in self.leaf_of:
                continue
            leaf = self.nodes[self.leaf_of.pop(i)]
            leaf.children.remove(i)
            touched.add(leaf.id)
            n += 1
        self._dir = None
        floor = self.cfg.merge_below * self.cfg.leaf_size
        for nid in touched:
            nd = self.nodes.get(nid)
            if nd is None:
                continue
            if len(nd.children) < floor and self._merge_leaf(nd):
                continue
            if nd.children:
                self._recentre(nd)
                self._requantize(nd)
            else:
                nd.quant = None
        return n

    def _merge_leaf(self, nd: Node) -> bool:
        """Fold an under-full leaf into its siblings (SPFresh-style posting merge): every remaining member moves to
        the sibling leaf with the nearest centroid, the leaf is removed from its parent, and a sibling that grows
        past twice the leaf size is split again.  Returns False when there is no sibling leaf to merge into."""
        parent = self.nodes.get(nd.parent)
        if parent is None:
            return False
        sibs = [self.nodes[c] for c in parent.children if c != nd.id and self.nodes[c].is_leaf]
        if not sibs:
            return False
        grew = set()
        if nd.children:
            cents = torch.stack([sb.centroid for sb in sibs])
            pts = self.vectors[torch.tensor(nd.children)]
            near = torch.argmin(R.distances(pts, cents, self.cfg.metric), dim=1).tolist()
            for v, j in zip(nd.children, near):
                sibs[j].children.append(v)
                self.leaf_of[v] = sibs[j].id
                grew.add(sibs[j].id)
        parent.children.remove(nd.id)
        del self.nodes[nd.id]
        for sid in grew:
            sb = self.nodes[sid]
            self._recentre(sb)
            if len(sb.children) > 2 * self.cfg.leaf_size:
                self._split(sb)
            else:
                self._requantize(sb)
        self._recentre(parent)
        self._requantize(parent)
        return True

    def stats(self) -> dict:
        leaves = sum(1 for n in self.nodes.values() if n.is_leaf)
        return {"nodes": len(self.nodes), "leaves": leaves, "levels": self.nodes[self.root].level + 1,
                "vectors": len(self.leaf_of)}          # vectors some leaf holds (deleted rows are not counted)
