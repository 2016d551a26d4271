"""A searchable table: documents with a dense vector index, a sparse (learned-term) index and a BM25 full-text
index, queried together.

One query may carry a dense vector (or text to embed), a sparse vector (or text to encode with a sparse model) and
full-text terms; each index returns its own ranking, the rankings are fused (reciprocal-rank or relative-score
fusion, or failover), pruned, optionally re-scored by a cross-encoder, and the documents are attached.  This is
the query path of the reference's table API condensed to one process (zig/pkg/antfly/src/api/query.zig,
storage/db/query/search_exec.zig:4348 per-shard dense search, search/fusion.zig:70-120 fusion and pruning,
reranking/mod.zig:26 rerank stage; request fields from specs/openapi/antfly/metadata.yaml:4077-4400).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Mapping, Optional, Sequence

import torch

from .fusion import FusedHit, MergeConfig, Pruner, fuse, prune
from .sparse import FullTextIndex, SparseIndex


@dataclass
class TableQuery:
    embedding: Optional[torch.Tensor] = None          # dense query vector [D]
    semantic_search: Optional[str] = None             # text for the dense embedder
    sparse_embedding: Optional[Mapping[int, float]] = None
    full_text_search: Optional[str] = None
    limit: int = 10
    search_effort: float = 0.5
    distance_under: Optional[float] = None
    distance_over: Optional[float] = None
    merge: MergeConfig = field(default_factory=MergeConfig)
    pruner: Optional[Pruner] = None
    rerank_query: Optional[str] = None                # set to re-score the fused hits with the cross-encoder
    rerank_field: str = "text"
    candidates: int = 0                               # per-index candidates before fusion (0: 4 x limit)


@dataclass
class TableHit:
    id: Hashable
    score: float
    index_scores: Dict[str, float]
    document: Optional[dict] = None


class Table:
    def __init__(self, name: str, dense_index=None, embed: Optional[Callable[[Sequence[str]], torch.Tensor]] = None,
                 sparse_terms: int = 0, sparse_encode: Optional[Callable[[Sequence[str]], torch.Tensor]] = None,
                 rerank: Optional[Callable[[str, Sequence[str]], Sequence[float]]] = None, text_field: str = "text",
                 device="cpu"):
        """``dense_index``: any index with ``add(vectors, ids)`` / ``search(q, k[, effort])`` returning distances
        and integer ids (flat, IVF, HBC, sharded).  ``embed`` / ``sparse_encode`` / ``rerank`` are the model
        pipelines (callables so that the table does not depend on how they are served)."""
        self.name, self.dense, self.embed, self.rerank = name, dense_index, embed, rerank
        self.sparse = SparseIndex(sparse_terms, device) if sparse_terms else None
        self.sparse_encode, self.text_field = sparse_encode, text_field
        self.fulltext = FullTextIndex(device=device)
        self.docs: Dict[Hashable, dict] = {}
        self._int_of: Dict[Hashable, int] = {}
        self._key_of: List[Hashable] = []

    def __len__(self) -> int:
        return len(self.docs)

    def upsert(self, docs: Mapping[Hashable, dict], embeddings: Optional[torch.Tensor] = None) -> None:
        keys = list(docs)
        texts = [str(docs[k].get(self.text_field, "")) for k in keys]
        for k, t in zip(keys, texts):
            self.docs[k] = docs[k]
            self.fulltext.add(k, t)
        if self.dense is not None:
            if embeddings is None:
                if self.embed is None:
                    raise ValueError("table has a dense index but neither embeddings nor an embedder were given")
                embeddings = self.embed(texts)
            ints = []
            for k in keys:
                if k not in self._int_of:
                    self._int_of[k] = len(self._key_of)
                    self._key_of.append(k)
                ints.append(self._int_of[k])
            self.dense.add(embeddings.float(), torch.tensor(ints, dtype=torch.int64))
        if self.sparse is not None and self.sparse_encode is not None:
            self.sparse.add_dense_rows(keys, self.sparse_encode(texts))

    def delete(self, key: Hashable) -> bool:
        found = self.docs.pop(key, None) is not None
        self.fulltext.delete(key)
        if self.sparse is not None:
            self.sparse.delete(key)
        return found                                   # dense entries are filtered at query time

    def query(self, q: TableQuery) -> List[TableHit]:
        n_cand = q.candidates or 4 * q.limit
        per_index: Dict[str, List] = {}
        emb = q.embedding
        if emb is None and q.semantic_search is not None and self.dense is not None:
            if self.embed is None:
                raise ValueError("semantic_search needs an embedder")
            emb = self.embed([q.semantic_search])[0]
        if emb is not None and self.dense is not None:
            try:
                res = self.dense.search(emb.float()[None], n_cand, effort=q.search_effort)
            except TypeError:
                res = self.dense.search(emb.float()[None], n_cand)
            hits = []
            for dist, i in zip(res.distances[0].tolist(), res.ids[0].tolist()):
                if i < 0 or i >= len(self._key_of) or self._key_of[i] not in self.docs:
                    continue
                if (q.distance_under is not None and dist >= q.distance_under) or \
                        (q.distance_over is not None and dist <= q.distance_over):
                    continue
                hits.append((self._key_of[i], -float(dist)))       # fusion wants higher-is-better
            per_index["dense"] = hits
        sp = q.sparse_embedding
        if sp is None and q.semantic_search is not None and self.sparse is not None and self.sparse_encode is not None:
            row = self.sparse_encode([q.semantic_search])[0]
            nz = (row > 0).nonzero().flatten()
            sp = dict(zip(nz.tolist(), row[nz].tolist()))
        if sp is not None and self.sparse is not None:
            per_index["sparse"] = self.sparse.search(sp, n_cand)
        if q.full_text_search:
            per_index["full_text"] = self.fulltext.search(q.full_text_search, n_cand)
        fused: List[FusedHit] = fuse(per_index, q.merge)
        if q.pruner is not None:
            fused = prune(fused, q.pruner)
        if q.rerank_query is not None and fused:
            if self.rerank is None:
                raise ValueError("rerank requested but the table has no reranker")
            head = fused[: max(q.limit, n_cand)]
            scores = self.rerank(q.rerank_query, [str(self.docs[h.doc_id].get(q.rerank_field, "")) for h in head])
            for h, s in zip(head, scores):
                h.index_scores["reranker"] = float(s)
                h.score = float(s)
            fused = sorted(head, key=lambda h: (-h.score, str(h.doc_id)))
        return [TableHit(h.doc_id, h.score, h.index_scores, self.docs.get(h.doc_id)) for h in fused[: q.limit]]
