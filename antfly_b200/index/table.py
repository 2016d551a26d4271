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
from typing import Callable, Dict, Hashable, List, Mapping, Optional, Sequence, Tuple

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
    # restrictions applied before scoring (specs/openapi/antfly/metadata.yaml QueryRequest): documents whose key
    # starts with filter_prefix, that match filter_query and do not match exclusion_query (index/docfilter.py)
    filter_prefix: Optional[str] = None
    filter_query: object = None
    exclusion_query: object = None
    # full-text-only queries: sort by document fields ([{"field", "desc"}]; "score" / "_score" is the match score,
    # "_id" the key) and page with a cursor of the previous page's last sort values
    order_by: Optional[List[dict]] = None
    search_after: Optional[List[str]] = None
    profile: Optional[dict] = None                    # a dictionary to fill with per-phase milliseconds


@dataclass
class TableHit:
    id: Hashable
    score: float
    index_scores: Dict[str, float]
    document: Optional[dict] = None
    sort: Optional[List[str]] = None                  # sort values under order_by (the cursor for search_after)


class Table:
    def __init__(self, name: str, dense_index=None, embed: Optional[Callable[[Sequence[str]], torch.Tensor]] = None,
                 sparse_terms: int = 0, sparse_encode: Optional[Callable[[Sequence[str]], torch.Tensor]] = None,
                 rerank: Optional[Callable[[str, Sequence[str]], Sequence[float]]] = None, text_field: str = "text",
                 device="cpu", store=None):
        """``dense_index``: any index with ``add(vectors, ids)`` / ``search(q, k[, effort])`` returning distances
        and integer ids (flat, IVF, HBC, sharded).  ``embed`` / ``sparse_encode`` / ``rerank`` are the model
        pipelines (callables so that the table does not depend on how they are served).

        ``store``: an :class:`antfly_b200.index.lsm_store.LsmStore`.  With one, every upsert / delete batch is one
        write transaction (documents as JSON under namespace 4, their embeddings as little-endian fp32 under
        namespace 5, sparse rows under 6), and :meth:`recover` rebuilds the in-memory indexes from it without
        running any model -- the document store / index split of the reference's shard database
        (zig/pkg/antfly/src/storage/docstore.zig over its LSM backend)."""
        self.store = store
        self.name, self.dense, self.embed, self.rerank = name, dense_index, embed, rerank
        self.sparse = SparseIndex(sparse_terms, device) if sparse_terms else None
        self.sparse_encode, self.text_field = sparse_encode, text_field
        self.fulltext = FullTextIndex(device=device)
        self.docs: Dict[Hashable, dict] = {}
        self._int_of: Dict[Hashable, int] = {}
        self._key_of: List[Hashable] = []

    def __len__(self) -> int:
        return len(self.docs)

    # -- durability ----------------------------------------------------------------------------------------
    NS_DOCS, NS_EMBEDDINGS, NS_SPARSE = 4, 5, 6

    @staticmethod
    def _store_key(key: Hashable) -> bytes:
        if isinstance(key, str):
            return b"s" + key.encode("utf-8")
        if isinstance(key, int) and not isinstance(key, bool) and 0 <= key < 1 << 64:
            return b"i" + key.to_bytes(8, "big")
        raise TypeError("a durable table takes string or non-negative integer keys")

    @staticmethod
    def _from_store_key(raw: bytes) -> Hashable:
        return raw[1:].decode("utf-8") if raw[:1] == b"s" else int.from_bytes(raw[1:], "big")

    def recover(self, batch: int = 1024) -> int:
        """Re-applies what the store holds to the in-memory indexes.  -> documents restored."""
        import json

        if self.store is None:
            return 0
        store, self.store = self.store, None                  # the replay must not write back
        try:
            n = 0
            with store.begin_read() as r:
                rows: List[Tuple[Hashable, dict, Optional[bytes], Optional[bytes]]] = []

                def apply():
                    if not rows:
                        return
                    docs = {k: d for k, d, _, _ in rows}
                    have = [e is not None for _, _, e, _ in rows]
                    emb = None
                    if self.dense is not None:
                        if not all(have):
                            raise ValueError(f"table {self.name!r}: stored documents without stored embeddings")
                        emb = torch.stack([torch.frombuffer(bytearray(e), dtype=torch.float32) for _, _, e, _ in rows])
                    sp = None
                    if self.sparse is not None and all(s is not None for _, _, _, s in rows):
                        sp = torch.stack([torch.frombuffer(bytearray(s), dtype=torch.float32) for _, _, _, s in rows])
                    self._apply(docs, emb, sp)
                    rows.clear()

                for raw, body in r.items(self.NS_DOCS):
                    rows.append((self._from_store_key(raw), json.loads(body), r.get(self.NS_EMBEDDINGS, raw),
                                 r.get(self.NS_SPARSE, raw)))
                    n += 1
                    if len(rows) >= batch:
                        apply()
                apply()
            return n
        finally:
            self.store = store

    def upsert(self, docs: Mapping[Hashable, dict], embeddings: Optional[torch.Tensor] = None) -> None:
        keys = list(docs)
        texts = [str(docs[k].get(self.text_field, "")) for k in keys]
        if self.dense is not None and embeddings is None:
            if self.embed is None:
                raise ValueError("table has a dense index but neither embeddings nor an embedder were given")
            embeddings = self.embed(texts)
        sparse_rows = self.sparse_encode(texts) if self.sparse is not None and self.sparse_encode is not None else None
        if self.store is not None:                            # durable first: a crash after this point replays it
            import json

            with self.store.begin_write() as w:
                for i, k in enumerate(keys):
                    raw = self._store_key(k)
                    w.put(self.NS_DOCS, raw, json.dumps(docs[k], separators=(",", ":")).encode("utf-8"))
                    if self.dense is not None:
                        w.put(self.NS_EMBEDDINGS, raw, embeddings[i].detach().float().cpu().numpy().astype("<f4").tobytes())
                    if sparse_rows is not None:
                        w.put(self.NS_SPARSE, raw, sparse_rows[i].detach().float().cpu().numpy().astype("<f4").tobytes())
        self._apply(docs, embeddings, sparse_rows)

    def _apply(self, docs: Mapping[Hashable, dict], embeddings: Optional[torch.Tensor],
               sparse_rows: Optional[torch.Tensor]) -> None:
        keys = list(docs)
        texts = [str(docs[k].get(self.text_field, "")) for k in keys]
        for k, t in zip(keys, texts):
            self.docs[k] = docs[k]
            self.fulltext.add(k, t)
        if self.dense is not None:
            ints = []
            for k in keys:
                if k not in self._int_of:
                    self._int_of[k] = len(self._key_of)
                    self._key_of.append(k)
                ints.append(self._int_of[k])
            self.dense.add(embeddings.float(), torch.tensor(ints, dtype=torch.int64))
        if self.sparse is not None and sparse_rows is not None:
            self.sparse.add_dense_rows(keys, sparse_rows)

    def delete(self, key: Hashable) -> bool:
        found = self.docs.pop(key, None) is not None
        if found and self.store is not None:
            raw = self._store_key(key)
            with self.store.begin_write() as w:
                for ns in (self.NS_DOCS, self.NS_EMBEDDINGS, self.NS_SPARSE):
                    w.delete(ns, raw)
        self.fulltext.delete(key)
        if self.sparse is not None:
            self.sparse.delete(key)
        return found                                   # dense entries are filtered at query time

    def allowed_keys(self, q: TableQuery) -> Optional[set]:
        """The keys a query may return, or None when it has no restriction."""
        if not (q.filter_prefix or q.filter_query or q.exclusion_query):
            return None
        from .docfilter import compile_filter

        keep = compile_filter(q.filter_query)
        drop = compile_filter(q.exclusion_query) if q.exclusion_query else None
        out = set()
        for k, d in self.docs.items():
            if q.filter_prefix and not str(k).startswith(q.filter_prefix):
                continue
            if keep(d) and not (drop is not None and drop(d)):
                out.add(k)
        return out

    def query(self, q: TableQuery) -> List[TableHit]:
        import time as _time

        t_start = _time.perf_counter()
        prof = q.profile if q.profile is not None else {}

        def lap(name, t0):
            prof[name] = prof.get(name, 0.0) + (_time.perf_counter() - t0) * 1e3

        n_cand = q.candidates or 4 * q.limit
        t0 = _time.perf_counter()
        allowed = self.allowed_keys(q)
        lap("filter_ms", t0)
        if allowed is not None:
            prof["filter_matches"] = len(allowed)
            if not allowed:
                prof["total_ms"] = (_time.perf_counter() - t_start) * 1e3
                return []
            # the indexes do not know the restriction: ask for more candidates in proportion to how selective it is
            n_cand = min(max(len(self.docs), 1), int(n_cand * max(len(self.docs), 1) / len(allowed)) + 1)
        ok = (lambda k: True) if allowed is None else allowed.__contains__
        per_index: Dict[str, List] = {}
        emb = q.embedding
        if emb is None and q.semantic_search is not None and self.dense is not None:
            if self.embed is None:
                raise ValueError("semantic_search needs an embedder")
            emb = self.embed([q.semantic_search])[0]
        if emb is not None and self.dense is not None:
            t0 = _time.perf_counter()
            try:
                res = self.dense.search(emb.float()[None], n_cand, effort=q.search_effort)
            except TypeError:
                res = self.dense.search(emb.float()[None], n_cand)
            hits = []
            for dist, i in zip(res.distances[0].tolist(), res.ids[0].tolist()):
                if i < 0 or i >= len(self._key_of) or self._key_of[i] not in self.docs or not ok(self._key_of[i]):
                    continue
                if (q.distance_under is not None and dist >= q.distance_under) or \
                        (q.distance_over is not None and dist <= q.distance_over):
                    continue
                hits.append((self._key_of[i], -float(dist)))       # fusion wants higher-is-better
            per_index["dense"] = hits
            lap("dense_ms", t0)
        sp = q.sparse_embedding
        if sp is None and q.semantic_search is not None and self.sparse is not None and self.sparse_encode is not None:
            row = self.sparse_encode([q.semantic_search])[0]
            nz = (row > 0).nonzero().flatten()
            sp = dict(zip(nz.tolist(), row[nz].tolist()))
        if sp is not None and self.sparse is not None:
            t0 = _time.perf_counter()
            per_index["sparse"] = [h for h in self.sparse.search(sp, n_cand) if ok(h[0])]
            lap("sparse_ms", t0)
        if q.full_text_search:
            t0 = _time.perf_counter()
            per_index["full_text"] = [h for h in self.fulltext.search(q.full_text_search, n_cand) if ok(h[0])]
            lap("full_text_ms", t0)
        if not per_index and allowed is not None:                 # a pure filter query: everything that passes
            per_index["filter"] = [(k, 1.0) for k in sorted(allowed, key=str)]
        t0 = _time.perf_counter()
        fused: List[FusedHit] = fuse(per_index, q.merge)
        lap("merge_ms", t0)
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
        if q.order_by:
            fused = self._ordered(fused, q.order_by, q.search_after)
        prof["total_ms"] = (_time.perf_counter() - t_start) * 1e3
        return [TableHit(h.doc_id, h.score, h.index_scores, self.docs.get(h.doc_id), getattr(h, "sort", None))
                for h in fused[: q.limit]]

    def _ordered(self, fused: List[FusedHit], order_by: List[dict], search_after: Optional[List[str]]):
        """Sort by document fields; each hit gets its sort values (strings, as they travel in a cursor); with
        ``search_after`` only hits strictly after that cursor remain."""
        def value(h, field):
            if field in ("score", "_score"):
                return h.score
            if field == "_id":
                return str(h.doc_id)
            return (self.docs.get(h.doc_id) or {}).get(field)

        def key_part(v, desc):
            # missing values last in either direction; numbers before strings; descending by negation / inversion
            if v is None:
                return (2, 0, "")
            if isinstance(v, (int, float)) and not isinstance(v, bool):
                return (0, -float(v) if desc else float(v), "")
            s = str(v)
            return (1, 0, "".join(chr(0x10FFFF - ord(c)) for c in s) if desc else s)

        specs = [(str(o.get("field", "_score")), bool(o.get("desc", False))) for o in order_by] + [("_id", False)]
        for h in fused:
            h.sort = [("" if value(h, f) is None else str(value(h, f))) for f, _ in specs]
            h._key = tuple(key_part(value(h, f), d) for f, d in specs)
        fused = sorted(fused, key=lambda h: h._key)
        if search_after:
            cur = list(search_after) + [""] * (len(specs) - len(search_after))

            def coerce(text, f):
                if text == "":
                    return None
                if f in ("score", "_score"):
                    return float(text)
                sample = next((value(h, f) for h in fused if value(h, f) is not None), None)
                return float(text) if isinstance(sample, (int, float)) and not isinstance(sample, bool) else text

            after = tuple(key_part(coerce(t, f), d) for t, (f, d) in zip(cur, specs))
            fused = [h for h in fused if h._key > after]
        return fused
