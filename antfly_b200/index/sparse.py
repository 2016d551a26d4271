"""Sparse (learned-term, SPLADE-style) inverted index and a BM25 full-text index over the same posting structure.

Postings are kept as one COO / CSR triple of tensors (term ids, doc slots, weights), so a query is: gather the
posting ranges of its terms, multiply by the query weights, scatter-add into a score vector, top-k -- all tensor ops
that run wherever the index lives (HBM for a GPU-resident index).  New documents go to a small append buffer that
is merged into the sorted arrays when it grows past a threshold; deletes clear a per-slot live flag.

The reference keeps sparse postings in chunked inverted lists (zig/pkg/antfly/src/sparse/, go/pkg/antfly/lib/
sparseindex) and scores full text with BM25 (zig/pkg/antfly/src/search/: scorer, analyzers); the scoring rules are
the same (dot product of term weights; BM25 with k1 = 1.2, b = 0.75 and the ``ln(1 + (N - df + 0.5) / (df + 0.5))``
idf).
"""
from __future__ import annotations

import math
import re
from typing import Dict, Hashable, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch


class SparseIndex:
    def __init__(self, num_terms: int, device="cpu", merge_threshold: int = 65536):
        self.num_terms, self.device, self.merge_threshold = num_terms, torch.device(device), merge_threshold
        self.ids: List[Hashable] = []                       # slot -> external id
        self.slot_of: Dict[Hashable, int] = {}
        self.live = torch.zeros(0, dtype=torch.bool, device=self.device)
        # merged postings, sorted by term
        self.terms = torch.zeros(0, dtype=torch.int64, device=self.device)
        self.slots = torch.zeros(0, dtype=torch.int64, device=self.device)
        self.weights = torch.zeros(0, dtype=torch.float32, device=self.device)
        self.offsets = torch.zeros(num_terms + 1, dtype=torch.int64, device=self.device)
        self._buf: List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = []
        self._buf_n = 0

    def __len__(self) -> int:
        return int(self.live.sum())

    # -- writes --------------------------------------------------------------------------------------------
    def add(self, doc_id: Hashable, vector: Mapping[int, float]) -> None:
        self.add_batch([doc_id], [vector])

    def add_batch(self, doc_ids: Sequence[Hashable], vectors: Sequence[Mapping[int, float]]) -> None:
        t, s, w = [], [], []
        for d, vec in zip(doc_ids, vectors):
            if d in self.slot_of:
                self.delete(d)
            slot = len(self.ids)
            self.ids.append(d)
            self.slot_of[d] = slot
            for term, weight in vec.items():
                if weight != 0.0:
                    if not 0 <= int(term) < self.num_terms:
                        raise ValueError(f"term id {term} outside [0, {self.num_terms})")
                    t.append(int(term)), s.append(slot), w.append(float(weight))
        grow = len(self.ids) - self.live.numel()
        self.live = torch.cat([self.live, torch.ones(grow, dtype=torch.bool, device=self.device)])
        if t:
            self._buf.append((torch.tensor(t, device=self.device), torch.tensor(s, device=self.device),
                              torch.tensor(w, dtype=torch.float32, device=self.device)))
            self._buf_n += len(t)
        if self._buf_n >= self.merge_threshold:
            self.merge()

    def add_dense_rows(self, doc_ids: Sequence[Hashable], rows: torch.Tensor, min_weight: float = 0.0) -> None:
        """Rows of a [B, num_terms] activation matrix (what the SPLADE pooling kernel produces)."""
        vecs = []
        for r in rows:
            nz = (r > min_weight).nonzero().flatten()
            vecs.append(dict(zip(nz.tolist(), r[nz].tolist())))
        self.add_batch(doc_ids, vecs)

    def delete(self, doc_id: Hashable) -> bool:
        slot = self.slot_of.pop(doc_id, None)
        if slot is None:
            return False
        self.live[slot] = False
        return True

    def merge(self) -> None:
        """Fold the append buffer into the sorted posting arrays and drop postings of deleted documents."""
        parts = [(self.terms, self.slots, self.weights)] + self._buf
        t = torch.cat([p[0] for p in parts])
        s = torch.cat([p[1] for p in parts])
        w = torch.cat([p[2] for p in parts])
        keep = self.live[s] if s.numel() else torch.zeros(0, dtype=torch.bool, device=self.device)
        t, s, w = t[keep], s[keep], w[keep]
        order = torch.sort(t, stable=True).indices
        self.terms, self.slots, self.weights = t[order], s[order], w[order]
        counts = torch.bincount(self.terms, minlength=self.num_terms)
        self.offsets = torch.cat([torch.zeros(1, dtype=torch.int64, device=self.device), counts.cumsum(0)])
        self._buf, self._buf_n = [], 0

    # -- reads ---------------------------------------------------------------------------------------------
    def doc_freq(self, term: int) -> int:
        self.merge() if self._buf else None
        return int(self.offsets[term + 1] - self.offsets[term])

    def scores(self, query: Mapping[int, float]) -> torch.Tensor:
        """Dot product of the query with every document slot (deleted slots score -inf)."""
        if self._buf:
            self.merge()
        acc = torch.zeros(len(self.ids), dtype=torch.float32, device=self.device)
        for term, qw in query.items():
            if 0 <= int(term) < self.num_terms and qw != 0.0:
                lo, hi = int(self.offsets[term]), int(self.offsets[term + 1])
                if hi > lo:
                    acc.index_add_(0, self.slots[lo:hi], self.weights[lo:hi] * float(qw))
        return acc.masked_fill(~self.live, float("-inf"))

    def search(self, query: Mapping[int, float], k: int) -> List[Tuple[Hashable, float]]:
        sc = self.scores(query)
        if sc.numel() == 0:
            return []
        v, i = torch.topk(sc, min(k, sc.numel()))
        return [(self.ids[j], float(x)) for x, j in zip(v.tolist(), i.tolist()) if x > 0.0]


_WORD = re.compile(r"\w+", re.UNICODE)
_STOP = frozenset("a an and are as at be but by for if in into is it no not of on or such that the their then there "
                  "these they this to was will with".split())


def analyze(text: str, stopwords: bool = True) -> List[str]:
    """Lower-cased unicode word tokens, English stop words removed, a light plural / -ing / -ed suffix strip."""
    out = []
    for tok in _WORD.findall(text.lower()):
        if stopwords and tok in _STOP:
            continue
        if len(tok) > 4:
            for suf, rep in (("ies", "y"), ("sses", "ss"), ("ing", ""), ("ed", ""), ("s", "")):
                if tok.endswith(suf) and not tok.endswith("ss") and len(tok) - len(suf) >= 3:
                    tok = tok[: len(tok) - len(suf)] + rep
                    break
        out.append(tok)
    return out


class FullTextIndex:
    """BM25 over analysed text.  Term frequencies are the posting weights of a :class:`SparseIndex` whose term ids
    come from a growing vocabulary; document lengths live beside it."""

    def __init__(self, k1: float = 1.2, b: float = 0.75, device="cpu", max_terms: int = 1 << 20):
        self.k1, self.b = k1, b
        self.vocab: Dict[str, int] = {}
        self.inv = SparseIndex(max_terms, device)
        self.doc_len: List[int] = []

    def _term(self, tok: str, create: bool) -> Optional[int]:
        t = self.vocab.get(tok)
        if t is None and create:
            t = self.vocab[tok] = len(self.vocab)
        return t

    def add(self, doc_id: Hashable, text: str) -> None:
        toks = analyze(text)
        tf: Dict[int, float] = {}
        for tok in toks:
            t = self._term(tok, True)
            tf[t] = tf.get(t, 0.0) + 1.0
        self.inv.add(doc_id, tf)
        self.doc_len.extend([0] * (len(self.inv.ids) - len(self.doc_len)))
        self.doc_len[self.inv.slot_of[doc_id]] = len(toks)

    def delete(self, doc_id: Hashable) -> bool:
        return self.inv.delete(doc_id)

    def search(self, text: str, k: int) -> List[Tuple[Hashable, float]]:
        inv = self.inv
        if inv._buf:
            inv.merge()
        n_docs = len(inv)
        if n_docs == 0:
            return []
        dl = torch.tensor(self.doc_len, dtype=torch.float32, device=inv.device)
        avg = float(dl[inv.live].mean()) or 1.0
        acc = torch.zeros(len(inv.ids), dtype=torch.float32, device=inv.device)
        for tok in set(analyze(text)):
            t = self._term(tok, False)
            if t is None:
                continue
            lo, hi = int(inv.offsets[t]), int(inv.offsets[t + 1])
            if hi == lo:
                continue
            slots, tf = inv.slots[lo:hi], inv.weights[lo:hi]
            live = inv.live[slots]
            df = int(live.sum())
            if df == 0:
                continue
            idf = math.log(1.0 + (n_docs - df + 0.5) / (df + 0.5))
            norm = tf * (self.k1 + 1.0) / (tf + self.k1 * (1.0 - self.b + self.b * dl[slots] / avg))
            acc.index_add_(0, slots, idf * norm * live)
        acc = acc.masked_fill(~inv.live, float("-inf"))
        v, i = torch.topk(acc, min(k, acc.numel()))
        return [(inv.ids[j], float(x)) for x, j in zip(v.tolist(), i.tolist()) if x > 0.0]
