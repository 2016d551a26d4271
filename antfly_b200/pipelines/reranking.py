"""Reranking pipeline: cross-encoder scoring and ColBERT-style late interaction.

Rules from the reference (zig/pkg/inference/src/pipelines/reranking.zig:83-383): a pair is encoded
``[CLS] query [SEP] doc [SEP]`` with the query keeping its tokens when the budget is short; logits map to a score as
``[B,1] -> sigmoid``, ``[B,>=2] -> softmax over the first two, P(label 1)``; late interaction scores a document as
the sum over query tokens of the best cosine with any document token, special tokens ignored.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..models.bert import BertModel, PackedBatch, pack_sequences
from ..ops import dense as Dn


def synthetic_pairs(n_queries: int, docs_per_query: int = 64, q_len: int = 32, d_len: int = 448,
                    vocab=(1000, 30000), seed: int = 0) -> List[PackedBatch]:
    """One packed batch per query: docs_per_query pairs of [CLS] q(q_len) [SEP] d(d_len) [SEP] (length q+d+3...)."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n_queries):
        q = torch.randint(vocab[0], vocab[1], (q_len - 2,), generator=g).tolist()
        seqs, types = [], []
        for _ in range(docs_per_query):
            d = torch.randint(vocab[0], vocab[1], (d_len - 1,), generator=g).tolist()
            ids = [101] + q + [102] + d + [102]
            seqs.append(ids)
            types.append([0] * (len(q) + 2) + [1] * (len(d) + 1))
        out.append(pack_sequences(seqs, types))
    return out


def scores_from_logits(logits: torch.Tensor) -> torch.Tensor:
    """reranking.zig:211-258."""
    if logits.dim() == 1 or logits.shape[-1] == 1:
        return torch.sigmoid(logits.reshape(-1).float())
    return torch.softmax(logits[:, :2].float(), -1)[:, 1]


class CrossEncoderReranker:
    def __init__(self, model: BertModel, tokenizer=None, max_length: int = 512, max_batch_tokens: int = 65536):
        assert model.cfg.num_labels > 0, "cross-encoder needs a classification head"
        self.model, self.tokenizer, self.max_length = model, tokenizer, max_length
        self.max_batch_tokens = max_batch_tokens
        self.device = model.device

    def score_packed(self, b: PackedBatch) -> torch.Tensor:
        return scores_from_logits(self.model.classify(b))

    def score_host(self, b: PackedBatch) -> torch.Tensor:
        return self.score_packed(b.to(self.device, non_blocking=True)).cpu()

    def rerank(self, query: str, docs: Sequence[str]) -> Tuple[List[float], int]:
        """Returns (scores in input order, prompt tokens)."""
        if self.tokenizer is None:
            raise RuntimeError("this reranker has no tokenizer")
        pairs = [self.tokenizer.encode_pair(query, d, self.max_length) for d in docs]
        scores = torch.empty(len(docs))
        i = 0
        while i < len(pairs):
            tok, j = 0, i
            while j < len(pairs) and (j == i or tok + len(pairs[j][0]) <= self.max_batch_tokens):
                tok += len(pairs[j][0])
                j += 1
            b = pack_sequences([p[0] for p in pairs[i:j]], [p[1] for p in pairs[i:j]],
                               position_offset=self.model.cfg.position_offset)
            if self.device.type == "cuda":
                b = b.pin()
            scores[i:j] = self.score_host(b)
            i = j
        return scores.tolist(), sum(len(p[0]) for p in pairs)


class LateInteractionReranker:
    """ColBERT MaxSim over token embeddings (optionally projected)."""

    def __init__(self, model: BertModel, tokenizer=None, projection: Optional[torch.Tensor] = None,
                 max_length: int = 512, batch_size: int = 32):
        self.model, self.tokenizer, self.proj = model, tokenizer, projection
        self.max_length, self.batch_size = max_length, batch_size

    def _token_embeddings(self, b: PackedBatch) -> torch.Tensor:
        h = self.model.encode(b)
        if self.proj is not None:
            h = Dn.gemm_bf16(h, self.proj)
        return h

    def score_ids(self, query_ids: Sequence[int], doc_ids: Sequence[Sequence[int]]) -> List[float]:
        dev = self.model.device
        # Special tokens ([CLS]/[SEP] at the ends) are left out of the interaction.
        qb = pack_sequences([list(query_ids)]).to(dev)
        q = self._token_embeddings(qb)[1:-1].contiguous()
        out: List[float] = []
        for i in range(0, len(doc_ids), self.batch_size):
            chunk = [list(d[: self.max_length]) for d in doc_ids[i:i + self.batch_size]]
            db = pack_sequences(chunk).to(dev)
            d = self._token_embeddings(db)
            starts = (db.starts + 1).int()
            lens = (db.lens - 2).clamp_min(0).int()
            out.extend(Dn.maxsim(q, d, starts, lens).cpu().tolist())
        return out

    def rerank(self, query: str, docs: Sequence[str]):
        q = self.tokenizer.encode_for_model(query, self.max_length)
        d = [self.tokenizer.encode_for_model(t, self.max_length) for t in docs]
        return self.score_ids(q, d), len(q) + sum(len(x) for x in d)
