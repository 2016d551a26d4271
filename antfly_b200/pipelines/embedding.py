"""Embedding pipeline: tokenize -> pack (no padding) -> encoder -> pool + L2-normalise on the GPU -> host.

Follows the reference's EmbeddingPipeline.embed (zig/pkg/inference/src/pipelines/embedding.zig:193-390): optional
task prefix, truncation to the model's max length, mean / cls / max / last pooling over active tokens, L2
normalise, optional ``dimensions`` truncation of the returned vector (zig/pkg/inference/src/server/server.zig:6717).
Differences that are the point of the B200 build: sequences are packed so no pad token reaches a GEMM, batches are
cut by a token budget and sorted by length, pooling runs on the device, and only [B, H] floats come back.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..models.bert import BertModel, PackedBatch, pack_sequences

TASK_PREFIXES = {
    "RETRIEVAL_QUERY": "query: ", "QUESTION_ANSWERING": "query: ", "FACT_VERIFICATION": "query: ",
    "CODE_RETRIEVAL_QUERY": "query: ", "RETRIEVAL_DOCUMENT": "passage: ",
}
INPUT_TYPE_ALIASES = {"search_query": "RETRIEVAL_QUERY", "query": "RETRIEVAL_QUERY",
                      "search_document": "RETRIEVAL_DOCUMENT", "document": "RETRIEVAL_DOCUMENT",
                      "classification": "CLASSIFICATION", "clustering": "CLUSTERING"}


def synthetic_batches(n: int, batch: int = 256, lo: int = 32, hi: int = 512, vocab=(1000, 30000), seed: int = 0
                      ) -> List[PackedBatch]:
    """Random packed batches: lengths uniform in [lo, hi], ids uniform in vocab, [CLS]=101 / [SEP]=102 at the ends."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        lens = torch.randint(lo, hi + 1, (batch,), generator=g)
        seqs = []
        for L in lens.tolist():
            ids = torch.randint(vocab[0], vocab[1], (L,), generator=g)
            ids[0], ids[-1] = 101, 102
            seqs.append(ids.tolist())
        out.append(pack_sequences(seqs))
    return out


class Embedder:
    def __init__(self, model: BertModel, tokenizer=None, max_length: int = 512, pooling: Optional[str] = None,
                 normalize: bool = True, max_batch_tokens: int = 131072, use_prefixes: bool = False):
        self.model, self.tokenizer = model, tokenizer
        self.max_length = min(max_length, model.cfg.max_position_embeddings)
        self.pooling = pooling or model.cfg.pooling
        self.normalize = normalize
        self.max_batch_tokens = max_batch_tokens
        self.use_prefixes = use_prefixes
        self.device = model.device

    @property
    def dim(self) -> int:
        return self.model.cfg.hidden_size

    # -- device-level entry points ---------------------------------------------------------------------
    def embed_packed(self, b: PackedBatch) -> torch.Tensor:
        """Device batch in, device embeddings out: fp32 [B, H]."""
        return self.model.embed(b, self.pooling, self.normalize)

    def embed_host(self, b: PackedBatch) -> torch.Tensor:
        """Host (ideally pinned) batch in, host embeddings out; the copies ride the current stream."""
        dev_b = b.to(self.device, non_blocking=True)
        out = self.embed_packed(dev_b)
        return out.cpu()

    # -- text-level API ----------------------------------------------------------------------------------
    def tokenize(self, texts: Sequence[str], task_type: Optional[str] = None) -> List[List[int]]:
        if self.tokenizer is None:
            raise RuntimeError("this embedder has no tokenizer; pass token ids to embed_ids()")
        prefix = TASK_PREFIXES.get(task_type or "", "") if self.use_prefixes else ""
        return [self.tokenizer.encode_for_model(prefix + t, self.max_length) for t in texts]

    def embed_ids(self, seqs: Sequence[Sequence[int]], dimensions: Optional[int] = None) -> torch.Tensor:
        """Token-id lists -> fp32 [N, H] on the host, input order preserved."""
        n = len(seqs)
        out = torch.empty((n, self.dim), dtype=torch.float32)
        order = sorted(range(n), key=lambda i: len(seqs[i]))
        i = 0
        off = self.model.cfg.position_offset
        while i < n:
            tok, j = 0, i
            while j < n and (j == i or tok + len(seqs[order[j]]) <= self.max_batch_tokens):
                tok += len(seqs[order[j]])
                j += 1
            idx = order[i:j]
            b = pack_sequences([list(seqs[k][: self.max_length]) for k in idx], position_offset=off)
            if self.device.type == "cuda":
                b = b.pin()
            out[torch.tensor(idx)] = self.embed_host(b)
            i = j
        if dimensions is not None:
            if not (0 < dimensions <= self.dim):
                raise ValueError(f"dimensions must be in [1, {self.dim}]")
            out = out[:, :dimensions].contiguous()
        return out

    def embed(self, texts: Sequence[str], task_type: Optional[str] = None, dimensions: Optional[int] = None):
        """Returns (embeddings fp32 [N, dims] on the host, number of prompt tokens)."""
        seqs = self.tokenize(texts, task_type)
        return self.embed_ids(seqs, dimensions), sum(len(s) for s in seqs)


class SparseEmbedder:
    """SPLADE: ``log(1 + relu(logits))`` max-pooled over the sequence, returned as sorted {indices, values}
    (zig/pkg/inference/src/pipelines/sparse_embedding.zig:19-21).  The MLM head is a GEMM over the vocabulary."""

    def __init__(self, model: BertModel, mlm_weight: torch.Tensor, mlm_bias: Optional[torch.Tensor] = None,
                 tokenizer=None, max_length: int = 512, top_k: int = 0):
        self.model, self.w, self.b, self.tokenizer = model, mlm_weight, mlm_bias, tokenizer
        self.max_length, self.top_k = max_length, top_k

    def embed_ids(self, seqs):
        from ..ops import dense as Dn

        b = pack_sequences([list(s[: self.max_length]) for s in seqs]).to(self.model.device)
        h = self.model.encode(b)
        logits = Dn.gemm_bf16(h, self.w, bias=self.b)
        pooled = Dn.splade_pool(logits, b.starts, b.lens).cpu()
        out = []
        for row in pooled:
            nz = torch.nonzero(row > 0).flatten()
            vals = row[nz]
            if self.top_k and nz.numel() > self.top_k:
                keep = torch.topk(vals, self.top_k).indices.sort().values
                nz, vals = nz[keep], vals[keep]
            out.append({"indices": nz.tolist(), "values": vals.tolist()})
        return out
