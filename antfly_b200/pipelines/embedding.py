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


class DecoderEmbedder:
    """Text embeddings from a decoder-only model (Qwen3-Embedding, E5-Mistral and the like): the prompt is run
    causally through the stack, the final-norm hidden state of the LAST token is the embedding, L2-normalised;
    ``dimensions`` truncates and re-normalises (Matryoshka).  The reference's resident Qwen3 embedding path does
    the same (zig/pkg/inference/src/pipelines/embedding.zig:893 ``tryEmbedTextResidentQwen3``).  Prompts are
    packed into one causal prefill pass over a scratch paged KV cache."""

    def __init__(self, model, tokenizer=None, max_length: int = 8192, append_eos: bool = True,
                 instruction: Optional[str] = None, page: int = 16):
        self.model, self.tokenizer, self.max_length = model, tokenizer, max_length
        self.append_eos, self.instruction, self.page = append_eos, instruction, page

    @property
    def dim(self) -> int:
        return self.model.cfg.hidden_size

    def tokenize(self, texts: Sequence[str], task_type: Optional[str] = None) -> List[List[int]]:
        if self.tokenizer is None:
            raise RuntimeError("this embedder has no tokenizer")
        out = []
        for t in texts:
            if self.instruction and task_type in (None, "query", "search_query"):
                t = f"Instruct: {self.instruction}\nQuery:{t}"
            ids = self.tokenizer.encode(t)[: self.max_length - 1]
            eos = self.tokenizer.special.eos_id
            out.append(ids + ([eos] if self.append_eos and eos is not None else []))
        return out

    def embed_ids(self, seqs: Sequence[Sequence[int]], dimensions: Optional[int] = None,
                  max_batch_tokens: int = 16384) -> torch.Tensor:
        from ..models.llama import StepBatch

        m, dev, page = self.model, self.model.device, self.page
        outs = []
        i = 0
        while i < len(seqs):
            j, tok = i, 0
            while j < len(seqs) and (j == i or tok + len(seqs[j]) <= max_batch_tokens):
                tok += len(seqs[j])
                j += 1
            group = seqs[i:j]
            lens = [len(s) for s in group]
            blocks = [(n + page - 1) // page for n in lens]
            nblk, maxb = sum(blocks), max(blocks)
            kc = torch.zeros((m.n_layers, nblk, page, m.Hkv, m.D), dtype=torch.bfloat16, device=dev)
            vc = torch.zeros_like(kc)
            tables = torch.zeros((len(group), maxb), dtype=torch.int32)
            slots, pos, b0 = [], [], 0
            for r, (n, nb) in enumerate(zip(lens, blocks)):
                tables[r, :nb] = torch.arange(b0, b0 + nb, dtype=torch.int32)
                slots.extend(range(b0 * page, b0 * page + n))
                pos.extend(range(n))
                b0 += nb
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            ql = i32(lens)
            qs = (torch.cumsum(ql, 0) - ql).to(torch.int32)
            batch = StepBatch(i32([t for s in group for t in s]), i32(pos), i32(slots), qs, ql, ql.clone(),
                              tables.to(dev), (qs + ql - 1).to(torch.int32), max(lens), 1)
            prev, m.return_hidden = m.return_hidden, True
            try:
                h = m.forward(batch, kc, vc).float()
            finally:
                m.return_hidden = prev
            outs.append(h)
            i = j
        e = torch.cat(outs, 0) if outs else torch.zeros((0, self.dim))
        if dimensions:
            if dimensions > e.shape[1]:
                raise ValueError(f"dimensions {dimensions} exceeds the model's {e.shape[1]}")
            e = e[:, :dimensions]
        return torch.nn.functional.normalize(e, dim=-1).cpu()

    def embed(self, texts: Sequence[str], task_type: Optional[str] = None, dimensions: Optional[int] = None):
        seqs = self.tokenize(texts, task_type)
        return self.embed_ids(seqs, dimensions), sum(len(s) for s in seqs)
