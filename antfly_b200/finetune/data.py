"""Datasets for fine-tuning: JSONL readers per recipe, tokenisation with loss masks, sequence packing, batching.

Row formats follow the reference's recipe documentation (zig/pkg/inference/docs/finetuning/FINETUNING.md "Run
Artifacts": text preference rows ``{prompt, chosen, rejected}``, GRPO rows ``{prompt, target}``, the ``rendered-*``
dataset formats whose prompts are already final decoder prompts) plus the usual SFT shapes (``messages`` chats,
``prompt`` / ``completion`` pairs, plain ``text``), reranker pairs ``{query, document, label}`` and retrieval
triples ``{query, positive, negatives}``.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from ..pipelines.generation import ChatTemplate


def read_jsonl(path: str, max_examples: int = 0) -> List[dict]:
    rows = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            rows.append(json.loads(line))
            if max_examples and len(rows) >= max_examples:
                break
    return rows


def fingerprint(path: str) -> Dict[str, object]:
    """What a run manifest records about a dataset file: size, line count, sha256."""
    h, n, size = hashlib.sha256(), 0, 0
    with open(path, "rb") as f:
        for line in f:
            h.update(line)
            n += 1
            size += len(line)
    return {"path": path, "bytes": size, "lines": n, "sha256": h.hexdigest()}


@dataclass
class TokenExample:
    ids: List[int]
    loss_mask: List[int]             # 1 where the token is a training target

    def __len__(self):
        return len(self.ids)


class DecoderTokenizer:
    """Prompt rendering + tokenisation for decoder recipes: ``rendered`` prompts are used as they are, others are
    wrapped as a user turn through the model's chat template."""

    def __init__(self, tokenizer, chat_template: Optional[str] = None, rendered: bool = False, add_bos: bool = True):
        self.tok, self.rendered, self.add_bos = tokenizer, rendered, add_bos
        self.template = ChatTemplate(chat_template)
        self.eos = tokenizer.special.eos_id

    def prompt_ids(self, prompt) -> List[int]:
        if isinstance(prompt, list):
            text = self.template.apply(prompt, add_generation_prompt=True)
        else:
            text = prompt if self.rendered else self.template.apply([{"role": "user", "content": str(prompt)}])
        return self.tok.encode_prompt(text, add_bos=self.add_bos)

    def completion_ids(self, text: str, end: bool = True) -> List[int]:
        ids = self.tok.encode(text)
        return ids + ([self.eos] if end and self.eos is not None else [])

    def sft_example(self, row: dict, max_seq_len: int) -> TokenExample:
        if "messages" in row:
            msgs = row["messages"]
            if not msgs or msgs[-1].get("role") != "assistant":
                raise ValueError("a messages row must end with an assistant turn")
            p, c = self.prompt_ids(msgs[:-1]), self.completion_ids(str(msgs[-1].get("content", "")))
        elif "prompt" in row and ("completion" in row or "response" in row):
            p, c = self.prompt_ids(row["prompt"]), self.completion_ids(str(row.get("completion", row.get("response"))))
        elif "text" in row:
            ids = self.tok.encode_prompt(str(row["text"]), add_bos=self.add_bos)
            ids = (ids + ([self.eos] if self.eos is not None else []))[:max_seq_len]
            return TokenExample(ids, [1] * len(ids))
        else:
            raise ValueError("an SFT row needs messages, prompt + completion, or text")
        if len(p) + len(c) > max_seq_len:                      # keep the end of the prompt and the whole answer
            c = c[:max_seq_len]
            p = p[len(p) - (max_seq_len - len(c)):] if max_seq_len > len(c) else []
        return TokenExample(p + c, [0] * len(p) + [1] * len(c))


def pack_examples(examples: Sequence[TokenExample], max_seq_len: int, pad_id: int = 0) -> List[dict]:
    """First-fit-decreasing packing of examples into rows of at most ``max_seq_len`` tokens.  Each row carries
    ``ids``, ``loss_mask`` and ``doc_ids`` (one id per example of the row; padding gets an id of its own, so nothing
    attends to it and it attends to nothing else)."""
    order = sorted(range(len(examples)), key=lambda i: -len(examples[i]))
    rows: List[List[int]] = []
    space: List[int] = []
    for i in order:
        n = len(examples[i])
        if n > max_seq_len:
            raise ValueError(f"example of {n} tokens exceeds max_seq_len {max_seq_len}")
        for r in range(len(rows)):
            if space[r] >= n:
                rows[r].append(i)
                space[r] -= n
                break
        else:
            rows.append([i])
            space.append(max_seq_len - n)
    out = []
    for members in rows:
        ids, lm, doc = [], [], []
        for d, i in enumerate(members):
            ex = examples[i]
            ids += ex.ids
            lm += ex.loss_mask
            doc += [d] * len(ex)
        pad = max_seq_len - len(ids)
        out.append({"ids": ids + [pad_id] * pad, "loss_mask": lm + [0] * pad, "doc_ids": doc + [len(members)] * pad,
                    "examples": list(members)})
    return out


def pad_batch(seqs: Sequence[Sequence[int]], pad_id: int = 0, masks: Optional[Sequence[Sequence[int]]] = None):
    """Right-pad -> ids [B, S], attention mask [B, S] (bool), optional loss mask [B, S]."""
    S = max(len(s) for s in seqs)
    ids = torch.full((len(seqs), S), pad_id, dtype=torch.long)
    att = torch.zeros((len(seqs), S), dtype=torch.bool)
    lm = torch.zeros((len(seqs), S), dtype=torch.bool) if masks is not None else None
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.tensor(s, dtype=torch.long)
        att[i, : len(s)] = True
        if lm is not None:
            lm[i, : len(s)] = torch.tensor(masks[i], dtype=torch.bool)
    return ids, att, lm


def batches(items: Sequence, batch_size: int, epochs: int, seed: int, rank: int = 0, world: int = 1,
            start_step: int = 0) -> Iterator[Tuple[int, int, list]]:
    """(epoch, step, batch) over ``epochs`` seeded shuffles; each rank of a data-parallel job takes its slice of
    every global batch of ``batch_size * world`` items; ``start_step`` skips what a resumed run has already done."""
    step = 0
    glob = batch_size * world
    for ep in range(epochs):
        g = torch.Generator().manual_seed(seed + ep)
        order = torch.randperm(len(items), generator=g).tolist()
        for i in range(0, len(order) - glob + 1 if len(order) >= glob else 1, glob):
            chunk = order[i:i + glob]
            mine = chunk[rank * batch_size:(rank + 1) * batch_size] if len(chunk) == glob else chunk[rank::world]
            if step >= start_step and mine:
                yield ep, step, [items[j] for j in mine]
            step += 1


def encoder_pairs(tokenizer, rows: Sequence[dict], max_seq_len: int):
    """Reranker rows -> (ids, token types, label, group) with the pair encoding the serving path uses."""
    out, groups = [], {}
    for r in rows:
        ids, types = tokenizer.encode_pair(str(r["query"]), str(r.get("document", r.get("passage", ""))), max_seq_len)
        out.append({"ids": ids, "types": types, "label": float(r.get("label", r.get("score", 0.0))),
                    "group": groups.setdefault(str(r["query"]), len(groups))})
    return out


def encoder_triples(tokenizer, rows: Sequence[dict], max_seq_len: int, query_prefix: str = "", doc_prefix: str = ""):
    out, docs = [], {}
    for r in rows:
        enc = lambda t, p: tokenizer.encode_for_model(p + str(t), max_seq_len)
        out.append({"query": enc(r["query"], query_prefix), "positive": enc(r["positive"], doc_prefix),
                    "negatives": [enc(n, doc_prefix) for n in r.get("negatives", [])],
                    "doc": docs.setdefault(str(r["positive"]), len(docs))})      # same text, same document id
    return out
