"""Classification pipelines on the BERT-family encoder: sequence classification (one label distribution per text)
and token classification with entity aggregation (NER).

Follows the reference's classification and NER pipelines (zig/pkg/inference/src/pipelines/classification.zig,
zig/pkg/inference/src/pipelines/ner.zig): softmax over the labels (sigmoid per label for multi-label heads); for
NER the per-token arg-max tags in the BIO scheme are merged into spans -- a ``B-X`` or an ``I-X`` that does not
continue the open span starts a new entity, special tokens and word-piece continuations extend the current word --
and a span's score is the mean probability of its tokens.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..models.bert import BertModel, pack_sequences


@dataclass
class Entity:
    label: str
    start_token: int   # inclusive, index into the sequence's tokens
    end_token: int     # exclusive
    score: float
    text: Optional[str] = None


class TextClassifier:
    def __init__(self, model: BertModel, tokenizer=None, id2label: Optional[Dict[int, str]] = None,
                 multi_label: bool = False, max_length: int = 512):
        assert model.cfg.num_labels > 0
        self.model, self.tokenizer, self.multi_label, self.max_length = model, tokenizer, multi_label, max_length
        self.id2label = id2label or {i: f"LABEL_{i}" for i in range(model.cfg.num_labels)}

    def probabilities(self, seqs: Sequence[Sequence[int]]) -> torch.Tensor:
        b = pack_sequences(list(seqs), None, position_offset=self.model.cfg.position_offset)
        logits = self.model.classify(b.to(self.model.device)).float().cpu()
        return torch.sigmoid(logits) if self.multi_label else torch.softmax(logits, -1)

    def classify_ids(self, seqs: Sequence[Sequence[int]], top_k: int = 1) -> List[List[dict]]:
        p = self.probabilities(seqs)
        k = min(top_k, p.shape[-1])
        vals, idx = p.topk(k, -1)
        return [[{"label": self.id2label[int(i)], "score": float(v)} for v, i in zip(vr, ir)]
                for vr, ir in zip(vals, idx)]

    def classify(self, texts: Sequence[str], top_k: int = 1) -> List[List[dict]]:
        if self.tokenizer is None:
            raise RuntimeError("this classifier has no tokenizer")
        return self.classify_ids([self.tokenizer.encode_for_model(t, self.max_length) for t in texts], top_k)


class ZeroShotClassifier:
    """Labels the model was never trained on, through a natural-language-inference cross-encoder: every (text,
    label) pair becomes premise = text, hypothesis = ``template.format(label)``; a label's score is the probability
    of *entailment* against *contradiction* for that pair, normalised over the labels (single-label) or taken as is
    (multi-label).  The reference's classification pipeline offers the same mode for NLI checkpoints
    (zig/pkg/inference/src/pipelines/classification.zig zero-shot path)."""

    def __init__(self, model, tokenizer, id2label: Dict[int, str], template: str = "This example is {}.",
                 max_length: int = 512):
        names = {v.lower(): k for k, v in id2label.items()}
        if "entailment" not in names or "contradiction" not in names:
            raise ValueError("zero-shot classification needs a model with entailment / contradiction labels")
        self.ent, self.con = names["entailment"], names["contradiction"]
        self.model, self.tokenizer, self.template, self.max_length = model, tokenizer, template, max_length

    def classify(self, texts: Sequence[str], labels: Sequence[str], multi_label: bool = False) -> List[List[dict]]:
        tk = self.tokenizer
        seqs, types = [], []
        for t in texts:
            for lab in labels:
                ids, ty = tk.encode_pair(t, self.template.format(lab), self.max_length)
                seqs.append(ids), types.append(ty)
        b = pack_sequences(seqs, types, position_offset=self.model.cfg.position_offset)
        logits = self.model.classify(b.to(self.model.device)).float().cpu()
        pair = torch.softmax(logits[:, [self.con, self.ent]], -1)[:, 1].view(len(texts), len(labels))
        if not multi_label:
            ent = logits[:, self.ent].view(len(texts), len(labels))
            pair = torch.softmax(ent, -1)
        out = []
        for row in pair:
            order = torch.argsort(row, descending=True)
            out.append([{"label": labels[int(i)], "score": float(row[int(i)])} for i in order])
        return out


def aggregate_bio(tags: Sequence[str], scores: Sequence[float], is_special: Optional[Sequence[bool]] = None,
                  is_continuation: Optional[Sequence[bool]] = None) -> List[Entity]:
    """Merge per-token BIO tags into entity spans.  ``is_special`` tokens never start or extend an entity;
    ``is_continuation`` tokens (word-piece ``##`` pieces) take the tag of the word they continue."""
    n = len(tags)
    ents: List[Entity] = []
    cur: Optional[Entity] = None
    acc: List[float] = []

    def close():
        nonlocal cur, acc
        if cur is not None:
            cur.score = sum(acc) / max(len(acc), 1)
            ents.append(cur)
        cur, acc = None, []

    for i in range(n):
        if is_special is not None and is_special[i]:
            close()
            continue
        tag = tags[i]
        if is_continuation is not None and is_continuation[i] and cur is not None and cur.end_token == i:
            cur.end_token = i + 1
            acc.append(scores[i])
            continue
        if tag == "O" or tag == "":
            close()
            continue
        prefix, _, label = tag.partition("-")
        if not label:  # a scheme without B-/I- prefixes: consecutive equal labels form one entity
            prefix, label = "I", tag
        if prefix == "I" and cur is not None and cur.label == label and cur.end_token == i:
            cur.end_token = i + 1
            acc.append(scores[i])
        else:
            close()
            cur, acc = Entity(label, i, i + 1, 0.0), [scores[i]]
    close()
    return ents


class TokenClassifier:
    """NER: token logits -> BIO tags -> entity spans."""

    def __init__(self, model: BertModel, id2label: Dict[int, str], tokenizer=None, max_length: int = 512):
        assert model.cfg.num_labels == len(id2label)
        self.model, self.id2label, self.tokenizer, self.max_length = model, id2label, tokenizer, max_length

    def tag_ids(self, seqs: Sequence[Sequence[int]]):
        """Per sequence: (tags, scores) for every token."""
        b = pack_sequences(list(seqs), None, position_offset=self.model.cfg.position_offset)
        p = torch.softmax(self.model.token_logits(b.to(self.model.device)).float().cpu(), -1)
        vals, idx = p.max(-1)
        out, o = [], 0
        for s in seqs:
            n = len(s)
            out.append(([self.id2label[int(i)] for i in idx[o:o + n]], [float(v) for v in vals[o:o + n]]))
            o += n
        return out

    def entities_ids(self, seqs: Sequence[Sequence[int]], special_ids: Sequence[int] = ()) -> List[List[Entity]]:
        sp = set(special_ids)
        return [aggregate_bio(tags, scores, [t in sp for t in s]) for s, (tags, scores) in zip(seqs, self.tag_ids(seqs))]

    def entities(self, texts: Sequence[str]) -> List[List[Entity]]:
        if self.tokenizer is None:
            raise RuntimeError("this tagger has no tokenizer")
        tk = self.tokenizer
        seqs = [tk.encode_for_model(t, self.max_length) for t in texts]
        sp = [getattr(tk.special, n) for n in ("cls_id", "sep_id", "pad_id") if getattr(tk.special, n, None) is not None]
        res = self.entities_ids(seqs, sp)
        for s, ents in zip(seqs, res):
            for e in ents:
                e.text = tk.decode(s[e.start_token:e.end_token])
        return res
