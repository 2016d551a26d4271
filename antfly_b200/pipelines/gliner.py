"""Zero-shot entity recognition, label scoring and relation extraction with a GLiNER model.

The prompt is ``( [P] entities ( [E] label1 [E] label2 ... ) ) [SEP_TEXT]`` followed by the text's words, each
lower-cased and tokenised on its own so that sub-tokens map back to words.  Every span of up to ``max_width``
words gets one logit per label; spans whose sigmoid clears the threshold become entities with character offsets
into the original text.  With ``flat_ner`` overlapping entities are resolved in favour of the higher score, and
entities with the same label and text (ignoring case) are merged.  Follows the reference pipeline
(zig/pkg/inference/src/pipelines/gliner.zig:99 ``recognizeBatch``, :215 ``classifyBatch``, :620
``decodeEntitiesFromLogits``, :1253 ``splitIntoWords``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..models.gliner import GlinerInput, GlinerModel


@dataclass
class GlinerConfig:
    max_width: int = 12
    max_length: int = 512
    threshold: float = 0.5
    flat_ner: bool = True
    default_labels: List[str] = field(default_factory=list)
    relation_labels: List[str] = field(default_factory=list)
    relation_threshold: float = 0.0
    token_p: int = 0          # [P]
    token_c: int = 0          # [C]
    token_e: int = 0          # [E]
    token_r: int = 0          # [R]
    token_sep_text: int = 0   # [SEP_TEXT]

    @classmethod
    def from_files(cls, config: dict, added_tokens: Dict[str, int]) -> "GlinerConfig":
        """``config`` is the model's gliner config, ``added_tokens`` maps the marker strings to token ids."""
        c = cls(**{k: v for k, v in config.items() if k in cls.__dataclass_fields__})
        for name, tok in (("token_p", "[P]"), ("token_c", "[C]"), ("token_e", "[E]"), ("token_r", "[R]"),
                          ("token_sep_text", "[SEP_TEXT]")):
            if tok in added_tokens:
                setattr(c, name, int(added_tokens[tok]))
        return c


@dataclass
class GlinerEntity:
    text: str
    label: str
    start: int      # byte offsets into the UTF-8 text, like the reference's
    end: int
    score: float


def _is_word_byte(b: bytes, i: int) -> bool:
    c = b[i]
    return c >= 0x80 or c == 0x5F or 0x30 <= c <= 0x39 or 0x41 <= c <= 0x5A or 0x61 <= c <= 0x7A


def _scalar_len(b: bytes, i: int) -> int:
    c = b[i]
    n = 1 if c < 0x80 else 2 if c < 0xE0 else 3 if c < 0xF0 else 4
    return min(n, len(b) - i)


def split_words(text: str) -> List[Tuple[str, int, int]]:
    """(word, byte start, byte end) triples.  Runs of letters / digits / underscores / non-ASCII characters form a
    word, hyphens inside a word join it, ``@name`` handles and URLs stay whole, every other non-space character
    is a word of its own."""
    b = text.encode("utf-8")
    out: List[Tuple[str, int, int]] = []
    i, n = 0, len(b)
    while i < n:
        if b[i] in b" \t\n\r\x0b\x0c":
            i += 1
            continue
        s = i
        low = b[i:i + 8].lower()
        if low.startswith(b"http://") or low.startswith(b"https://") or low.startswith(b"www."):
            while i < n and b[i] not in b" \t\n\r\x0b\x0c":
                i += 1
        elif b[i] == 0x40 and i + 1 < n and _is_word_byte(b, i + 1):
            i += 1
            while i < n and _is_word_byte(b, i):
                i += _scalar_len(b, i)
        elif _is_word_byte(b, i):
            i += _scalar_len(b, i)
            while i < n:
                if _is_word_byte(b, i):
                    i += _scalar_len(b, i)
                elif b[i] == 0x2D and i + 1 < n and _is_word_byte(b, i + 1):
                    i += 1 + _scalar_len(b, i + 1)
                else:
                    break
        else:
            i += _scalar_len(b, i)
        out.append((b[s:i].decode("utf-8", "replace"), s, i))
    return out


def _sigmoid(x: float) -> float:
    return 1.0 / (1.0 + math.exp(-x)) if x >= 0 else math.exp(x) / (1.0 + math.exp(x))


@dataclass
class GlinerRelation:
    head: GlinerEntity
    tail: GlinerEntity
    label: str
    score: float


def parse_relation_label(label: str) -> Optional[Tuple[str, str, Optional[str]]]:
    """``head::relation`` or ``head::relation::tail`` -> (head label, relation, tail label or None)."""
    head, sep, rest = label.partition("::")
    if not sep or not head or not rest:
        return None
    rel, sep2, tail = rest.partition("::")
    if sep2:
        return (head, rel, tail) if rel and tail else None
    return head, rest, None


def relation_candidates(entity_labels: Sequence[str], relation_labels: Sequence[str]) -> List[str]:
    """The composite labels the model is asked about: a relation spelled ``head::rel[::tail]`` is kept when its
    entity types are among the requested ones, a bare relation name is paired with every entity type."""
    low = [e.lower() for e in entity_labels]
    out: List[str] = []
    for r in relation_labels:
        c = parse_relation_label(r)
        if c is None:
            out += [f"{e}::{r}" for e in entity_labels]
            continue
        head, rel, tail = c
        if tail is not None and tail.lower() not in low:
            continue
        if head.lower() in low:
            e = entity_labels[low.index(head.lower())]
            out.append(f"{e}::{rel}::{tail}" if tail is not None else f"{e}::{rel}")
    return out


def decode_entities(text: str, words: Sequence[Tuple[str, int, int]], num_words: int, logits, labels: Sequence[str],
                    threshold: float, flat_ner: bool) -> List[GlinerEntity]:
    """Span logits [words, widths, labels] -> entities (thresholded, overlaps resolved, duplicates merged)."""
    raw = text.encode("utf-8")
    ents: List[GlinerEntity] = []
    lg = logits.tolist()
    for w in range(min(num_words, len(lg))):
        for k, row in enumerate(lg[w]):
            if w + k >= num_words:
                break
            for li, v in enumerate(row):
                s = _sigmoid(v)
                if s >= threshold:
                    a, b = words[w][1], words[w + k][2]
                    ents.append(GlinerEntity(raw[a:b].decode("utf-8", "replace"), labels[li], a, b, s))
    if flat_ner and len(ents) > 1:
        keep: List[GlinerEntity] = []
        for e in sorted(ents, key=lambda e: -e.score):
            if not any(e.start < o.end and e.end > o.start for o in keep):
                keep.append(e)
        ents = keep
    ents.sort(key=lambda e: (e.start, e.end))
    merged: List[GlinerEntity] = []
    for e in ents:
        for i, o in enumerate(merged):
            if o.label.lower() == e.label.lower() and o.text.lower() == e.text.lower():
                if e.score > o.score:
                    merged[i] = e
                break
        else:
            merged.append(e)
    merged.sort(key=lambda e: (e.start, e.end))
    return merged


def match_relations(entities: Sequence[GlinerEntity], heads: Sequence[GlinerEntity]) -> List[GlinerRelation]:
    """A span found under a composite label is a relation's head; its tail is the nearest entity of the wanted
    type that does not overlap it."""
    out: List[GlinerRelation] = []
    for h in heads:
        c = parse_relation_label(h.label)
        if c is None:
            continue
        head_label, rel, tail_label = c
        head, mismatch = None, False
        for e in entities:
            if e.start == h.start and e.end == h.end:
                if e.label.lower() == head_label.lower():
                    head = e
                    break
                mismatch = True
        if head is None and mismatch:
            continue
        best, best_d = None, None
        for e in entities:
            if tail_label is not None and e.label.lower() != tail_label.lower():
                continue
            if h.start < e.end and e.start < h.end:
                continue
            d = e.start - h.end if h.end <= e.start else h.start - e.end
            if best_d is None or d < best_d:
                best, best_d = e, d
        if best is None:
            continue
        out.append(GlinerRelation(head or GlinerEntity(h.text, head_label, h.start, h.end, h.score), best, rel, h.score))
    return out


class GlinerPipeline:
    def __init__(self, model: GlinerModel, tokenizer, cfg: GlinerConfig):
        if not (cfg.token_p and cfg.token_e and cfg.token_sep_text):
            raise ValueError("the [P], [E] and [SEP_TEXT] marker token ids are required")
        self.model, self.tok, self.cfg = model, tokenizer, cfg

    def _encode(self, s: str) -> List[int]:
        return list(self.tok.encode(s))

    def prepare(self, text: str, labels: Sequence[str], label_token: int):
        """Prompt ids + word map for one text.  Words that would run past ``max_length`` are dropped whole."""
        words = split_words(text)
        ids = self._encode("(") + [self.cfg.token_p] + self._encode("entities") + self._encode("(")
        for lab in labels:
            ids += [label_token] + self._encode(lab)
        ids += self._encode(")") + self._encode(")") + [self.cfg.token_sep_text]
        mask = [0] * len(ids)
        kept = 0
        for wi, (w, _, _) in enumerate(words):
            sub = self._encode(w.lower())
            if len(ids) + len(sub) > self.cfg.max_length:
                break
            ids += sub
            mask += [wi + 1] * len(sub)
            kept = wi + 1
        return GlinerInput(ids[: self.cfg.max_length], mask[: self.cfg.max_length], kept), words

    def _recognize(self, texts: Sequence[str], labels: Sequence[str], label_token: int, threshold: float,
                   flat_ner: bool, batch_size: int = 16) -> List[List[GlinerEntity]]:
        if not labels:
            raise ValueError("no labels given and the model has no default labels")
        prepared = [self.prepare(t, labels, label_token) for t in texts]
        out: List[List[GlinerEntity]] = []
        for lo in range(0, len(prepared), batch_size):
            chunk = prepared[lo:lo + batch_size]
            logits = self.model.span_logits([p[0] for p in chunk], [label_token], self.cfg.max_width)
            for (inp, words), lg, text in zip(chunk, logits, texts[lo:lo + batch_size]):
                out.append(decode_entities(text, words, inp.num_words, lg.cpu(), labels, threshold, flat_ner))
        return out

    def recognize(self, texts: Sequence[str], labels: Optional[Sequence[str]] = None,
                  threshold: Optional[float] = None, flat_ner: Optional[bool] = None) -> List[List[GlinerEntity]]:
        return self._recognize(list(texts), list(labels or self.cfg.default_labels), self.cfg.token_e,
                               self.cfg.threshold if threshold is None else threshold,
                               self.cfg.flat_ner if flat_ner is None else flat_ner)

    def score_labels(self, text: str, labels: Sequence[str]) -> List[float]:
        """One score per label: the sigmoid of the best span logit under the classification marker."""
        token = self.cfg.token_c or self.cfg.token_e
        inp, _ = self.prepare(text, labels, token)
        if inp.num_words == 0:
            return []
        lg = self.model.span_logits([inp], [token], self.cfg.max_width)[0]
        if lg.numel() == 0:
            return [0.0] * len(labels)
        return [_sigmoid(v) for v in lg.reshape(-1, lg.shape[-1]).max(0).values.tolist()]

    def classify(self, text: str, labels: Sequence[str], threshold: float = 0.0, multi_label: bool = False,
                 top_k: int = 0) -> List[Tuple[str, float]]:
        if not text:
            return []
        scored = sorted(((l, s) for l, s in zip(labels, self.score_labels(text, labels)) if s >= threshold),
                        key=lambda p: -p[1])
        if not multi_label and scored:
            return scored[: top_k if top_k > 0 else 1]
        return scored[:top_k] if top_k > 0 else scored

    def extract_relations(self, texts: Sequence[str], entity_labels: Optional[Sequence[str]] = None,
                          relation_labels: Optional[Sequence[str]] = None):
        """(entities per text, relations per text).  Texts with fewer than two entities are not asked about
        relations."""
        ent_labels = list(entity_labels or self.cfg.default_labels)
        ents = self.recognize(texts, ent_labels)
        rels: List[List[GlinerRelation]] = [[] for _ in texts]
        composite = relation_candidates(ent_labels, list(relation_labels or self.cfg.relation_labels))
        active = [i for i, e in enumerate(ents) if len(e) >= 2]
        if composite and active:
            token = self.cfg.token_r or self.cfg.token_e
            thr = self.cfg.relation_threshold if self.cfg.relation_threshold > 0 else self.cfg.threshold
            heads = self._recognize([texts[i] for i in active], composite, token, thr, self.cfg.flat_ner)
            for i, h in zip(active, heads):
                rels[i] = match_relations(ents[i], h)
        return ents, rels
