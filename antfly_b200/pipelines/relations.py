"""Relation extraction with a sequence-to-sequence model that writes triplets as text (REBEL and its derivatives).

The model linearises relations as ``<triplet> head <subj> tail <obj> relation``; further tails of the same head
continue with ``<subj> tail <obj> relation``, a new head starts with another ``<triplet>``.  The parser below is
the state machine that reads this back (the reference's version: zig/pkg/inference/src/pipelines/rebel.zig);
entities are de-duplicated and relations refer to them by index, which is the shape of the extraction API's
``relations`` (source / target ``entity_index``).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

_MARK = re.compile(r"(<triplet>|<subj>|<obj>)")
_DROP = re.compile(r"</?s>|<pad>")


@dataclass
class Triplet:
    head: str
    relation: str
    tail: str


def parse_triplets(text: str) -> List[Triplet]:
    """Linearised triplets -> list of (head, relation, tail); incomplete trailing pieces are dropped."""
    out: List[Triplet] = []
    head = tail = rel = ""
    state = None                      # which field the next text span fills
    for piece in _MARK.split(_DROP.sub("", text)):
        if piece == "<triplet>":
            if head.strip() and rel.strip() and tail.strip():
                out.append(Triplet(head.strip(), rel.strip(), tail.strip()))
            head = tail = rel = ""
            state = "head"
        elif piece == "<subj>":
            if head.strip() and rel.strip() and tail.strip():
                out.append(Triplet(head.strip(), rel.strip(), tail.strip()))
            tail = rel = ""
            state = "tail"
        elif piece == "<obj>":
            rel = ""
            state = "rel"
        elif state == "head":
            head += piece
        elif state == "tail":
            tail += piece
        elif state == "rel":
            rel += piece
    if head.strip() and rel.strip() and tail.strip():
        out.append(Triplet(head.strip(), rel.strip(), tail.strip()))
    seen, uniq = set(), []
    for t in out:
        k = (t.head, t.relation, t.tail)
        if k not in seen:
            seen.add(k)
            uniq.append(t)
    return uniq


def to_extraction(triplets: Sequence[Triplet], text: str = "", allowed: Optional[Sequence[str]] = None
                  ) -> Tuple[List[dict], List[dict]]:
    """(entities, relations) in the extraction API's shape; ``allowed`` keeps only the listed relation types
    (compared case-insensitively).  Entity spans are located in ``text`` when they occur there."""
    keep = {a.lower() for a in allowed} if allowed else None
    ents: List[dict] = []
    index: Dict[str, int] = {}

    def ent(name: str) -> int:
        if name not in index:
            e = {"label": "entity", "text": name}
            at = text.lower().find(name.lower()) if text else -1
            if at >= 0:
                e["start"], e["end"] = at, at + len(name)
            index[name] = len(ents)
            ents.append(e)
        return index[name]

    rels = []
    for t in triplets:
        if keep is not None and t.relation.lower() not in keep:
            continue
        rels.append({"type": t.relation, "source": {"entity_index": ent(t.head)},
                     "target": {"entity_index": ent(t.tail)}})
    return ents, rels


class RelationExtractor:
    def __init__(self, seq2seq_pipeline, max_new_tokens: int = 256):
        self.pipe, self.max_new_tokens = seq2seq_pipeline, max_new_tokens

    def extract(self, text: str, allowed: Optional[Sequence[str]] = None) -> Tuple[List[dict], List[dict]]:
        from ..runtime.sampling_params import SamplingParams

        out = self.pipe.generate(text, SamplingParams(max_tokens=self.max_new_tokens), raw_prompt=True,
                                 keep_special=True)
        return to_extraction(parse_triplets(out.text), text, allowed)
