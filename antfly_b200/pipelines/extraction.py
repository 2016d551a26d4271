"""Structured extraction: a schema of named structures with typed fields is answered by a zero-shot span model.

What the reference does (zig/pkg/inference/src/pipelines/extraction.zig:272-384 field definitions and
extractStructure, :528-650 assembleInstances / buildInstance, :906-940 cluster threshold):

* A field is ``name``, ``name::str``, ``name::list`` or ``name::[a|b|c]::str`` (a choice field); in the request's
  canonical form a field maps to ``"str"`` / ``"list"`` or an object with ``type`` (and optionally ``choices``).
* The field names are the span model's labels.  Spans of a choice field are reduced to the best one, whose text is
  replaced by the matching choice (case-insensitive equality, else the best label of a classification of the span
  text over the choices).
* Spans are sorted by position and cut into *instances* where the gap between neighbours exceeds a threshold:
  three times the median gap, but at least min(100, text length / 10) characters (or a fixed ``cluster_gap``).
  Within an instance a ``str`` field takes its best-scoring span, a ``list`` field all of its spans.
* Values are ``{"value": ...}`` with ``score`` and ``start`` / ``end`` when asked for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


@dataclass
class SchemaField:
    name: str
    is_list: bool = False
    choices: List[str] = field(default_factory=list)


@dataclass
class ExtractionConfig:
    threshold: float = 0.3
    flat_ner: bool = True
    include_confidence: bool = False
    include_spans: bool = False
    cluster_gap: int = 0


_TYPES = {"str": False, "string": False, "list": True, "array": True}


def parse_field_def(text: str) -> SchemaField:
    """``"role::[engineer|manager]::str"`` -> SchemaField; type and choice specifiers are read from the right, what
    is left (rejoined with ``::``) is the name."""
    parts = [p.strip() for p in text.strip().split("::")]
    if not text.strip():
        raise ValueError("empty field definition")
    out = SchemaField("")
    end = len(parts)
    i = len(parts)
    while i > 1:
        i -= 1
        p = parts[i]
        if len(p) >= 2 and p[0] == "[" and p[-1] == "]":
            choices = [c.strip() for c in p[1:-1].split("|")]
            if any(not c for c in choices):
                raise ValueError("empty choice value")
            if len(choices) < 2:
                raise ValueError("a choice field needs at least two choices")
            out.choices, end = choices, i
            continue
        if p.lower() in _TYPES:
            out.is_list, end = _TYPES[p.lower()], i
            continue
        break
    out.name = "::".join(parts[:end])
    if not out.name:
        raise ValueError("empty field name")
    return out


def canonical_structures(structures: Dict[str, object]) -> Dict[str, List[SchemaField]]:
    """The request's ``schema.structures`` ({name: {fields: {field: "str" | "list" | {type, choices}}}} or the short
    form {name: ["field::type", ...]}) -> {name: [SchemaField]}."""
    out: Dict[str, List[SchemaField]] = {}
    for name, spec in structures.items():
        name = str(name).strip()
        if not name:
            raise ValueError("empty structure name")
        if isinstance(spec, (list, tuple)):
            fields = [parse_field_def(str(f)) for f in spec]
        else:
            fmap = (spec or {}).get("fields") if isinstance(spec, dict) else None
            if not fmap:
                raise ValueError(f"structure {name!r} has no fields")
            fields = []
            for fname, ftype in fmap.items():
                fname = str(fname).strip()
                if not fname:
                    raise ValueError("empty field name")
                if isinstance(ftype, dict):
                    f = SchemaField(fname, str(ftype.get("type", "str")).lower() in ("list", "array"),
                                    [str(c) for c in ftype.get("choices") or []])
                else:
                    f = SchemaField(fname, str(ftype).lower() in ("list", "array"))
                fields.append(f)
        if not fields:
            raise ValueError(f"structure {name!r} has no fields")
        out[name] = fields
    return out


def cluster_threshold(spans: Sequence[dict], cluster_gap: int, text_length: int) -> int:
    if cluster_gap > 0:
        return cluster_gap
    if len(spans) <= 1:
        return 0
    gaps = sorted(max(b["start"] - a["end"], 0) for a, b in zip(spans, spans[1:]))
    mid = len(gaps) // 2
    median = gaps[mid - 1] if len(gaps) % 2 == 0 else gaps[mid]
    return max(median * 3, min(100, text_length // 10))


def _value(span: dict, cfg: ExtractionConfig) -> dict:
    v = {"value": span["text"]}
    if cfg.include_confidence:
        v["score"] = span["score"]
    if cfg.include_spans:
        v["start"], v["end"] = span["start"], span["end"]
    return v


def build_instance(fields: Sequence[SchemaField], spans: Sequence[dict], cfg: ExtractionConfig) -> dict:
    inst: dict = {}
    for f in fields:
        mine = [s for s in spans if s["label"] == f.name]
        if not mine:
            continue
        if f.is_list:
            inst[f.name] = [_value(s, cfg) for s in mine]
        else:
            best = mine[0]
            for s in mine[1:]:
                if s["score"] > best["score"]:
                    best = s
            inst[f.name] = _value(best, cfg)
    return inst


def assemble_instances(fields: Sequence[SchemaField], spans: Sequence[dict], cfg: ExtractionConfig,
                       text_length: int) -> List[dict]:
    if not spans:
        return []
    spans = sorted(spans, key=lambda s: (s["start"], s["end"]))
    if len(spans) == 1:
        inst = build_instance(fields, spans, cfg)
        return [inst] if inst else []
    thr = cluster_threshold(spans, cfg.cluster_gap, text_length)
    out, first = [], 0
    for i in range(len(spans) - 1):
        if max(spans[i + 1]["start"] - spans[i]["end"], 0) > thr:
            inst = build_instance(fields, spans[first:i + 1], cfg)
            if inst:
                out.append(inst)
            first = i + 1
    tail = build_instance(fields, spans[first:], cfg)
    if tail:
        out.append(tail)
    if not out:
        inst = build_instance(fields, spans, cfg)
        if inst:
            out.append(inst)
    return out


def extract_structures(pipe, text: str, structures: Dict[str, List[SchemaField]],
                       cfg: Optional[ExtractionConfig] = None) -> Dict[str, List[dict]]:
    """``pipe``: a zero-shot span pipeline with ``recognize(texts, labels, threshold=)`` (entities with byte offsets
    ``start`` / ``end``, ``label``, ``text``, ``score``) and ``classify(text, labels, ...)``."""
    cfg = cfg or ExtractionConfig()
    raw = text.encode("utf-8")
    out: Dict[str, List[dict]] = {}
    for name, fields in structures.items():
        ents = pipe.recognize([text], [f.name for f in fields], threshold=cfg.threshold)[0]
        spans: List[dict] = []
        for f in fields:
            mine = [e for e in ents if e.label == f.name]
            if not mine:
                continue
            if f.choices:
                best = mine[0]
                for e in mine[1:]:
                    if e.score > best.score:
                        best = e
                chosen, score = None, best.score
                for c in f.choices:
                    if c.lower() == best.text.lower():
                        chosen = c
                        break
                if chosen is None:
                    ranked = pipe.classify(best.text, f.choices, threshold=0.0, multi_label=False)
                    chosen, score = (ranked[0][0], float(ranked[0][1])) if ranked else (best.text, best.score)
                mine, texts = [best], {id(best): chosen}
                scores = {id(best): score}
            else:
                texts, scores = {}, {}
            for e in mine:
                start = len(raw[: e.start].decode("utf-8", "replace"))           # character offsets from byte offsets
                spans.append({"label": f.name, "text": texts.get(id(e), e.text), "start": start,
                              "end": start + len(e.text), "score": float(scores.get(id(e), e.score))})
        out[name] = assemble_instances(fields, spans, cfg, len(text))
    return out
