"""After extraction: merge the mentions found across texts into entities and relations of one knowledge graph,
and clean a mention list by validity and embedding similarity.

Knowledge graph (zig/pkg/inference/src/pipelines/resolver.zig:107-438): mentions whose normalised texts are similar
(Jaro-Winkler, lifted to ``0.7 + 0.3 * len ratio`` when every word of the shorter name occurs in the longer one)
and whose labels agree form one entity; its canonical name is the longest mention (ties: the best score), its score
the best mention score.  A relation's ends are looked up among the mentions (exact normalised text first, else the
most similar above the threshold); relations with the same ends and label merge, keeping the best score and the
union of the texts they came from, and are listed in (head, tail, label) order.

Cleanup (zig/pkg/inference/src/pipelines/entity_cleanup.zig:110-270): mentions below a validity score are dropped
(and reported); the rest are clustered transitively by the cosine similarity of their embeddings -- one similarity
matrix from a single GEMM on the embeddings' device -- and each cluster is represented by its best mention
(representative score, then validity, then detection score).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# -- string similarity ------------------------------------------------------------------------------------------
def jaro(a: str, b: str) -> float:
    if a == b:
        return 1.0
    if not a or not b:
        return 0.0
    reach = max(max(len(a), len(b)) // 2 - 1, 0)
    am, bm = [False] * len(a), [False] * len(b)
    m = 0
    for i, ch in enumerate(a):
        for j in range(max(0, i - reach), min(len(b), i + reach + 1)):
            if not bm[j] and b[j] == ch:
                am[i] = bm[j] = True
                m += 1
                break
    if m == 0:
        return 0.0
    t, j = 0, 0
    for i, ch in enumerate(a):
        if not am[i]:
            continue
        while j < len(b) and not bm[j]:
            j += 1
        if j < len(b) and ch != b[j]:
            t += 1
        j += 1
    return (m / len(a) + m / len(b) + (m - t / 2.0) / m) / 3.0


def jaro_winkler(a: str, b: str) -> float:
    if a == b:
        return 1.0
    if not a or not b:
        return 0.0
    j = jaro(a, b)
    p = 0
    while p < min(len(a), len(b), 4) and a[p] == b[p]:
        p += 1
    return j + p * 0.1 * (1.0 - j)


def entity_similarity(a: str, b: str) -> float:
    """Similarity of two normalised names (compared as UTF-8 bytes, like the reference)."""
    if a == b:
        return 1.0
    if not a or not b:
        return 0.0
    ab, bb = a.encode("utf-8"), b.encode("utf-8")
    jw = jaro_winkler(ab.decode("latin-1"), bb.decode("latin-1"))
    short, long_ = (a, b) if len(ab) <= len(bb) else (b, a)
    st, lt = short.split(), long_.split()
    if st and lt and all(w in lt for w in st):
        ratio = len(short.encode("utf-8")) / len(long_.encode("utf-8"))
        return max(0.7 + 0.3 * ratio, jw)
    return jw


def normalize_name(text: str) -> str:
    return "".join(c.lower() if c.isascii() else c for c in text.strip(" \t\r\n"))


# -- knowledge graph ----------------------------------------------------------------------------------------------
@dataclass
class ResolverConfig:
    similarity_threshold: float = 0.85
    type_must_match: bool = True
    min_entity_confidence: float = 0.0
    min_relation_confidence: float = 0.0
    deduplicate_relations: bool = True
    track_provenance: bool = True


@dataclass
class ResolvedEntity:
    id: str
    canonical_name: str
    label: str
    score: float
    mentions: Optional[List[str]] = None
    text_indices: Optional[List[int]] = None


@dataclass
class ResolvedRelation:
    head_id: str
    tail_id: str
    label: str
    score: float
    text_indices: Optional[List[int]] = None


@dataclass
class KnowledgeGraph:
    entities: List[ResolvedEntity]
    relations: List[ResolvedRelation]


def build_knowledge_graph(entities_by_text: Sequence[Sequence], relations_by_text: Optional[Sequence[Sequence]] = None,
                          cfg: Optional[ResolverConfig] = None) -> KnowledgeGraph:
    """``entities_by_text[i]`` are the mentions of text ``i`` (objects with ``text``, ``label``, ``score``);
    ``relations_by_text[i]`` its relations (``head`` / ``tail`` mentions, ``label``, ``score``)."""
    cfg = cfg or ResolverConfig()
    ents = [(e, ti) for ti, es in enumerate(entities_by_text) for e in es if e.score >= cfg.min_entity_confidence]
    norm = [normalize_name(e.text) for e, _ in ents]
    assign = [-1] * len(ents)
    clusters: List[List[int]] = []
    for i, (e, _) in enumerate(ents):
        if assign[i] >= 0:
            continue
        assign[i] = len(clusters)
        members = [i]
        for j in range(i + 1, len(ents)):
            if assign[j] >= 0 or (cfg.type_must_match and ents[j][0].label != e.label):
                continue
            if entity_similarity(norm[i], norm[j]) >= cfg.similarity_threshold:
                assign[j] = len(clusters)
                members.append(j)
        clusters.append(members)
    resolved: List[ResolvedEntity] = []
    refs: List[Tuple[str, str, str]] = []                      # (normalised text, label, entity id)
    for ci, members in enumerate(clusters):
        best = members[0]
        for k in members:
            e, b = ents[k][0], ents[best][0]
            if len(e.text.encode()) > len(b.text.encode()) or (len(e.text.encode()) == len(b.text.encode())
                                                                and e.score > b.score):
                best = k
        mentions, seen, texts = [], set(), []
        for k in members:
            if norm[k] not in seen:
                seen.add(norm[k])
                mentions.append(ents[k][0].text)
            if ents[k][1] not in texts:
                texts.append(ents[k][1])
        rid = f"entity-{ci}"
        resolved.append(ResolvedEntity(rid, ents[best][0].text, ents[best][0].label,
                                       max(ents[k][0].score for k in members),
                                       mentions if cfg.track_provenance else None,
                                       texts if cfg.track_provenance else None))
        refs += [(norm[k], ents[k][0].label, rid) for k in members]

    def lookup(m) -> str:
        n = normalize_name(m.text)
        for t, lab, rid in refs:
            if (not cfg.type_must_match or lab == m.label) and t == n:
                return rid
        best_s, best_id = 0.0, ""
        for t, lab, rid in refs:
            if cfg.type_must_match and lab != m.label:
                continue
            s = entity_similarity(n, t)
            if s >= cfg.similarity_threshold and s > best_s:
                best_s, best_id = s, rid
        return best_id

    rels: List[ResolvedRelation] = []
    for ti, rs in enumerate(relations_by_text or []):
        for r in rs:
            if r.score < cfg.min_relation_confidence:
                continue
            h, t = lookup(r.head), lookup(r.tail)
            if h and t:
                rels.append(ResolvedRelation(h, t, r.label, r.score, [ti]))
    if cfg.deduplicate_relations:
        merged: Dict[Tuple[str, str, str], ResolvedRelation] = {}
        for r in rels:
            k = (r.head_id, r.tail_id, r.label)
            if k in merged:
                m = merged[k]
                m.score = max(m.score, r.score)
                m.text_indices += [i for i in r.text_indices if i not in m.text_indices]
            else:
                merged[k] = ResolvedRelation(r.head_id, r.tail_id, r.label, r.score, list(r.text_indices))
        rels = sorted(merged.values(), key=lambda r: (r.head_id, r.tail_id, r.label))
    return KnowledgeGraph(resolved, rels)


# -- mention cleanup ------------------------------------------------------------------------------------------------
@dataclass
class CleanupConfig:
    min_validity_score: float = 0.5
    dedup_similarity_threshold: float = 0.9
    type_must_match: bool = True
    track_provenance: bool = True


@dataclass
class CleanupMention:
    entity: object                      # text, label, start, end, score
    validity_score: float
    representative_score: float
    embedding: torch.Tensor             # [dim]


@dataclass
class CleanedEntity:
    id: str
    text: str
    label: str
    start: int
    end: int
    detect_score: float
    validity_score: float
    representative_score: float
    mentions: Optional[List[str]] = None


@dataclass
class CleanupResult:
    resolved_entities: List[CleanedEntity]
    dropped_mentions: List[dict] = field(default_factory=list)


def cleanup_mentions(mentions: Sequence[CleanupMention], cfg: Optional[CleanupConfig] = None) -> CleanupResult:
    cfg = cfg or CleanupConfig()
    dropped = [{"text": m.entity.text, "label": m.entity.label, "start": m.entity.start, "end": m.entity.end,
                "detect_score": m.entity.score, "validity_score": m.validity_score}
               for m in mentions if m.validity_score < cfg.min_validity_score]
    kept = [i for i, m in enumerate(mentions) if m.validity_score >= cfg.min_validity_score]
    if not kept:
        return CleanupResult([], dropped)
    E = torch.stack([mentions[i].embedding.float() for i in kept])
    nrm = E.norm(dim=-1, keepdim=True)
    sim = (E / nrm.clamp(min=1e-30)) @ (E / nrm.clamp(min=1e-30)).T         # one GEMM for all pairs
    sim = torch.where((nrm > 0) & (nrm.T > 0), sim, torch.zeros_like(sim))
    link = (sim >= cfg.dedup_similarity_threshold).cpu()
    if cfg.type_must_match:
        labs = [mentions[i].entity.label for i in kept]
        same = torch.tensor([[a == b for b in labs] for a in labs])
        link &= same
    assign = [-1] * len(kept)
    clusters: List[List[int]] = []
    for s in range(len(kept)):
        if assign[s] >= 0:
            continue
        assign[s] = len(clusters)
        members, cur = [s], 0
        while cur < len(members):                 # transitive: every member's neighbours join, in index order
            for o in torch.nonzero(link[members[cur]]).flatten().tolist():
                if assign[o] < 0:
                    assign[o] = len(clusters)
                    members.append(o)
            cur += 1
        clusters.append(members)
    out: List[CleanedEntity] = []
    for ci, members in enumerate(clusters):
        key = lambda k: (mentions[kept[k]].representative_score, mentions[kept[k]].validity_score,
                         mentions[kept[k]].entity.score)
        best = members[0]
        for k in members[1:]:
            if key(k) > key(best):
                best = k
        m = mentions[kept[best]]
        out.append(CleanedEntity(f"cleanup-entity-{ci}", m.entity.text, m.entity.label, m.entity.start, m.entity.end,
                                 m.entity.score, m.validity_score, m.representative_score,
                                 [mentions[kept[k]].entity.text for k in members] if cfg.track_provenance else None))
    return CleanupResult(out, dropped)
