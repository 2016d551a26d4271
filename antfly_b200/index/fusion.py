"""Result fusion and pruning for hybrid (multi-index) search.

RRF: ``sum_i w_i / (k + rank + 1)`` with rank 0-based and ``rank_constant`` k = 60; RSF: per-index min-max
normalisation over a window, weighted sum; ``failover`` returns the first non-empty list
(zig/pkg/antfly/src/search/fusion.zig:70-200, specs/openapi/antfly/indexes.yaml:388-427).  The pruner implements
min_score_ratio, max_score_gap_percent, min_absolute_score, require_multi_index and std_dev_threshold
(indexes.yaml:428-478).  Scores here are "higher is better"; distances are converted by the caller.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

Hit = Tuple[Hashable, float]  # (doc id, score)


@dataclass
class FusedHit:
    doc_id: Hashable
    score: float
    index_scores: Dict[str, float] = field(default_factory=dict)

    @property
    def index_count(self) -> int:
        return len(self.index_scores)


@dataclass
class MergeConfig:
    strategy: str = "rrf"  # rrf | rsf | failover
    weights: Dict[str, float] = field(default_factory=dict)
    window_size: int = 0
    rank_constant: float = 60.0


@dataclass
class Pruner:
    min_score_ratio: Optional[float] = None
    max_score_gap_percent: Optional[float] = None
    min_absolute_score: Optional[float] = None
    require_multi_index: bool = False
    std_dev_threshold: Optional[float] = None


def _sorted(acc: Dict[Hashable, FusedHit]) -> List[FusedHit]:
    return sorted(acc.values(), key=lambda h: (-h.score, str(h.doc_id)))


def fuse(results: Dict[str, Sequence[Hit]], config: MergeConfig = MergeConfig()) -> List[FusedHit]:
    """results: index name -> hits ranked best first."""
    if config.strategy == "failover":
        for name, hits in results.items():
            if hits:
                return [FusedHit(d, s, {name: s}) for d, s in hits]
        return []
    acc: Dict[Hashable, FusedHit] = {}
    for name, hits in results.items():
        w = config.weights.get(name, 1.0)
        if not hits:
            continue
        if config.strategy == "rrf":
            contrib = [w / (config.rank_constant + r + 1.0) for r in range(len(hits))]
        elif config.strategy == "rsf":
            win = min(config.window_size, len(hits)) if config.window_size > 0 else len(hits)
            ws = [s for _, s in hits[:win]]
            lo, hi = min(ws), max(ws)
            contrib = [w * ((s - lo) / (hi - lo) if hi > lo else 1.0) for _, s in hits]
        else:
            raise ValueError(f"unknown fusion strategy {config.strategy!r}")
        for (doc, s), c in zip(hits, contrib):
            h = acc.setdefault(doc, FusedHit(doc, 0.0))
            h.score += c
            h.index_scores[name] = s
    return _sorted(acc)


def prune(hits: Sequence[FusedHit], p: Pruner) -> List[FusedHit]:
    out = list(hits)
    if not out:
        return out
    if p.require_multi_index:
        out = [h for h in out if h.index_count > 1]
    if p.min_absolute_score is not None:
        out = [h for h in out if h.score >= p.min_absolute_score]
    if out and p.min_score_ratio is not None:
        top = max(h.score for h in out)
        out = [h for h in out if h.score >= top * p.min_score_ratio]
    if out and p.std_dev_threshold is not None and len(out) > 1:
        mean = sum(h.score for h in out) / len(out)
        sd = (sum((h.score - mean) ** 2 for h in out) / len(out)) ** 0.5
        out = [h for h in out if h.score >= mean - p.std_dev_threshold * sd]
    if out and p.max_score_gap_percent is not None and len(out) > 1:
        rng = out[0].score - out[-1].score
        if rng > 0:
            keep = [out[0]]
            for a, b in zip(out, out[1:]):
                if (a.score - b.score) / rng * 100.0 > p.max_score_gap_percent:
                    break
                keep.append(b)
            out = keep
    return out
