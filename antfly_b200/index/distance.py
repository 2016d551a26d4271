"""Distance metrics and the search_effort -> index-knob mapping.

All three metrics are "lower is closer" (zig/lib/vector/src/vector.zig:359-376):
``l2_squared = max(0, |a|^2 + |b|^2 - 2ab)``, ``inner_product = -ab``, ``cosine = 1 - ab / (|a||b|)`` (1.0 when a
norm is zero).  A GPU score is always written ``row_term[q] + col_term[x] + scale * <q, x>`` so one GEMM epilogue
serves all of them; cosine indexes store unit-normalised rows and normalise the query.
"""
from __future__ import annotations

from dataclasses import dataclass

METRICS = ("l2_squared", "inner_product", "cosine")


@dataclass
class ScoreForm:
    scale: float
    use_row_norm: bool
    use_col_norm: bool
    row_const: float
    clamp_zero: bool
    normalize: bool


def score_form(metric: str) -> ScoreForm:
    if metric == "l2_squared":
        return ScoreForm(-2.0, True, True, 0.0, True, False)
    if metric == "inner_product":
        return ScoreForm(-1.0, False, False, 0.0, False, False)
    if metric == "cosine":
        return ScoreForm(-1.0, False, False, 1.0, False, True)
    raise ValueError(f"unknown distance metric {metric!r}; expected one of {METRICS}")


def resolve_search_effort(k: int, effort: float, index_size: int = 0):
    """search_effort in [0, 1] -> (search_width, epsilon2), the rule of
    go/pkg/antfly/src/store/db/indexes/embeddings_index.go:563-598: width min = max(k, 64); balanced =
    min + 0.5 * (max(20 * min, 4096) - min); effort <= 0.5 interpolates min -> balanced, above that balanced ->
    a size-aware cap; epsilon2 = 1 + 12 e for e < 0.5 else 7 + 186 (e - 0.5)."""
    e = min(max(float(effort), 0.0), 1.0)
    wmin = max(k, 64)
    wmax = max(20 * wmin, 4096)
    balanced = wmin + 0.5 * (wmax - wmin)
    if e <= 0.5:
        width = wmin + (balanced - wmin) * (e / 0.5)
    else:
        cap = wmax if index_size <= 0 else max(balanced, min(wmax, index_size))
        width = balanced + (cap - balanced) * ((e - 0.5) / 0.5)
    eps2 = 1.0 + 12.0 * e if e < 0.5 else 7.0 + 186.0 * (e - 0.5)
    return int(round(width)), eps2
