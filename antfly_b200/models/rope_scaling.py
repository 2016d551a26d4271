"""Frequency tables for rotary position embeddings with context-extension schemes.

The plain rotary frequencies are ``theta ** (-2 j / rope_dim)`` and the kernels compute them on the fly.  Checkpoints
trained or extended for long contexts declare a scheme in ``rope_scaling`` / ``rope_parameters`` that changes the
frequencies per pair, and sometimes scales cos / sin by an attention factor:

* ``linear``: every frequency divided by ``factor`` -- a scalar the kernels already take (``freq_scale``); this is the
  one scheme the reference reads (zig/pkg/inference/src/models/gpt.zig:901-912).
* ``llama3`` (Llama 3.1 / 3.2): wavelengths longer than ``original / low_freq_factor`` are divided by ``factor``,
  shorter than ``original / high_freq_factor`` are kept, the band between is blended linearly in
  ``original / wavelength``.
* ``yarn``: per-pair blend of interpolated (``1 / factor``) and original frequencies with a linear ramp between the
  correction dimensions of ``beta_fast`` and ``beta_slow`` rotations over the original context; cos / sin scaled by
  ``0.1 ln(factor) + 1`` (or the ratio of the two ``mscale`` forms).
* ``longrope`` (Phi-3 long): per-pair divisors ``short_factor`` / ``long_factor`` and an attention factor
  ``sqrt(1 + ln(scale) / ln(original))``.  The short factors serve contexts up to the original length, the long
  ones beyond it; a serving process decides once, from the context length it is configured for.
* ``factors``: per-pair divisors given outright (the ``rope_freqs.weight`` tensor of a GGUF file).

:func:`rope_frequencies` returns ``(inv_freq, attention_factor)`` with ``inv_freq`` ``None`` when the plain formula
(with ``freq_scale``) applies, so the default models keep their on-the-fly path.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple


def _base(theta: float, rope_dim: int) -> List[float]:
    return [theta ** (-2.0 * j / rope_dim) for j in range(rope_dim // 2)]


def llama3_frequencies(theta: float, rope_dim: int, factor: float, low_freq_factor: float, high_freq_factor: float,
                       original_max_position: int) -> List[float]:
    low_wavelen = original_max_position / low_freq_factor
    high_wavelen = original_max_position / high_freq_factor
    out = []
    for f in _base(theta, rope_dim):
        wavelen = 2.0 * math.pi / f
        if wavelen > low_wavelen:
            out.append(f / factor)
        elif wavelen < high_wavelen:
            out.append(f)
        else:
            smooth = (original_max_position / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


def _yarn_mscale(scale: float, m: float = 1.0) -> float:
    return 1.0 if scale <= 1.0 else 0.1 * m * math.log(scale) + 1.0


def yarn_frequencies(theta: float, rope_dim: int, factor: float, original_max_position: int, beta_fast: float = 32.0,
                     beta_slow: float = 1.0, truncate: bool = True) -> List[float]:
    def correction_dim(rotations: float) -> float:
        return rope_dim * math.log(original_max_position / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))

    low, high = correction_dim(beta_fast), correction_dim(beta_slow)
    if truncate:
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, rope_dim - 1)
    if low == high:
        high += 0.001                                                    # keeps the ramp finite
    out = []
    for j, f in enumerate(_base(theta, rope_dim)):
        ramp = min(max((j - low) / (high - low), 0.0), 1.0)
        keep = 1.0 - ramp                                                # 1: original frequency, 0: interpolated
        out.append((f / factor) * (1.0 - keep) + f * keep)
    return out


def rope_frequencies(rope: Optional[dict], theta: float, rope_dim: int, max_position: int = 0,
                     serve_context: int = 0) -> Tuple[Optional[List[float]], float]:
    """``rope``: the checkpoint's ``rope_scaling`` / ``rope_parameters`` dictionary (or None).  ``max_position``: the
    configuration's ``max_position_embeddings``; ``serve_context``: the longest context this process will serve
    (0 = up to the original length), which picks ``longrope``'s factor set."""
    if not rope:
        return None, 1.0
    kind = rope.get("rope_type", rope.get("type")) or "default"
    factor = float(rope.get("factor") or 1.0)
    original = int(rope.get("original_max_position_embeddings") or max_position or 0)
    if kind == "llama3":
        return llama3_frequencies(theta, rope_dim, factor, float(rope.get("low_freq_factor", 1.0)),
                                  float(rope.get("high_freq_factor", 4.0)), original), 1.0
    if kind == "yarn":
        if rope.get("original_max_position_embeddings") and max_position and not rope.get("factor"):
            factor = max_position / original
        att = rope.get("attention_factor")
        if att is None:
            ms, ms_all = rope.get("mscale"), rope.get("mscale_all_dim")
            att = _yarn_mscale(factor, ms) / _yarn_mscale(factor, ms_all) if ms and ms_all else _yarn_mscale(factor)
        inv = yarn_frequencies(theta, rope_dim, factor, original, float(rope.get("beta_fast") or 32.0),
                               float(rope.get("beta_slow") or 1.0), rope.get("truncate", True) is not False)
        return inv, float(att)
    if kind in ("longrope", "su"):
        short, long_ = rope.get("short_factor"), rope.get("long_factor")
        if not short or not long_:
            raise ValueError("longrope needs short_factor and long_factor")
        scale = max_position / original if original and max_position else factor
        att = rope.get("attention_factor")
        if att is None:
            att = 1.0 if scale <= 1.0 else math.sqrt(1.0 + math.log(scale) / math.log(original))
        div = long_ if serve_context > original > 0 else short
        if len(div) != rope_dim // 2:
            raise ValueError(f"longrope factors have {len(div)} entries, expected {rope_dim // 2}")
        return [f / float(d) for f, d in zip(_base(theta, rope_dim), div)], float(att)
    if kind == "factors":                                                # a file's own per-pair divisors
        div = rope.get("factors") or []
        if len(div) != rope_dim // 2:
            raise ValueError(f"rope factors have {len(div)} entries, expected {rope_dim // 2}")
        return [f / float(d) for f, d in zip(_base(theta, rope_dim), div)], float(rope.get("attention_factor") or 1.0)
    return None, 1.0                                                     # default / linear: the scalar path
