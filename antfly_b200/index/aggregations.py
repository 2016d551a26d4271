"""Aggregations over the documents a table query matched.

Request and result shapes of specs/openapi/antfly/metadata.yaml (``AggregationRequest``: type, field, size, ranges,
date_ranges, interval, calendar_interval, min_doc_count, sub_aggregations; ``AggregationResult``: value / count / min /
max / sum / sum_of_squares / avg / std_deviation / variance or ``buckets`` of ``AggregationBucket`` with key,
doc_count, from / to and nested sub_aggregations).  Metric types: sum, avg, min, max, count, sumsquares, stats,
cardinality.  Bucket types: terms, range, date_range, histogram, date_histogram.  The geo types and
significant_terms need index structures this table layer does not keep and are refused by name.
"""
from __future__ import annotations

import math
from collections import Counter
from datetime import datetime, timezone
from typing import Dict, Iterable, List, Optional, Sequence

from .docfilter import _get

METRICS = ("sum", "avg", "min", "max", "count", "sumsquares", "stats", "cardinality")
BUCKETS = ("terms", "range", "date_range", "histogram", "date_histogram")


def _numbers(docs: Sequence[dict], field: str) -> List[float]:
    out = []
    for d in docs:
        v = _get(d, field)
        for x in (v if isinstance(v, (list, tuple)) else [v]):
            if isinstance(x, (int, float)) and not isinstance(x, bool):
                out.append(float(x))
    return out


def _values(docs: Sequence[dict], field: str) -> Iterable:
    for d in docs:
        v = _get(d, field)
        if v is None:
            continue
        for x in (v if isinstance(v, (list, tuple)) else [v]):
            yield x


def _parse_time(v) -> Optional[datetime]:
    if isinstance(v, (int, float)) and not isinstance(v, bool):
        return datetime.fromtimestamp(float(v), tz=timezone.utc)
    if not isinstance(v, str):
        return None
    text = v.strip().replace("Z", "+00:00")
    for fmt in (None, "%Y-%m-%d", "%Y-%m", "%Y"):
        try:
            t = datetime.fromisoformat(text) if fmt is None else datetime.strptime(text, fmt)
            return t if t.tzinfo else t.replace(tzinfo=timezone.utc)
        except ValueError:
            continue
    return None


def _metric(kind: str, nums: List[float], docs: Sequence[dict], field: str) -> dict:
    if kind == "count":
        return {"value": float(len(list(_values(docs, field))) if field else len(docs)), "count": len(docs)}
    if kind == "cardinality":
        return {"value": float(len({str(v) for v in _values(docs, field)}))}
    n = len(nums)
    total, sq = sum(nums), sum(x * x for x in nums)
    if kind == "sum":
        return {"value": total}
    if kind == "sumsquares":
        return {"value": sq}
    if kind == "min":
        return {"value": min(nums) if nums else None}
    if kind == "max":
        return {"value": max(nums) if nums else None}
    avg = total / n if n else None
    if kind == "avg":
        return {"value": avg}
    var = (sq / n - avg * avg) if n else None
    return {"count": n, "min": min(nums) if nums else None, "max": max(nums) if nums else None, "sum": total,
            "sum_of_squares": sq, "avg": avg, "variance": max(var, 0.0) if var is not None else None,
            "std_deviation": math.sqrt(max(var, 0.0)) if var is not None else None}


def _with_subs(bucket: dict, members: Sequence[dict], req: dict) -> dict:
    subs = req.get("sub_aggregations")
    if subs:
        bucket["sub_aggregations"] = aggregate(members, subs)
    return bucket


def aggregate(docs: Sequence[dict], requests: Dict[str, dict]) -> Dict[str, dict]:
    out: Dict[str, dict] = {}
    for name, req in (requests or {}).items():
        kind, field = str(req.get("type", "")).lower(), req.get("field") or ""
        min_count = int(req.get("min_doc_count", 0) or 0)
        if kind in METRICS:
            if kind != "count" and not field:
                raise ValueError(f"aggregation {name!r}: {kind} needs a field")
            out[name] = _metric(kind, _numbers(docs, field) if field else [], docs, field)
        elif kind == "terms":
            cnt: Counter = Counter()
            members: Dict[object, list] = {}
            for d in docs:
                v = _get(d, field)
                for x in set(v if isinstance(v, (list, tuple)) else ([] if v is None else [v])):
                    cnt[x] += 1
                    members.setdefault(x, []).append(d)
            size = int(req.get("size", 10) or 10)
            rows = sorted(cnt.items(), key=lambda kv: (-kv[1], str(kv[0])))[:size]
            out[name] = {"buckets": [_with_subs({"key": k, "doc_count": c}, members[k], req)
                                     for k, c in rows if c >= min_count]}
        elif kind in ("range", "date_range"):
            ranges = req.get("ranges" if kind == "range" else "date_ranges") or []
            conv = (lambda v: v if isinstance(v, (int, float)) and not isinstance(v, bool) else None) if kind == "range" \
                else _parse_time
            edge = (lambda v: None if v is None else float(v)) if kind == "range" else (
                lambda v: None if v is None else _parse_time(v))
            buckets = []
            for r in ranges:
                lo, hi = edge(r.get("from")), edge(r.get("to"))
                inside = []
                for d in docs:
                    vals = [conv(x) for x in _values([d], field)]
                    if any(x is not None and (lo is None or x >= lo) and (hi is None or x < hi) for x in vals):
                        inside.append(d)
                b = {"key": r.get("name") or f"{r.get('from', '*')}-{r.get('to', '*')}", "doc_count": len(inside)}
                if r.get("from") is not None:
                    b["from" if kind == "range" else "from_as_string"] = r["from"]
                if r.get("to") is not None:
                    b["to" if kind == "range" else "to_as_string"] = r["to"]
                if len(inside) >= min_count:
                    buckets.append(_with_subs(b, inside, req))
            out[name] = {"buckets": buckets}
        elif kind == "histogram":
            step = float(req.get("interval") or 0)
            if step <= 0:
                raise ValueError(f"aggregation {name!r}: histogram needs a positive interval")
            origin = float(req.get("origin") or 0.0)
            groups: Dict[float, list] = {}
            for d in docs:
                for x in _numbers([d], field):
                    groups.setdefault(origin + math.floor((x - origin) / step) * step, []).append(d)
            out[name] = {"buckets": [_with_subs({"key": k, "doc_count": len(v)}, v, req)
                                     for k, v in sorted(groups.items()) if len(v) >= min_count]}
        elif kind == "date_histogram":
            unit = str(req.get("calendar_interval") or req.get("interval") or "month").lower()
            fmt = {"year": "%Y", "1y": "%Y", "month": "%Y-%m", "1m": "%Y-%m", "day": "%Y-%m-%d", "1d": "%Y-%m-%d",
                   "hour": "%Y-%m-%dT%H", "1h": "%Y-%m-%dT%H"}.get(unit)
            if fmt is None:
                raise ValueError(f"aggregation {name!r}: calendar_interval {unit!r} is not supported")
            groups2: Dict[str, list] = {}
            for d in docs:
                for x in _values([d], field):
                    t = _parse_time(x)
                    if t is not None:
                        groups2.setdefault(t.astimezone(timezone.utc).strftime(fmt), []).append(d)
            out[name] = {"buckets": [_with_subs({"key": k, "key_as_string": k, "doc_count": len(v)}, v, req)
                                     for k, v in sorted(groups2.items()) if len(v) >= min_count]}
        else:
            raise ValueError(f"aggregation {name!r}: type {kind!r} is not supported "
                             f"(supported: {', '.join(METRICS + BUCKETS)})")
    return out
