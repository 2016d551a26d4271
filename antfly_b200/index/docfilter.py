"""Document predicates for table queries: the ``filter_query`` / ``exclusion_query`` of a query request.

A filter is given as a query string or as a query object (specs/openapi/antfly/metadata.yaml QueryRequest
``filter_query`` -- "status:published", "created_at:>2023-01-01", "+category:technology +language:en" -- and
``exclusion_query`` -- "category:deprecated OR status:archived"; object forms in specs/openapi/antfly/query.yaml:
``{"query": "..."}``, ``{"term", "field"}``, ``{"match", "field"}``, ``{"prefix", "field"}``, ``{"field", "min",
"max"}`` ranges, ``{"conjuncts": [...]}``, ``{"disjuncts": [...]}``, ``{"must" / "should" / "must_not"}``).

Query-string grammar handled here: whitespace-separated clauses ``field:value`` (equality on scalars, membership on
lists, case-insensitive token containment on text), ``field:"a phrase"``, ``field:>v`` ``>=`` ``<`` ``<=`` (numbers
compare numerically, everything else as strings, which orders ISO dates), a leading ``+`` (required) or ``-``
(forbidden), bare words (contained in any string field), and the connectors ``AND`` / ``OR`` between clauses.  As in
the reference's query-string language, clauses without ``+`` / ``-`` are optional: a document passes when every
required clause holds, no forbidden clause holds, and -- if there are no required clauses -- at least one optional
clause holds.  ``a AND b`` makes both required; ``OR`` leaves its neighbours optional.

:func:`compile_filter` turns either form into a function ``document -> bool``.
"""
from __future__ import annotations

import re
from typing import Any, Callable, List, Optional, Tuple

Predicate = Callable[[dict], bool]

_TOKEN = re.compile(r'[+-]?(?:[\w.]+:)?(?:"[^"]*"|\S+)')


def _get(doc: dict, field: str):
    cur: Any = doc
    for part in field.split("."):
        if isinstance(cur, dict) and part in cur:
            cur = cur[part]
        else:
            return None
    return cur


def _num(v) -> Optional[float]:
    if isinstance(v, bool):
        return None
    if isinstance(v, (int, float)):
        return float(v)
    try:
        return float(str(v))
    except ValueError:
        return None


def _compare(value, op: str, ref: str) -> bool:
    if value is None:
        return False
    a, b = _num(value), _num(ref)
    if a is None or b is None:
        a, b = str(value), str(ref)
    return {">": a > b, ">=": a >= b, "<": a < b, "<=": a <= b}[op]


def _matches(value, want: str, phrase: bool) -> bool:
    if value is None:
        return False
    if isinstance(value, (list, tuple, set)):
        return any(_matches(v, want, phrase) for v in value)
    if isinstance(value, bool):
        return str(value).lower() == want.lower()
    if isinstance(value, (int, float)):
        n = _num(want)
        return n is not None and float(value) == n
    text, w = str(value).lower(), want.lower()
    if text == w:
        return True
    if phrase:
        return w in text
    return w in re.findall(r"\w+", text)


def _clause(token: str) -> Tuple[str, Predicate]:
    """-> (kind, predicate) with kind one of "+", "-", "" (optional)."""
    kind = ""
    if token[0] in "+-" and len(token) > 1:
        kind, token = token[0], token[1:]
    field, sep, rest = token.partition(":")
    if not sep or not re.fullmatch(r"[\w.]+", field):
        word = token.strip('"').lower()
        return kind, lambda d: any(isinstance(v, str) and word in v.lower() for v in d.values())
    m = re.match(r"(>=|<=|>|<)(.+)", rest)
    if m:
        op, ref = m.group(1), m.group(2).strip('"')
        return kind, lambda d: _compare(_get(d, field), op, ref)
    phrase = len(rest) >= 2 and rest[0] == '"' and rest[-1] == '"'
    want = rest.strip('"')
    if want.endswith("*") and not phrase:                         # prefix match
        pre = want[:-1].lower()
        return kind, lambda d: isinstance(_get(d, field), str) and str(_get(d, field)).lower().startswith(pre)
    return kind, lambda d: _matches(_get(d, field), want, phrase)


def parse_query_string(text: str) -> Predicate:
    tokens = _TOKEN.findall(text or "")
    must: List[Predicate] = []
    must_not: List[Predicate] = []
    should: List[Predicate] = []
    pending_and = False
    last: Optional[Tuple[str, Predicate]] = None
    for tok in tokens:
        if tok == "AND":
            pending_and = True
            if last is not None and last[0] == "" and last[1] in should:      # promote the left operand
                should.remove(last[1])
                must.append(last[1])
            continue
        if tok == "OR":
            pending_and = False
            continue
        if tok == "NOT":
            last = ("NOT", None)
            continue
        kind, pred = _clause(tok)
        if last is not None and last[0] == "NOT":
            kind = "-"
        if kind == "" and pending_and:
            kind = "+"
        pending_and = False
        (must if kind == "+" else must_not if kind == "-" else should).append(pred)
        last = (kind, pred)
    if not (must or must_not or should):
        return lambda d: True

    def test(d: dict) -> bool:
        if any(p(d) for p in must_not):
            return False
        if not all(p(d) for p in must):
            return False
        return bool(must) or not should or any(p(d) for p in should)

    return test


def compile_filter(q) -> Predicate:
    """A query string, ``{"query": string}`` or a structured query object -> predicate over documents."""
    if q is None or q == "" or q == {}:
        return lambda d: True
    if isinstance(q, str):
        return parse_query_string(q)
    if not isinstance(q, dict):
        raise ValueError(f"unsupported filter {q!r}")
    if "query" in q and isinstance(q["query"], str):
        return parse_query_string(q["query"])
    if "conjuncts" in q:
        parts = [compile_filter(x) for x in q["conjuncts"]]
        return lambda d: all(p(d) for p in parts)
    if "disjuncts" in q:
        parts = [compile_filter(x) for x in q["disjuncts"]]
        need = int(q.get("min", 1) or 1)
        return lambda d: sum(1 for p in parts if p(d)) >= need
    if any(k in q for k in ("must", "should", "must_not")):
        sub = lambda k: compile_filter(q[k]) if isinstance(q.get(k), dict) else None
        must, should, must_not = sub("must"), sub("should"), sub("must_not")
        return lambda d: (must is None or must(d)) and (must_not is None or not must_not(d)) and \
            (should is None or must is not None or should(d))
    field = q.get("field")
    if "term" in q and field:
        want = q["term"]
        return lambda d: _matches(_get(d, field), str(want), True) and (
            not isinstance(_get(d, field), str) or str(_get(d, field)).lower() == str(want).lower())
    if "match" in q and field:
        words = re.findall(r"\w+", str(q["match"]))
        return lambda d: any(_matches(_get(d, field), w, False) for w in words)
    if "match_phrase" in q and field:
        want = str(q["match_phrase"])
        return lambda d: _matches(_get(d, field), want, True)
    if "prefix" in q and field:
        pre = str(q["prefix"]).lower()
        return lambda d: isinstance(_get(d, field), str) and _get(d, field).lower().startswith(pre)
    if "bool" in q and field:
        want = bool(q["bool"])
        return lambda d: _get(d, field) is want
    if field and ("min" in q or "max" in q or "start" in q or "end" in q):
        lo, hi = q.get("min", q.get("start")), q.get("max", q.get("end"))
        lo_op = ">=" if q.get("inclusive_min", q.get("inclusive_start", True)) else ">"
        hi_op = "<=" if q.get("inclusive_max", q.get("inclusive_end", False)) else "<"
        return lambda d: (lo is None or _compare(_get(d, field), lo_op, str(lo))) and \
            (hi is None or _compare(_get(d, field), hi_op, str(hi)))
    if "match_all" in q:
        return lambda d: True
    if "match_none" in q:
        return lambda d: False
    raise ValueError(f"unsupported filter object with keys {sorted(q)}")
