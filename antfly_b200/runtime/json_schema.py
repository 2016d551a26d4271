"""JSON Schema -> GBNF grammar, so that a reply can be constrained to documents that validate against a schema
(``response_format: {"type": "json_schema", ...}`` and tool-argument schemas).

Supported: ``type`` (string, number, integer, boolean, null, object, array, or a list of them), ``enum``, ``const``,
``properties`` + ``required`` (properties are emitted in declaration order; optional ones may be left out),
``additionalProperties`` (false / true / schema), ``items``, ``minItems`` / ``maxItems``, ``minLength`` /
``maxLength``, ``anyOf`` / ``oneOf``, ``$ref`` into ``$defs`` / ``definitions`` (recursive schemas become recursive
rules), and the string formats ``date``, ``time``, ``date-time`` and ``uuid``.  Keywords that restrict values
further (``pattern``, numeric ranges, ``uniqueItems`` ...) are ignored: the grammar then accepts a superset.  The
reference validates structured output with its JSON-schema library (zig/lib/jsonschema) next to its grammar engine
(zig/pkg/inference/src/pipelines/grammar.zig); here the schema is compiled into the grammar itself so that invalid
tokens are never sampled.
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Optional

_PRIMS = {
    "ws": r'[ \t\n]*',
    "string": r'"\"" char* "\""',
    "char": r'[^"\\\x00-\x1f] | "\\" (["\\/bfnrt] | "u" hex hex hex hex)',
    "hex": r'[0-9a-fA-F]',
    "integer": r'"-"? ("0" | [1-9] [0-9]*)',
    "number": r'integer ("." [0-9]+)? ([eE] [-+]? [0-9]+)?',
    "boolean": r'"true" | "false"',
    "null": r'"null"',
    "value": r'object | array | string | number | boolean | null',
    "object": r'"{" ws (member (ws "," ws member)*)? ws "}"',
    "member": r'string ws ":" ws value',
    "array": r'"[" ws (value (ws "," ws value)*)? ws "]"',
    "date": r'"\"" [0-9] [0-9] [0-9] [0-9] "-" [0-1] [0-9] "-" [0-3] [0-9] "\""',
    "time": r'"\"" [0-2] [0-9] ":" [0-5] [0-9] ":" [0-5] [0-9] ("." [0-9]+)? ("Z" | [-+] [0-2] [0-9] ":" [0-5] [0-9])? "\""',
    "date-time": r'"\"" [0-9] [0-9] [0-9] [0-9] "-" [0-1] [0-9] "-" [0-3] [0-9] "T" [0-2] [0-9] ":" [0-5] [0-9] ":" '
                 r'[0-5] [0-9] ("." [0-9]+)? ("Z" | [-+] [0-2] [0-9] ":" [0-5] [0-9]) "\""',
    "uuid": r'"\"" hex8 "-" hex4 "-" hex4 "-" hex4 "-" hex4 hex8 "\""',
    "hex4": r'hex hex hex hex',
    "hex8": r'hex4 hex4',
}
_DEPS = {"string": ["char"], "char": ["hex"], "number": ["integer"],
         "value": ["object", "array", "string", "number", "boolean", "null"], "object": ["member", "ws", "string"],
         "member": ["string", "ws", "value"], "array": ["value", "ws"], "uuid": ["hex8", "hex4"], "hex8": ["hex4"],
         "hex4": ["hex"]}


def _literal(v: Any) -> str:
    """GBNF literal matching the JSON encoding of v."""
    text = json.dumps(v, ensure_ascii=False, separators=(",", ":"))
    out = []
    for ch in text:
        if ch == '"':
            out.append('\\"')
        elif ch == "\\":
            out.append("\\\\")
        elif ch == "\n":
            out.append("\\n")
        elif ch == "\r":
            out.append("\\r")
        elif ch == "\t":
            out.append("\\t")
        else:
            out.append(ch)
    return '"' + "".join(out) + '"'


class _Builder:
    def __init__(self, root_schema: Dict[str, Any]):
        self.root_schema = root_schema
        self.rules: Dict[str, str] = {}
        self.refs: Dict[str, str] = {}

    def prim(self, name: str) -> str:
        if name not in self.rules:
            self.rules[name] = _PRIMS[name]
            for d in _DEPS.get(name, []):
                self.prim(d)
        return name

    def fresh(self, hint: str) -> str:
        base = re.sub(r"[^a-zA-Z0-9]+", "-", hint).strip("-").lower() or "r"
        if base in _PRIMS or base == "root":
            base += "-s"
        name, i = base, 1
        while name in self.rules:
            i += 1
            name = f"{base}-{i}"
        self.rules[name] = ""            # reserve (recursive references resolve to the name)
        return name

    def resolve(self, ref: str) -> Dict[str, Any]:
        if not ref.startswith("#/"):
            raise ValueError(f"only local $ref is supported, got {ref!r}")
        node: Any = self.root_schema
        for part in ref[2:].split("/"):
            part = part.replace("~1", "/").replace("~0", "~")
            if not isinstance(node, dict) or part not in node:
                raise ValueError(f"unresolvable $ref {ref!r}")
            node = node[part]
        return node

    def visit(self, schema: Any, hint: str) -> str:
        """Returns a rule name (or an inline expression) matching the schema."""
        if schema is True or schema == {} or schema is None:
            return self.prim("value")
        if schema is False:
            raise ValueError("a schema of `false` matches nothing")
        if "$ref" in schema:
            ref = schema["$ref"]
            if ref not in self.refs:
                name = self.fresh(ref.rsplit("/", 1)[-1])
                self.refs[ref] = name
                self.rules[name] = self.visit(self.resolve(ref), name)
            return self.refs[ref]
        if "const" in schema:
            return _literal(schema["const"])
        if "enum" in schema:
            return "(" + " | ".join(_literal(v) for v in schema["enum"]) + ")"
        for key in ("anyOf", "oneOf"):
            if key in schema:
                alts = [self.visit(s, f"{hint}-{i}") for i, s in enumerate(schema[key])]
                return "(" + " | ".join(alts) + ")"
        t = schema.get("type")
        if isinstance(t, list):
            return "(" + " | ".join(self.visit({**schema, "type": x}, f"{hint}-{x}") for x in t) + ")"
        if t is None:
            t = "object" if "properties" in schema else "array" if "items" in schema else None
        if t == "object":
            return self.obj(schema, hint)
        if t == "array":
            return self.arr(schema, hint)
        if t == "string":
            fmt = schema.get("format")
            if fmt in ("date", "time", "date-time", "uuid"):
                return self.prim(fmt)
            lo, hi = schema.get("minLength"), schema.get("maxLength")
            if lo is not None or hi is not None:
                self.prim("char")
                rep = f"{{{int(lo or 0)},{int(hi)}}}" if hi is not None else f"{{{int(lo or 0)},}}"
                return f'("\\"" char{rep} "\\"")'
            return self.prim("string")
        if t in ("number", "integer", "boolean", "null"):
            return self.prim(t)
        if t is None:
            return self.prim("value")
        raise ValueError(f"unsupported schema type {t!r}")

    def arr(self, schema: Dict[str, Any], hint: str) -> str:
        ws = self.prim("ws")
        item = self.visit(schema.get("items", True), hint + "-item")
        lo, hi = int(schema.get("minItems", 0) or 0), schema.get("maxItems")
        if hi is not None and int(hi) < lo:
            raise ValueError("maxItems < minItems")
        more = f'({ws} "," {ws} {item})'
        if hi is not None and int(hi) == 0:
            body = ""
        elif lo == 0:
            tail = "*" if hi is None else f"{{0,{int(hi) - 1}}}"
            body = f"({item} {more}{tail})?"
        else:
            tail = f"{{{lo - 1},}}" if hi is None else f"{{{lo - 1},{int(hi) - 1}}}"
            body = f"{item} {more}{tail}"
        name = self.fresh(hint + "-arr")
        self.rules[name] = f'"[" {ws} {body} {ws} "]"'
        return name

    def obj(self, schema: Dict[str, Any], hint: str) -> str:
        ws = self.prim("ws")
        props: Dict[str, Any] = schema.get("properties") or {}
        required = set(schema.get("required") or [])
        extra = schema.get("additionalProperties", True if not props else False)
        kv: List[tuple] = []
        for k, sub in props.items():
            kv.append((k in required, f'{_literal(k)} {ws} ":" {ws} {self.visit(sub, f"{hint}-{k}")}'))
        extra_kv: Optional[str] = None
        if extra is not False:
            val = self.visit(extra if isinstance(extra, dict) else True, hint + "-extra")
            extra_kv = f'{self.prim("string")} {ws} ":" {ws} {val}'
        sep = f'{ws} "," {ws}'
        name = self.fresh(hint + "-obj" if hint else "obj")
        # Members in declaration order.  rest(i) = what may follow once at least one member has been written,
        # starting at property i; first(i) = the same before any member (no leading comma).
        n = len(kv)
        rest_names = [self.fresh(f"{name}-rest{i}") for i in range(n + 1)]
        tail = f"({sep} {extra_kv})*" if extra_kv else ""
        self.rules[rest_names[n]] = tail or '""'
        for i in range(n - 1, -1, -1):
            req, member = kv[i]
            take = f"{sep} {member} {rest_names[i + 1]}"
            self.rules[rest_names[i]] = take if req else f"({take}) | {rest_names[i + 1]}"
        first_alts: List[str] = []
        for i in range(n):
            req, member = kv[i]
            first_alts.append(f"{member} {rest_names[i + 1]}")
            if req:
                break
        else:
            if extra_kv:
                first_alts.append(f"{extra_kv} {rest_names[n]}")
            first_alts.append('""')
        self.rules[name] = f'"{{" {ws} ({" | ".join(first_alts)}) {ws} "}}"'
        return name


def json_schema_to_gbnf(schema: Dict[str, Any]) -> str:
    """Compile a JSON Schema into a GBNF grammar whose ``root`` matches exactly one document."""
    b = _Builder(schema)
    body = b.visit(schema, "")
    b.rules["root"] = f"{b.prim('ws')} {body} {b.prim('ws')}"
    order = ["root"] + sorted(k for k in b.rules if k != "root")
    return "\n".join(f"{k} ::= {b.rules[k]}" for k in order) + "\n"
