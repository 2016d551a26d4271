"""Tool calling: rendering tool definitions into the prompt and parsing tool calls out of the model's reply,
incrementally while tokens stream.

Formats (picked from the model directory's chat template / tokens, or named explicitly):

* ``hermes``   -- ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (Hermes, Qwen)
* ``gemma``    -- ``<|tool_call>call:NAME{key:value,...}<tool_call|>`` with ``<|tool>`` declarations, the function
                  format the reference parses (zig/pkg/inference/src/pipelines/tool_parser.zig:82-90, :1213-1272)
* ``mistral``  -- ``[TOOL_CALLS] [{"name": ..., "arguments": {...}}, ...]``
* ``llama3``   -- the whole reply (optionally after ``<|python_tag|>``) is one JSON object with ``name`` and
                  ``parameters`` / ``arguments``

The parser is fed text chunks (``feed``) and separates them into user-visible content and tool-call payloads
without ever emitting a partial start marker as content; ``finish`` returns the calls in OpenAI shape
(``{"id", "type": "function", "function": {"name", "arguments": <JSON string>}}``).  ``tool_choice`` follows the
OpenAI contract: ``none`` / ``auto`` / ``required`` / ``{"type": "function", "function": {"name": ...}}``.
"""
from __future__ import annotations

import itertools
import json
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

_counter = itertools.count(1)

FORMATS = {
    "hermes": ("<tool_call>", "</tool_call>"),
    "gemma": ("<|tool_call>", "<tool_call|>"),
    "mistral": ("[TOOL_CALLS]", None),
    "llama3": ("<|python_tag|>", None),
}


@dataclass
class ToolChoice:
    mode: str = "auto"            # none | auto | required | function
    function: Optional[str] = None

    @property
    def enabled(self) -> bool:
        return self.mode != "none"


def parse_tool_choice(choice: Any) -> ToolChoice:
    if choice is None:
        return ToolChoice("auto")
    if isinstance(choice, str):
        if choice in ("none", "auto", "required"):
            return ToolChoice(choice)
        raise ValueError(f"tool_choice must be none, auto, required or a function object (got {choice!r})")
    if isinstance(choice, dict) and choice.get("type") == "function":
        name = (choice.get("function") or {}).get("name")
        if not name:
            raise ValueError("tool_choice.function.name is required")
        return ToolChoice("function", name)
    raise ValueError("unrecognised tool_choice")


def detect_format(chat_template: Optional[str], vocab_tokens: Optional[List[str]] = None) -> str:
    hay = (chat_template or "") + " ".join(vocab_tokens or [])
    if "<|tool_call>" in hay:
        return "gemma"
    if "[TOOL_CALLS]" in hay:
        return "mistral"
    if "<|python_tag|>" in hay:
        return "llama3"
    return "hermes"


def format_tools_prompt(tools: List[Dict[str, Any]], fmt: str = "hermes", choice: Optional[ToolChoice] = None) -> str:
    """System-prompt text that declares the tools and the call syntax (used when the chat template has no tools
    section of its own)."""
    choice = choice or ToolChoice()
    fns = [t.get("function", t) for t in tools]
    if fmt == "gemma":
        decl = "".join(f"<|tool>{f['name']}{json.dumps(f.get('parameters') or {}, separators=(',', ':'))}<tool|>"
                       for f in fns)
        how = "To call a tool reply with <|tool_call>call:function_name{argument:value}<tool_call|>."
    else:
        decl = "\n".join(json.dumps({"type": "function", "function": f}, separators=(",", ":")) for f in fns)
        start, end = FORMATS.get(fmt, FORMATS["hermes"])
        if fmt == "hermes":
            how = ('To call a tool reply with <tool_call>{"name": <function-name>, "arguments": <args-json-object>}'
                   "</tool_call>.")
        elif fmt == "mistral":
            how = 'To call tools reply with [TOOL_CALLS] [{"name": <function-name>, "arguments": <args-json-object>}].'
        else:
            how = 'To call a tool reply with only {"name": <function-name>, "parameters": <args-json-object>}.'
    must = ""
    if choice.mode == "required":
        must = " You must call at least one tool."
    elif choice.mode == "function":
        must = f" You must call the tool {choice.function}."
    return f"You have access to these tools:\n{decl}\n{how}{must}"


def forced_call_grammar(tools: List[Dict[str, Any]], fmt: str, choice: ToolChoice) -> Optional[str]:
    """GBNF grammar that makes the reply one syntactically valid tool call whose arguments validate against the
    chosen function's parameter schema -- for ``tool_choice`` = "required" (any declared function) or a named
    function.  None when the choice does not force a call or the format has no JSON call syntax."""
    from ..runtime.json_schema import json_schema_to_gbnf

    if choice.mode not in ("required", "function") or fmt not in ("hermes", "mistral", "llama3"):
        return None
    fns = [t.get("function", t) for t in tools]
    if choice.mode == "function":
        fns = [f for f in fns if f.get("name") == choice.function]
        if not fns:
            raise ValueError(f"tool_choice names an undeclared function {choice.function!r}")
    key = "parameters" if fmt == "llama3" else "arguments"
    calls = {"anyOf": [{"type": "object", "properties": {"name": {"const": f["name"]},
                                                          key: f.get("parameters") or {"type": "object"}},
                        "required": ["name", key]} for f in fns]}
    body = json_schema_to_gbnf(calls)
    body = body.replace("root ::=", "call ::=", 1)
    wrap = {"hermes": 'root ::= "<tool_call>" call "</tool_call>"',
            "mistral": 'root ::= "[TOOL_CALLS] [" call "]"', "llama3": "root ::= call"}[fmt]
    return wrap + "\n" + body


def _relaxed_object(text: str) -> Dict[str, Any]:
    """``{id:42,name:"x",flag:true}`` -> dict.  Accepts strict JSON too."""
    text = text.strip()
    try:
        v = json.loads(text)
        if isinstance(v, dict):
            return v
    except json.JSONDecodeError:
        pass
    quoted = re.sub(r'([{,]\s*)([A-Za-z_][A-Za-z0-9_\-]*)\s*:', r'\1"\2":', text)
    try:
        v = json.loads(quoted)
        if isinstance(v, dict):
            return v
    except json.JSONDecodeError:
        pass
    # bare string values: {city:Paris}
    fixed = re.sub(r':\s*([A-Za-z_][^,}\]"]*)', lambda m: ":" + (m.group(1).strip() if m.group(1).strip() in (
        "true", "false", "null") else json.dumps(m.group(1).strip())), quoted)
    return json.loads(fixed)


def _call(name: str, arguments: Any) -> Dict[str, Any]:
    args = arguments if isinstance(arguments, str) else json.dumps(arguments if arguments is not None else {},
                                                                     separators=(",", ":"))
    return {"id": f"call_{next(_counter):08x}", "type": "function", "function": {"name": name, "arguments": args}}


def _calls_from_json(obj: Any) -> List[Dict[str, Any]]:
    items = obj if isinstance(obj, list) else [obj]
    out = []
    for it in items:
        if isinstance(it, dict) and isinstance(it.get("name"), str):
            out.append(_call(it["name"], it.get("arguments", it.get("parameters", {}))))
    return out


@dataclass
class ToolCallParser:
    fmt: str = "hermes"
    _buf: str = ""
    _content: List[str] = field(default_factory=list)
    _calls: List[Dict[str, Any]] = field(default_factory=list)
    _in_call: bool = False

    def reset(self) -> None:
        self._buf, self._content, self._calls, self._in_call = "", [], [], False

    # -- streaming ------------------------------------------------------------------------------------------------
    def feed(self, chunk: str) -> str:
        """Consumes a chunk; returns the text that is safe to show the user now (never part of a call, never a
        partial start marker)."""
        start, end = FORMATS[self.fmt]
        self._buf += chunk
        emitted: List[str] = []
        while True:
            if self._in_call:
                if end is None:
                    break  # the call payload runs to the end of the reply
                i = self._buf.find(end)
                if i < 0:
                    break
                self._parse_payload(self._buf[:i])
                self._buf, self._in_call = self._buf[i + len(end):], False
                continue
            i = self._buf.find(start)
            if i >= 0:
                emitted.append(self._buf[:i])
                self._buf, self._in_call = self._buf[i + len(start):], True
                continue
            # hold back a tail that could be the beginning of the start marker
            keep = 0
            for n in range(min(len(start) - 1, len(self._buf)), 0, -1):
                if start.startswith(self._buf[-n:]):
                    keep = n
                    break
            cut = len(self._buf) - keep
            emitted.append(self._buf[:cut])
            self._buf = self._buf[cut:]
            break
        text = "".join(emitted)
        if text:
            self._content.append(text)
        return text

    def _parse_payload(self, payload: str) -> None:
        payload = payload.strip()
        if not payload:
            return
        if self.fmt == "gemma":
            m = re.match(r"call:\s*([A-Za-z_][\w\-.]*)\s*(\{.*\})?\s*$", payload, re.S)
            if m:
                try:
                    self._calls.append(_call(m.group(1), _relaxed_object(m.group(2) or "{}")))
                    return
                except json.JSONDecodeError:
                    pass
            self._content.append(payload)
            return
        try:
            self._calls.extend(_calls_from_json(json.loads(payload)))
        except json.JSONDecodeError:
            # several objects back to back, or trailing text: take every decodable object
            dec, pos, found = json.JSONDecoder(), 0, False
            while pos < len(payload):
                j = min((k for k in (payload.find("{", pos), payload.find("[", pos)) if k >= 0), default=-1)
                if j < 0:
                    break
                try:
                    obj, endpos = dec.raw_decode(payload, j)
                except json.JSONDecodeError:
                    pos = j + 1
                    continue
                calls = _calls_from_json(obj)
                found = found or bool(calls)
                self._calls.extend(calls)
                pos = endpos
            if not found:
                self._content.append(payload)

    def finish(self) -> Tuple[str, List[Dict[str, Any]]]:
        """End of the reply: returns (content, tool_calls)."""
        if self._in_call:
            self._parse_payload(self._buf)
        else:
            self._content.append(self._buf)
        self._buf, self._in_call = "", False
        content = "".join(self._content)
        if self.fmt == "llama3" and not self._calls:
            # no python tag: the whole reply may still be a bare call object
            stripped = content.strip()
            if stripped.startswith("{") and stripped.endswith("}"):
                try:
                    calls = _calls_from_json(json.loads(stripped))
                except json.JSONDecodeError:
                    calls = []
                if calls:
                    self._calls, content = calls, ""
        return content.strip() if self._calls else content, list(self._calls)


def parse_tool_calls(text: str, fmt: str = "hermes") -> Tuple[str, List[Dict[str, Any]]]:
    p = ToolCallParser(fmt)
    p.feed(text)
    return p.finish()
