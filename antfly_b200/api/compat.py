"""Wire-format adapters: the Anthropic Messages API on top of the native generate handler.

Request translation and the response / streaming event shapes follow the reference's compatibility layer
(go/pkg/termite/anthropic.go:29-330): ``system`` (string or text blocks) becomes the leading system message,
content blocks are flattened to text, ``tool_use`` / ``tool_result`` blocks become assistant tool calls and tool
messages, tools are re-declared in the function-calling format, ``stop_sequences`` become stop strings.  Responses
carry ``content`` blocks (``text`` and ``tool_use``), ``stop_reason`` (``end_turn`` / ``max_tokens`` /
``tool_use`` / ``stop_sequence``) and ``usage.input_tokens`` / ``output_tokens``; streams use the named-event
sequence ``message_start``, ``content_block_start``, ``content_block_delta``..., ``content_block_stop``,
``message_delta``, ``message_stop``.
"""
from __future__ import annotations

import json
import uuid
from typing import Any, Dict, List, Optional

STOP_REASON = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use", "stop_sequence": "stop_sequence"}


def _text_of(content) -> str:
    if isinstance(content, str):
        return content
    out = []
    for b in content or []:
        if isinstance(b, dict) and b.get("type") == "text":
            out.append(b.get("text", ""))
    return "".join(out)


def anthropic_to_generate(body: Dict[str, Any]) -> Dict[str, Any]:
    if not body.get("model"):
        raise ValueError("model is required")
    if not isinstance(body.get("max_tokens"), int) or body["max_tokens"] <= 0:
        raise ValueError("max_tokens is required and must be positive")
    if not body.get("messages"):
        raise ValueError("messages must not be empty")
    msgs: List[Dict[str, Any]] = []
    system = body.get("system")
    if system:
        msgs.append({"role": "system", "content": _text_of(system)})
    for m in body["messages"]:
        role, content = m.get("role"), m.get("content")
        if role not in ("user", "assistant"):
            raise ValueError(f"unsupported role {role!r}")
        if isinstance(content, str):
            msgs.append({"role": role, "content": content})
            continue
        calls, image_parts = [], []
        for b in content or []:
            t = b.get("type")
            if t == "tool_result":
                msgs.append({"role": "tool", "tool_call_id": b.get("tool_use_id", ""),
                             "content": _text_of(b.get("content"))})
            elif t == "tool_use":
                calls.append({"id": b.get("id") or "toolu_" + uuid.uuid4().hex[:16], "type": "function",
                              "function": {"name": b.get("name", ""), "arguments": json.dumps(b.get("input") or {})}})
            elif t == "image" and isinstance(b.get("source"), dict) and b["source"].get("type") == "base64":
                src = b["source"]
                image_parts.append({"type": "image_url", "image_url": {
                    "url": f"data:{src.get('media_type', 'image/png')};base64,{src.get('data', '')}"}})
        text = _text_of(content)
        if calls:
            msgs.append({"role": "assistant", "content": text or None, "tool_calls": calls})
        elif image_parts:
            msgs.append({"role": role, "content": ([{"type": "text", "text": text}] if text else []) + image_parts})
        elif text or not any(b.get("type") == "tool_result" for b in content or []):
            msgs.append({"role": role, "content": text})
    out: Dict[str, Any] = {"model": body["model"], "messages": msgs, "max_tokens": body["max_tokens"],
                           "stream": bool(body.get("stream", False))}
    for src, dst in (("temperature", "temperature"), ("top_p", "top_p"), ("top_k", "top_k")):
        if body.get(src) is not None:
            out[dst] = body[src]
    if body.get("stop_sequences"):
        out["stop"] = list(body["stop_sequences"])
    if body.get("tools"):
        out["tools"] = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                                          "parameters": t.get("input_schema") or {}}}
                        for t in body["tools"]]
        tc = body.get("tool_choice") or {}
        if tc.get("type") == "any":
            out["tool_choice"] = "required"
        elif tc.get("type") == "tool":
            out["tool_choice"] = {"type": "function", "function": {"name": tc.get("name", "")}}
        elif tc.get("type") == "none":
            out["tool_choice"] = "none"
    return out


def _tool_blocks(calls) -> List[Dict[str, Any]]:
    blocks = []
    for c in calls or []:
        fn = c.get("function", {}) if isinstance(c, dict) else {}
        try:
            args = json.loads(fn.get("arguments") or "{}")
        except ValueError:
            args = {"_raw": fn.get("arguments")}
        blocks.append({"type": "tool_use", "id": (c.get("id") or "").replace("call_", "toolu_") or
                       "toolu_" + uuid.uuid4().hex[:16], "name": fn.get("name", ""), "input": args})
    return blocks


class AnthropicFramer:
    """Turns a native generate result (or its stream of deltas) into Messages-API JSON / server-sent events."""

    def __init__(self):
        self.id, self.model = "msg_" + uuid.uuid4().hex[:24], ""
        self.block_open, self.index = False, 0

    def begin(self, rid: str, model: str) -> None:
        self.model = model

    # -- whole response --------------------------------------------------------------------------------------
    def response(self, resp: Dict[str, Any]) -> Dict[str, Any]:
        choice = resp["choices"][0]
        msg = choice["message"]
        content: List[Dict[str, Any]] = []
        if msg.get("content"):
            content.append({"type": "text", "text": msg["content"]})
        content += _tool_blocks(msg.get("tool_calls"))
        return {"id": self.id, "type": "message", "role": "assistant", "content": content, "model": resp["model"],
                "stop_reason": STOP_REASON.get(choice.get("finish_reason"), "end_turn"), "stop_sequence": None,
                "usage": {"input_tokens": resp["usage"]["prompt_tokens"],
                          "output_tokens": resp["usage"]["completion_tokens"]}}

    # -- stream ------------------------------------------------------------------------------------------------
    @staticmethod
    def _ev(name: str, data: Dict[str, Any]) -> str:
        return f"event: {name}\ndata: {json.dumps(data)}\n\n"

    def start(self) -> str:
        return self._ev("message_start", {"type": "message_start", "message": {
            "id": self.id, "type": "message", "role": "assistant", "content": [], "model": self.model,
            "stop_reason": None, "stop_sequence": None, "usage": {"input_tokens": 0, "output_tokens": 0}}})

    def _close_block(self) -> str:
        if not self.block_open:
            return ""
        self.block_open = False
        ev = self._ev("content_block_stop", {"type": "content_block_stop", "index": self.index})
        self.index += 1
        return ev

    def text(self, t: str) -> str:
        out = ""
        if not self.block_open:
            self.block_open = True
            out += self._ev("content_block_start", {"type": "content_block_start", "index": self.index,
                                                    "content_block": {"type": "text", "text": ""}})
        return out + self._ev("content_block_delta", {"type": "content_block_delta", "index": self.index,
                                                      "delta": {"type": "text_delta", "text": t}})

    def tool_calls(self, calls) -> str:
        out = self._close_block()
        for b in _tool_blocks(calls):
            out += self._ev("content_block_start", {"type": "content_block_start", "index": self.index,
                                                    "content_block": {"type": "tool_use", "id": b["id"],
                                                                      "name": b["name"], "input": {}}})
            out += self._ev("content_block_delta", {"type": "content_block_delta", "index": self.index, "delta": {
                "type": "input_json_delta", "partial_json": json.dumps(b["input"])}})
            out += self._ev("content_block_stop", {"type": "content_block_stop", "index": self.index})
            self.index += 1
        return out

    def finish(self, reason: Optional[str], prompt_tokens: int, completion_tokens: int) -> str:
        return self._close_block() + self._ev("message_delta", {
            "type": "message_delta", "delta": {"stop_reason": STOP_REASON.get(reason, "end_turn"),
                                               "stop_sequence": None},
            "usage": {"input_tokens": prompt_tokens, "output_tokens": completion_tokens}}) + \
            self._ev("message_stop", {"type": "message_stop"})

    def error(self, body: str) -> str:
        try:
            msg = json.loads(body).get("message", body)
        except ValueError:
            msg = body
        return self._ev("error", {"type": "error", "error": {"type": "api_error", "message": msg}})
