"""Tool-call rendering and parsing (all formats, streamed in arbitrary chunks)."""
import json
import random

import pytest

from antfly_b200.pipelines.tool_calls import (ToolCallParser, ToolChoice, detect_format, format_tools_prompt,
                                               parse_tool_calls, parse_tool_choice)

TOOLS = [{"type": "function", "function": {"name": "lookup", "description": "find a record",
                                           "parameters": {"type": "object", "properties": {"id": {"type": "integer"}}}}}]


def _args(call):
    return json.loads(call["function"]["arguments"])


def test_hermes_and_streaming_in_random_chunks():
    reply = ('Let me check.\n<tool_call>\n{"name": "lookup", "arguments": {"id": 42}}\n</tool_call>\n'
             '<tool_call>{"name": "lookup", "arguments": {"id": 7}}</tool_call> done')
    content, calls = parse_tool_calls(reply, "hermes")
    assert [c["function"]["name"] for c in calls] == ["lookup", "lookup"] and [_args(c)["id"] for c in calls] == [42, 7]
    assert "tool_call" not in content and content.startswith("Let me check.") and content.endswith("done")
    rng = random.Random(0)
    for _ in range(50):
        p, shown, i = ToolCallParser("hermes"), [], 0
        while i < len(reply):
            n = rng.randint(1, 9)
            shown.append(p.feed(reply[i:i + n]))
            i += n
            assert "<tool" not in "".join(shown)  # never leaks a (partial) marker
        c2, calls2 = p.finish()
        assert [_args(c)["id"] for c in calls2] == [42, 7] and c2 == content


def test_gemma_function_format():
    # the example from the reference parser's own tests: <|tool_call>call:lookup{id:42}<tool_call|>
    content, calls = parse_tool_calls("<|tool_call>call:lookup{id:42}<tool_call|>", "gemma")
    assert content == "" and calls[0]["function"]["name"] == "lookup" and _args(calls[0]) == {"id": 42}
    _, calls = parse_tool_calls('ok <|tool_call>call:weather{city:Paris,units:"metric",days:3,detail:true}<tool_call|>', "gemma")
    assert _args(calls[0]) == {"city": "Paris", "units": "metric", "days": 3, "detail": True}
    prompt = format_tools_prompt(TOOLS, "gemma")
    assert "<|tool>lookup" in prompt and "<|tool_call>call:function_name" in prompt


def test_mistral_and_llama3_formats():
    content, calls = parse_tool_calls('[TOOL_CALLS] [{"name": "lookup", "arguments": {"id": 1}}, {"name": "lookup", "arguments": {"id": 2}}]', "mistral")
    assert content == "" and [_args(c)["id"] for c in calls] == [1, 2]
    content, calls = parse_tool_calls('{"name": "lookup", "parameters": {"id": 9}}', "llama3")
    assert content == "" and _args(calls[0]) == {"id": 9}
    content, calls = parse_tool_calls('<|python_tag|>{"name": "lookup", "parameters": {"id": 3}}', "llama3")
    assert _args(calls[0]) == {"id": 3}
    content, calls = parse_tool_calls("The answer is 4.", "llama3")
    assert calls == [] and content == "The answer is 4."


def test_malformed_payload_falls_back_to_text():
    content, calls = parse_tool_calls("<tool_call>not json at all</tool_call>", "hermes")
    assert calls == [] and "not json" in content
    content, calls = parse_tool_calls("<tool_call>{\"name\": \"lookup\", \"arguments\": {\"id\": 5}}", "hermes")  # tag never closed
    assert _args(calls[0]) == {"id": 5}


def test_tool_choice_and_prompt_and_detection():
    assert parse_tool_choice(None) == ToolChoice("auto") and parse_tool_choice("none").enabled is False
    assert parse_tool_choice({"type": "function", "function": {"name": "lookup"}}) == ToolChoice("function", "lookup")
    with pytest.raises(ValueError):
        parse_tool_choice("sometimes")
    with pytest.raises(ValueError):
        parse_tool_choice({"type": "function", "function": {}})
    p = format_tools_prompt(TOOLS, "hermes", ToolChoice("function", "lookup"))
    assert '"name":"lookup"' in p and "<tool_call>" in p and "must call the tool lookup" in p
    assert detect_format("... <|tool_call> ...") == "gemma" and detect_format("x [TOOL_CALLS] y") == "mistral"
    assert detect_format(None, ["<|python_tag|>"]) == "llama3" and detect_format("plain") == "hermes"
    ids = {c["id"] for c in parse_tool_calls('<tool_call>{"name":"a","arguments":{}}</tool_call><tool_call>{"name":"b","arguments":{}}</tool_call>')[1]}
    assert len(ids) == 2


def test_forced_call_grammar_constrains_name_and_arguments():
    from antfly_b200.pipelines import tool_calls as TC
    from antfly_b200.runtime.grammar import GbnfGrammar

    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "unit": {"enum": ["c", "f"]}},
        "required": ["city"]}}},
        {"type": "function", "function": {"name": "ping"}}]

    def ok(g, text):
        m = GbnfGrammar([bytes([i]) for i in range(256)], g)
        return m.accept_text(text) and m.complete

    g = TC.forced_call_grammar(tools, "hermes", TC.parse_tool_choice("required"))
    assert ok(g, '<tool_call>{"name":"get_weather","arguments":{"city":"Oslo","unit":"c"}}</tool_call>')
    assert ok(g, '<tool_call>{"name": "ping", "arguments": {}}</tool_call>')
    assert not ok(g, '<tool_call>{"name":"get_weather","arguments":{"unit":"c"}}</tool_call>')      # city required
    assert not ok(g, '<tool_call>{"name":"other","arguments":{}}</tool_call>')
    assert not ok(g, 'Sure! <tool_call>{"name":"ping","arguments":{}}</tool_call>')
    one = TC.forced_call_grammar(tools, "mistral", TC.parse_tool_choice(
        {"type": "function", "function": {"name": "get_weather"}}))
    assert ok(one, '[TOOL_CALLS] [{"name":"get_weather","arguments":{"city":"x"}}]')
    assert not ok(one, '[TOOL_CALLS] [{"name":"ping","arguments":{}}]')
    l3 = TC.forced_call_grammar(tools, "llama3", TC.parse_tool_choice("required"))
    assert ok(l3, '{"name":"ping","parameters":{"anything":1}}')
    # what the grammar admits is what the parser extracts
    text = '<tool_call>{"name":"get_weather","arguments":{"city":"Oslo"}}</tool_call>'
    _, calls = TC.parse_tool_calls(text, "hermes")
    assert calls[0]["function"]["name"] == "get_weather"
    assert TC.forced_call_grammar(tools, "hermes", TC.parse_tool_choice("auto")) is None
    assert TC.forced_call_grammar(tools, "gemma", TC.parse_tool_choice("required")) is None
    import pytest

    with pytest.raises(ValueError):
        TC.forced_call_grammar(tools, "hermes", TC.parse_tool_choice({"type": "function", "function": {"name": "nope"}}))
