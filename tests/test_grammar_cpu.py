"""JSON-constrained decoding: the C++ recogniser (strings it must accept / reject), the token mask (random walks
over allowed tokens always end in text that ``json.loads`` parses), and the engine applying the mask."""
import json
import random

import numpy as np
import pytest
import torch

from antfly_b200.runtime.grammar import JsonGrammar, token_bytes_table

BYTE_VOCAB = [bytes([b]) for b in range(256)]
MULTI = [b'{"', b'":', b'": ', b'", "', b'true', b'false', b'null', b', ', b'[]', b'{}', b'0.5e', b'-1', b'"}',
         b'\\u00e9', b'\\n', b'  ', b'}]', b'[[', b'12', b'e+3', b'"a"', b'":[', b'\xc3\xa9']
VOCAB = BYTE_VOCAB + MULTI + [b""]  # last id plays end-of-sequence
EOS = len(VOCAB) - 1


@pytest.mark.parametrize("text", ['{"a": 1, "b": [true, false, null], "c": {"d": "x\\n\\u00e9"}}', '[]', '{}', '  [1, 2.5e-3, -0]  ',
                                  '"just a string"', '-12.75E+2', 'null', '[[[]]]', '{"k":"v","k2":[{}]}'])
def test_accepts_valid_documents(text):
    g = JsonGrammar(VOCAB, eos_id=EOS)
    assert g.accept_text(text), text
    assert g.complete
    json.loads(text)


@pytest.mark.parametrize("text", ['{"a":1,}', '01', '[1 2]', '"\x01"', '{"a" 1}', 'tru e', '{a:1}', '[1,,2]', '{"a":}',
                                  '1.', '-', '"\\x"', '"\\u12g4"', ']', '{"a":1}}', '[1]]', '+1', '.5', 'nul1'])
def test_rejects_invalid_documents(text):
    g = JsonGrammar(VOCAB, eos_id=EOS)
    ok = g.accept_text(text)
    assert not (ok and g.complete), text
    if ok:  # a valid *prefix* at most ('1.' / '-'): never complete, and the json module agrees it is not a document
        with pytest.raises(json.JSONDecodeError):
            json.loads(text)


def test_root_object_only_mode():
    g = JsonGrammar(VOCAB, eos_id=EOS, root_object_only=True)
    m = g.mask()
    allowed = {i for i in range(len(VOCAB)) if m[i]}
    assert ord("{") in allowed and ord("[") not in allowed and ord("1") not in allowed
    assert g.accept_text('  {"x": [1]}') and g.complete


def test_random_walks_over_the_mask_always_produce_json():
    rng = random.Random(0)
    closers = {ord("}"), ord("]"), ord('"')}
    for walk in range(120):
        g = JsonGrammar(VOCAB, eos_id=EOS)
        out = bytearray()
        for step in range(400):
            m = g.mask()
            ids = np.flatnonzero(m)
            assert len(ids) > 0
            if m[EOS] and (step > 40 or rng.random() < 0.2):
                assert g.accept(EOS)
                break
            cand = [int(i) for i in ids if i != EOS]
            # keep documents finite: past a length, favour tokens that close something
            pref = [i for i in cand if i in closers or VOCAB[i] in (b'"}', b'}]')] if step > 60 else []
            if g._lib.afb_grammar_depth(g._h) == 0 and step > 60 and m[EOS]:
                assert g.accept(EOS)
                break
            tok = rng.choice(pref or cand)
            assert g.accept(tok)
            out += VOCAB[tok]
        else:
            continue  # did not finish within the budget: nothing to parse
        json.loads(out.decode("utf-8", errors="strict") if all(b < 0x80 for b in out) else out.decode("utf-8", "ignore"))


def test_mask_matches_stepwise_acceptance():
    g = JsonGrammar(VOCAB, eos_id=EOS)
    assert g.accept_text('{"key": [1, ')
    m = g.mask()
    for t in range(len(VOCAB) - 1):
        h = JsonGrammar(VOCAB, eos_id=EOS)
        assert h.accept_text('{"key": [1, ')
        assert bool(m[t]) == h.accept(t), (t, VOCAB[t])
    assert not m[EOS]


def test_engine_applies_the_grammar_mask():
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    tok = ByteTokenizer(vocab_size=512)
    cfg = LlamaConfig.tiny(vocab_size=512)
    model = LlamaModel.random_init(cfg, device="cpu", seed=1, fast_init=False)
    eng = LLMEngine(model, num_blocks=32, page=16, max_batch=2, max_step_tokens=128, prefill_chunk=64,
                    max_seq_len=128, use_cuda_graph=False, eos_token_id=tok.special.eos_id)
    table = token_bytes_table(tok, 512)
    for temperature in (0.0, 0.9):
        gr = JsonGrammar(table, eos_id=tok.special.eos_id)
        rid = eng.add_request(tok.encode_prompt("reply in json: "),
                              SamplingParams(max_tokens=48, temperature=temperature, seed=7, grammar=gr))
        while eng.has_work():
            eng.step()
        r = eng.reqs[rid]
        text = b"".join(table[t] for t in r.out if t != tok.special.eos_id)
        check = JsonGrammar(table, eos_id=tok.special.eos_id)
        assert check._lib.afb_grammar_accept_bytes(check._h, text, len(text)) == 1, text
        if r.finish_reason == "stop":
            json.loads(text.decode("utf-8", "ignore"))


# ---------------------------------------------------------------------------------------------------------------
# GBNF
# ---------------------------------------------------------------------------------------------------------------
from antfly_b200.runtime.grammar import GbnfGrammar

ARITH = r"""
# arithmetic with parentheses
root  ::= expr
expr  ::= term (("+" | "-") term)*
term  ::= factor (("*" | "/") factor)*
factor ::= number | "(" expr ")"
number ::= [0-9]+ ("." [0-9]{1,3})?
"""

ISO_DATE = 'root ::= [0-9]{4} "-" ("0" [1-9] | "1" [0-2]) "-" [0-3] [0-9]'

CHOICE = 'root ::= ("yes" | "no" | "maybe") "\\n"?'


def _gb(text, **kw):
    return GbnfGrammar(VOCAB, text, eos_id=EOS, **kw)


@pytest.mark.parametrize("grammar,good,bad", [
    (ARITH, ["1", "12+3", "(1+2)*3.25", "((7))", "4/2-1"], ["", "+", "1+", "(1", "1.2345", "1 + 2", "a"]),
    (ISO_DATE, ["2026-11-25", "1999-01-01"], ["2026-13-01", "26-11-25", "2026-1-1", "2026-00-10"]),
    (CHOICE, ["yes", "no\n", "maybe"], ["ye", "nope", "yes\n\n", "YES"]),
    ('root ::= [^"\\\\\\x00-\\x1f]* "!"', ["abc!", "!", "café!"], ['a"b!', "a\\b!", "abc"]),
])
def test_gbnf_accepts_and_rejects(grammar, good, bad):
    for text in good:
        g = _gb(grammar)
        assert g.accept_text(text) and g.complete, text
    for text in bad:
        g = _gb(grammar)
        assert not (g.accept_text(text) and g.complete), text


def test_gbnf_mask_and_random_walks():
    rng = random.Random(1)
    g0 = _gb(ARITH)
    m = g0.mask()
    allowed = {VOCAB[i] for i in np.flatnonzero(m)}
    assert b"(" in allowed and b"7" in allowed and b"12" in allowed and b"[[" not in allowed
    assert b"+" not in allowed and not m[EOS]
    for walk in range(60):
        g = _gb(ARITH)
        out = bytearray()
        for step in range(200):
            m = g.mask()
            ids = [int(i) for i in np.flatnonzero(m)]
            assert ids
            if m[EOS] and (step > 20 or rng.random() < 0.15):
                assert g.accept(EOS)
                break
            cand = [i for i in ids if i != EOS]
            closing = [i for i in cand if VOCAB[i] in (b")", b"1", b"12")] if step > 30 else []
            tok = rng.choice(closing or cand)
            assert g.accept(tok)
            out += VOCAB[tok]
        else:
            continue
        text = out.decode()
        assert set(text) <= set("0123456789.+-*/()") and text.count("(") == text.count(")")
        check = _gb(ARITH)  # the emitted text, re-read in one piece, is a complete sentence of the grammar
        assert check.accept_text(text) and check.complete, text
        assert text[-1] in "0123456789)" and text[0] in "0123456789("


def test_gbnf_errors():
    with pytest.raises(ValueError, match="never defined"):
        _gb('root ::= missing "x"')
    with pytest.raises(ValueError, match="no rule named"):
        _gb('start ::= "x"')
    with pytest.raises(ValueError, match="left recursion|terminate"):
        _gb('root ::= root "a" | "a"')
    with pytest.raises(ValueError):
        _gb('root ::= "unterminated')
    assert _gb('start ::= "x"', root="start").accept_text("x")


def _matches(grammar: str, text: str) -> bool:
    from antfly_b200.runtime.grammar import GbnfGrammar

    g = GbnfGrammar([bytes([i]) for i in range(256)], grammar)
    return g.accept_text(text) and g.complete


def test_json_schema_compiles_to_a_grammar_that_accepts_exactly_valid_documents():
    from antfly_b200.runtime.json_schema import json_schema_to_gbnf

    schema = {
        "type": "object",
        "properties": {
            "name": {"type": "string", "minLength": 1, "maxLength": 8},
            "age": {"type": "integer"},
            "tags": {"type": "array", "items": {"enum": ["a", "b", "c d"]}, "minItems": 1, "maxItems": 3},
            "address": {"$ref": "#/$defs/addr"},
            "score": {"type": ["number", "null"]},
            "kind": {"const": "person"},
        },
        "required": ["name", "tags"],
        "$defs": {"addr": {"type": "object", "properties": {"city": {"type": "string"},
                                                              "zip": {"type": "string", "format": "uuid"}},
                           "required": ["city"]}},
    }
    g = json_schema_to_gbnf(schema)
    ok = ['{"name":"bob","tags":["a"]}',
          ' { "name" : "x", "age": -12, "tags": ["a", "c d", "b"] } ',
          '{"name":"bob","tags":["b"],"address":{"city":"Paris"},"score":null,"kind":"person"}',
          '{"name":"bob","tags":["b"],"address":{"city":"P","zip":"123e4567-e89b-12d3-a456-426614174000"},"score":1.5e3}',
          '{"name":"q\\"uote","tags":["a","a"]}']
    bad = ['{"tags":["a"]}',                                   # required name missing
           '{"name":"bob"}',                                   # required tags missing
           '{"name":"","tags":["a"]}',                         # minLength
           '{"name":"toolongname","tags":["a"]}',              # maxLength
           '{"name":"bob","tags":[]}',                         # minItems
           '{"name":"bob","tags":["a","a","a","a"]}',          # maxItems
           '{"name":"bob","tags":["z"]}',                      # enum
           '{"name":"bob","age":1.5,"tags":["a"]}',            # integer
           '{"tags":["a"],"name":"bob"}',                      # declaration order is fixed
           '{"name":"bob","tags":["a"],"extra":1}',            # no additional properties
           '{"name":"bob","tags":["a"],"kind":"robot"}',       # const
           '{"name":"bob","tags":["a"],"address":{}}',         # nested required
           '{"name":"bob","tags":["a"]', '[1]', 'null']
    for t in ok:
        assert _matches(g, t), t
    for t in bad:
        assert not _matches(g, t), t


def test_json_schema_recursion_additional_properties_and_anyof():
    from antfly_b200.runtime.json_schema import json_schema_to_gbnf

    tree = {"$ref": "#/definitions/node", "definitions": {"node": {
        "type": "object", "properties": {"v": {"type": "integer"},
                                         "kids": {"type": "array", "items": {"$ref": "#/definitions/node"}}},
        "required": ["v"]}}}
    g = json_schema_to_gbnf(tree)
    assert _matches(g, '{"v":1,"kids":[{"v":2},{"v":3,"kids":[{"v":4,"kids":[]}]}]}')
    assert not _matches(g, '{"v":1,"kids":[{"x":2}]}')
    free = json_schema_to_gbnf({"type": "object", "properties": {"id": {"type": "integer"}}, "required": ["id"],
                                "additionalProperties": {"type": "boolean"}})
    assert _matches(free, '{"id":1,"a":true,"b":false}') and not _matches(free, '{"id":1,"a":3}')
    assert _matches(free, '{"id":7}') and not _matches(free, '{"a":true}')
    opt = json_schema_to_gbnf({"type": "object", "properties": {"a": {"type": "null"}, "b": {"type": "boolean"}}})
    for t in ('{}', '{"a":null}', '{"b":true}', '{"a":null,"b":false}'):
        assert _matches(opt, t), t
    assert not _matches(opt, '{"b":true,"a":null}') and not _matches(opt, '{"a":null,}')
    any_of = json_schema_to_gbnf({"anyOf": [{"type": "string", "format": "date"}, {"type": "array", "maxItems": 0},
                                            {"type": "object"}]})
    for t in ('"2024-02-29"', '[]', '{"anything":[1,{"x":null}]}'):
        assert _matches(any_of, t), t
    assert not _matches(any_of, '"yesterday"') and not _matches(any_of, '[1]')
    with pytest.raises(ValueError):
        json_schema_to_gbnf({"$ref": "http://elsewhere/schema"})
    with pytest.raises(ValueError):
        json_schema_to_gbnf({"type": "array", "minItems": 3, "maxItems": 1})
