"""Structured extraction: field definitions, choice resolution, gap clustering into instances, and the endpoint's
``structures`` schema (checked with a scripted span model so every number is known)."""
from dataclasses import dataclass

import pytest
from fastapi.testclient import TestClient

from antfly_b200.api.model_manager import ModelManager
from antfly_b200.api.server import create_app
from antfly_b200.pipelines import extraction as EX


@dataclass
class Ent:
    label: str
    text: str
    start: int
    end: int
    score: float


class Scripted:
    """Finds every occurrence of scripted (label, phrase, score) triples; classifies by a scripted table."""

    def __init__(self, phrases, verdicts=None):
        self.phrases, self.verdicts, self.calls = phrases, verdicts or {}, []

    def recognize(self, texts, labels, threshold=None, flat_ner=None):
        self.calls.append((list(labels), threshold))
        out = []
        for t in texts:
            raw, ents = t.encode(), []
            for label, phrase, score in self.phrases:
                at = raw.find(phrase.encode())
                while at >= 0 and label in labels and score >= (threshold or 0):
                    ents.append(Ent(label, phrase, at, at + len(phrase.encode()), score))
                    at = raw.find(phrase.encode(), at + 1)
            out.append(ents)
        return out

    def classify(self, text, labels, threshold=0.0, multi_label=False, top_k=0):
        return [(self.verdicts.get(text, labels[0]), 0.77)]


def test_field_definitions():
    f = EX.parse_field_def("name::str")
    assert (f.name, f.is_list, f.choices) == ("name", False, [])
    f = EX.parse_field_def("skills::list")
    assert (f.name, f.is_list) == ("skills", True)
    f = EX.parse_field_def(" role::[engineer|manager]::str ")
    assert (f.name, f.is_list, f.choices) == ("role", False, ["engineer", "manager"])
    assert EX.parse_field_def("plain").name == "plain" and EX.parse_field_def("a::b::array").name == "a::b"
    for bad in ("", "::str", "x::[only]::str", "x::[a||b]"):
        with pytest.raises(ValueError):
            EX.parse_field_def(bad)
    canon = EX.canonical_structures({"person": {"fields": {"name": "str", "skills": "list",
                                                           "role": {"type": "str", "choices": ["a", "b"]}}},
                                     "short": ["x::list", "y"]})
    assert [(f.name, f.is_list) for f in canon["person"]] == [("name", False), ("skills", True), ("role", False)]
    assert canon["person"][2].choices == ["a", "b"] and [f.is_list for f in canon["short"]] == [True, False]
    with pytest.raises(ValueError):
        EX.canonical_structures({"empty": {"fields": {}}})


def test_cluster_threshold_and_instances():
    spans = [dict(label="n", text="a", start=0, end=1, score=.5), dict(label="n", text="b", start=3, end=4, score=.9),
             dict(label="n", text="c", start=400, end=401, score=.7)]
    assert EX.cluster_threshold(spans, 0, 1000) == 100            # median gap 2 -> 6, floor min(100, 1000 / 10)
    assert EX.cluster_threshold(spans, 0, 200) == 20 and EX.cluster_threshold(spans, 7, 1000) == 7
    assert EX.cluster_threshold(spans[:1], 0, 1000) == 0
    fields = [EX.SchemaField("n"), EX.SchemaField("tags", True)]
    inst = EX.assemble_instances(fields, spans, EX.ExtractionConfig(include_confidence=True), 1000)
    assert inst == [{"n": {"value": "b", "score": .9}}, {"n": {"value": "c", "score": .7}}]   # best of a cluster
    both = spans + [dict(label="tags", text="t1", start=5, end=7, score=.4), dict(label="tags", text="t2", start=9, end=11, score=.3)]
    inst = EX.assemble_instances(fields, both, EX.ExtractionConfig(include_spans=True), 1000)
    assert inst[0]["tags"] == [{"value": "t1", "start": 5, "end": 7}, {"value": "t2", "start": 9, "end": 11}]
    assert "tags" not in inst[1] and EX.assemble_instances(fields, [], EX.ExtractionConfig(), 10) == []


def test_structures_from_a_span_model_with_choices_and_unicode_offsets():
    text = ("Ana Müller is a Senior Engineer who knows Zig and CUDA. " + "x" * 300 +
            " Bo Li is the boss and knows Go.")
    pipe = Scripted([("name", "Ana Müller", .9), ("name", "Bo Li", .8), ("role", "Senior Engineer", .7),
                     ("role", "boss", .6), ("skills", "Zig", .5), ("skills", "CUDA", .5), ("skills", "Go", .4)],
                    verdicts={"Senior Engineer": "engineer", "boss": "manager"})
    canon = EX.canonical_structures({"person": ["name::str", "skills::list", "role::[engineer|manager]::str"]})
    got = EX.extract_structures(pipe, text, canon, EX.ExtractionConfig(include_spans=True, include_confidence=True))
    people = got["person"]
    assert len(people) == 2 and pipe.calls[0] == (["name", "skills", "role"], 0.3)
    assert people[0]["name"] == {"value": "Ana Müller", "score": .9, "start": 0, "end": 10}     # characters, not bytes
    assert [s["value"] for s in people[0]["skills"]] == ["Zig", "CUDA"]
    # a choice field keeps only its best span (here the first person's) and rewrites it to the chosen label
    assert people[0]["role"]["value"] == "engineer" and people[0]["role"]["score"] == 0.77 and "role" not in people[1]
    assert people[1]["name"]["value"] == "Bo Li" and [s["value"] for s in people[1]["skills"]] == ["Go"]
    assert text[people[1]["name"]["start"]:people[1]["name"]["end"]] == "Bo Li"
    exact = Scripted([("role", "Manager", .9)])
    got = EX.extract_structures(exact, "The Manager left.", EX.canonical_structures({"p": ["role::[engineer|manager]"]}))
    assert got["p"] == [{"role": {"value": "manager"}}]                                       # matched without a model call


def test_extract_endpoint_answers_structures():
    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    pipe = Scripted([("name", "Ada", .9), ("skills", "math", .6), ("skills", "engines", .5)])
    mgr.register("spans", "recognizer", pipe, None)
    c = TestClient(create_app(mgr))
    body = {"model": "spans", "inputs": [{"id": "d1", "content": "Ada knows math and engines."},
                                         {"content": [{"type": "text", "text": "nothing here"}]}],
            "schema": {"structures": {"person": {"fields": {"name": "str", "skills": "list"}}}}}
    r = c.post("/ai/v1/extract", json=body)
    assert r.status_code == 200, r.text
    d = r.json()["data"]
    assert d[0]["id"] == "d1" and d[0]["structures"] == {"person": [{"name": {"value": "Ada"}, "skills": [
        {"value": "math"}, {"value": "engines"}]}]}
    assert d[1]["structures"] == {"person": []}
    body["options"] = {"include_confidence": True, "include_spans": True, "threshold": 0.55}
    d = c.post("/ai/v1/extract", json=body).json()["data"]
    assert d[0]["structures"]["person"][0]["skills"] == [{"value": "math", "score": .6, "start": 10, "end": 14}]
    bad = dict(body, schema={"structures": {"person": {"fields": {}}}})
    assert c.post("/ai/v1/extract", json=bad).status_code == 400
    assert c.post("/ai/v1/extract", json=dict(body, schema={})).status_code == 400


def test_image_inputs_are_read_first(tmp_path):
    import base64
    import io

    import numpy as np
    from PIL import Image

    class FakeReader:
        def __init__(self):
            self.calls = []

        def read(self, images, max_tokens=256, prompt=None):
            from antfly_b200.pipelines.reading import ReadResult

            self.calls.append((len(images), max_tokens, prompt, tuple(images[0].shape)))
            return [ReadResult("Ada knows math.", []) for _ in images]

    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    reader = FakeReader()
    mgr.register("spans", "recognizer", Scripted([("name", "Ada", .9), ("skills", "math", .6)]), None)
    mgr.register("ocr", "reader", reader, None)
    buf = io.BytesIO()
    Image.fromarray(np.zeros((6, 9, 3), dtype=np.uint8)).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    c = TestClient(create_app(mgr))
    body = {"model": "spans", "inputs": [{"content": [{"type": "image_url", "image_url": {"url": url}}]}],
            "schema": {"structures": {"person": ["name", "skills::list"]}},
            "options": {"reader": {"model": "ocr", "prompt": "<OCR>"}, "max_tokens": 32}}
    r = c.post("/ai/v1/extract", json=body)
    assert r.status_code == 200, r.text
    assert r.json()["data"][0]["structures"]["person"] == [{"name": {"value": "Ada"}, "skills": [{"value": "math"}]}]
    assert reader.calls == [(1, 32, "<OCR>", (6, 9, 3))]
    body["options"] = {}
    assert c.post("/ai/v1/extract", json=body).status_code == 400          # images without a reader model
