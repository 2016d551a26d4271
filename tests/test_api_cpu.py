"""HTTP contract on the CPU path, modelled on the reference's product-level pytest suites
(zig/e2e/inference/test_embed.py:37-85, test_rerank.py:27-50, test_generate.py, test_openai_compat.py)."""
import json
import math

import pytest
from fastapi.testclient import TestClient

from antfly_b200.api.model_manager import ModelManager
from antfly_b200.api.server import RequestQueue, create_app
from antfly_b200.runtime.scheduler import QueueFull


@pytest.fixture(scope="module")
def client():
    mgr = ModelManager(models_dir="/nonexistent", device="cpu", kv_blocks=128, max_batch=4)
    mgr.register_random("tiny-embed", "embedder")
    mgr.register_random("tiny-rerank", "reranker")
    mgr.register_random("tiny-gen", "generator")
    return TestClient(create_app(mgr))


def test_health_ready_models(client):
    assert client.get("/healthz").json()["status"] == "ok"
    assert client.get("/readyz").status_code == 200
    m = client.get("/ai/v1/models").json()
    assert m["object"] == "list" and "tiny-embed" in m["embedders"] and "tiny-gen" in m["generators"]
    assert "fixed" in m["chunkers"] and {"rerankers", "backends", "allow_downloads"} <= set(m)


@pytest.mark.parametrize("path", ["/ai/v1/embed", "/ai/v1/embeddings"])
def test_embed_shape_norm_and_dimensions(client, path):
    r = client.post(path, json={"model": "tiny-embed", "input": ["hello world", "second text"]})
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "list" and body["model"] == "tiny-embed" and len(body["data"]) == 2
    for i, d in enumerate(body["data"]):
        assert d["object"] == "embedding" and d["index"] == i and len(d["embedding"]) == 128
        assert abs(math.sqrt(sum(x * x for x in d["embedding"])) - 1.0) < 1e-2
    assert body["usage"]["prompt_tokens"] == body["usage"]["total_tokens"] > 0
    r = client.post(path, json={"model": "tiny-embed", "input": "one", "dimensions": 16})
    assert len(r.json()["data"][0]["embedding"]) == 16
    assert client.post(path, json={"model": "tiny-embed", "input": "x", "dimensions": 4096}).status_code == 400


def test_embed_errors(client):
    assert client.post("/ai/v1/embed", json={"model": "missing", "input": "x"}).status_code == 404
    r = client.post("/ai/v1/embed", json={"input": "x"})
    assert r.status_code == 400 and set(r.json()) == {"error", "message"}
    assert client.post("/ai/v1/embed", json={"model": "tiny-embed", "input": "x", "encoding_format": "base64"}).status_code == 400


def test_rerank_contract(client):
    r = client.post("/ai/v1/rerank", json={"model": "tiny-rerank", "query": "q", "prompts": ["doc a", "doc b", "c"]})
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "list" and [d["index"] for d in body["data"]] == [0, 1, 2]
    assert all(d["object"] == "rerank.score" and 0.0 <= d["score"] <= 1.0 for d in body["data"])
    assert body["usage"]["completion_tokens"] == 0
    assert client.post("/ai/v1/rerank", json={"model": "tiny-rerank", "query": "q", "prompts": []}).status_code == 400


@pytest.mark.parametrize("path", ["/ai/v1/generate", "/ai/v1/chat/completions"])
def test_generate_contract(client, path):
    r = client.post(path, json={"model": "tiny-gen", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5,
                                "temperature": 0})
    assert r.status_code == 200
    b = r.json()
    assert b["object"] == "chat.completion" and b["choices"][0]["message"]["role"] == "assistant"
    assert b["choices"][0]["finish_reason"] in ("length", "stop")
    u = b["usage"]
    assert u["completion_tokens"] <= 5 and u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]
    r2 = client.post(path, json={"model": "tiny-gen", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5,
                                 "temperature": 0})
    assert r2.json()["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]


def test_generate_streaming_sse(client):
    with client.stream("POST", "/ai/v1/chat/completions",
                       json={"model": "tiny-gen", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                             "temperature": 0, "stream": True}) as r:
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert all(c["object"] == "chat.completion.chunk" for c in chunks)
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"
    assert chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop")


def test_generate_json_mode_gbnf_and_tools(client):
    """Constrained decoding and tool plumbing through the HTTP API (random weights: only the constraints are
    checked, not what the model says)."""
    base = {"model": "tiny-gen", "messages": [{"role": "user", "content": "give me json"}], "max_tokens": 24,
            "temperature": 0}
    r = client.post("/ai/v1/chat/completions", json=dict(base, response_format={"type": "json_object"}))
    assert r.status_code == 200
    text = r.json()["choices"][0]["message"]["content"] or ""
    assert text.lstrip().startswith("{")      # root must be an object; every prefix stays valid JSON
    if r.json()["choices"][0]["finish_reason"] == "stop":
        json.loads(text)
    r = client.post("/ai/v1/chat/completions", json=dict(base, grammar='root ::= ("yes" | "no") "!"'))
    assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"] in ("yes!", "no!")
    assert r.json()["choices"][0]["finish_reason"] == "stop"
    r = client.post("/ai/v1/chat/completions", json=dict(base, grammar='root ::= undefined-rule'))
    assert r.status_code == 400 and "never defined" in r.json()["message"]
    # structured output: a schema with only finite choices, so even random weights must produce a valid document
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "level": {"enum": ["low", "high"]},
                                               "n": {"const": 7}}, "required": ["ok", "level", "n"]}
    r = client.post("/ai/v1/chat/completions", json=dict(base, max_tokens=120, response_format={
        "type": "json_schema", "json_schema": {"name": "verdict", "schema": schema}}))
    assert r.status_code == 200, r.text
    if r.json()["choices"][0]["finish_reason"] == "stop":
        doc = json.loads(r.json()["choices"][0]["message"]["content"])
        assert set(doc) == {"ok", "level", "n"} and isinstance(doc["ok"], bool) and doc["level"] in ("low", "high")
        assert doc["n"] == 7
    else:       # ran out of tokens inside optional whitespace: what was produced is still a valid prefix
        assert (r.json()["choices"][0]["message"]["content"] or "").lstrip().startswith("{")
    r = client.post("/ai/v1/chat/completions", json=dict(base, response_format={
        "type": "json_schema", "json_schema": {"schema": {"$ref": "http://remote/schema"}}}))
    assert r.status_code == 400 and "$ref" in r.json()["message"]
    tools = [{"type": "function", "function": {"name": "lookup", "parameters": {"type": "object"}}}]
    r = client.post("/ai/v1/chat/completions", json=dict(base, tools=tools, tool_choice="sometimes"))
    assert r.status_code == 400
    # force a syntactically valid tool call with a grammar and check it comes back parsed
    call_grammar = 'root ::= "<tool_call>{\\"name\\": \\"lookup\\", \\"arguments\\": {\\"id\\": " [1-9] "}}</tool_call>"'
    r = client.post("/ai/v1/chat/completions", json=dict(base, max_tokens=80, tools=tools, grammar=call_grammar))
    assert r.status_code == 200, r.text
    choice = r.json()["choices"][0]
    assert choice["finish_reason"] == "tool_calls" and choice["message"]["tool_calls"][0]["function"]["name"] == "lookup"
    assert 1 <= json.loads(choice["message"]["tool_calls"][0]["function"]["arguments"])["id"] <= 9


def test_embed_images_and_text_with_a_clip_model():
    """Content parts of type image_url (data: URLs) and text through one CLIP-style embedder."""
    import base64
    import io

    import numpy as np
    import torch

    transformers = pytest.importorskip("transformers")
    pil = pytest.importorskip("PIL.Image")
    from antfly_b200.models.clip import ClipConfig, ClipModel
    from antfly_b200.pipelines.multimodal import ClipEmbedder
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    torch.manual_seed(0)
    hf_cfg = transformers.CLIPConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                         num_attention_heads=4, max_position_embeddings=32, eos_token_id=2),
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                           image_size=32, patch_size=16), projection_dim=32)
    model = ClipModel.from_state_dict(ClipConfig.from_hf(hf_cfg.to_dict()), transformers.CLIPModel(hf_cfg).state_dict(),
                                      device="cpu", dtype=torch.float32)
    tok = ByteTokenizer(512)
    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register("tiny-clip", "embedder", ClipEmbedder(model, tok), tok)
    c = TestClient(create_app(mgr))
    buf = io.BytesIO()
    pil.fromarray(np.random.default_rng(0).integers(0, 256, size=(40, 60, 3), dtype=np.uint8)).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    r = c.post("/ai/v1/embed", json={"model": "tiny-clip", "input": [
        {"type": "text", "text": "a photo"}, {"type": "image_url", "image_url": {"url": url}},
        {"type": "text", "text": "another"}]})
    assert r.status_code == 200, r.text
    data = r.json()["data"]
    assert [d["index"] for d in data] == [0, 1, 2] and all(len(d["embedding"]) == 32 for d in data)
    assert all(abs(sum(v * v for v in d["embedding"]) - 1.0) < 1e-3 for d in data)
    r = c.post("/ai/v1/embed", json={"model": "tiny-clip", "input": [{"type": "image_url", "image_url": {"url": "http://x/y.png"}}]})
    assert r.status_code == 400 and "data:" in r.json()["message"]
    r = c.post("/ai/v1/embed", json={"model": "tiny-clip", "input": [{"type": "audio", "text": "x"}]})
    assert r.status_code == 400
    # multimodal rerank: image documents scored by the dual-tower model, text-only ones by the cross-encoder
    mgr.register_random("tiny-rerank", "reranker")
    r = c.post("/ai/v1/rerank_multimodal", json={"model": "tiny-clip", "query": "a photo", "documents": [
        {"id": "a", "content": [{"type": "image_url", "image_url": {"url": url}}]},
        {"id": "b", "content": [{"type": "text", "text": "a photo"}, {"type": "image_url", "image_url": {"url": url}}]},
        {"content": "just text"}]})
    body = r.json()
    assert r.status_code == 200 and [d["index"] for d in body["data"]] == [0, 1, 2]
    qv = c.post("/ai/v1/embed", json={"model": "tiny-clip", "input": "a photo"}).json()["data"][0]["embedding"]
    iv = data[1]["embedding"]
    assert abs(body["data"][0]["score"] - sum(x * y for x, y in zip(qv, iv))) < 1e-4
    assert body["data"][1]["score"] >= body["data"][0]["score"] - 1e-6 and body["data"][1]["score"] > 0.999
    r = c.post("/ai/v1/rerank_multimodal", json={"model": "tiny-rerank", "query": "q", "documents": [
        {"content": "first"}, {"content": [{"type": "text", "text": "second"}]}]})
    assert r.status_code == 200 and len(r.json()["data"]) == 2
    r = c.post("/ai/v1/rerank_multimodal", json={"model": "tiny-rerank", "query": "q", "documents": [
        {"content": [{"type": "image_url", "image_url": {"url": url}}]}]})
    assert r.status_code in (400, 404)
    assert c.post("/ai/v1/rerank_multimodal", json={"model": "tiny-clip", "query": "q",
                                                   "documents": []}).status_code == 400


def test_chunk_and_metrics(client):
    r = client.post("/ai/v1/chunk", json={"text": "a b c d e f g h i j", "target_tokens": 4, "overlap_tokens": 1})
    ch = r.json()["chunks"]
    assert ch[0]["text"] == "a b c d" and ch[1]["text"].startswith("d e") and ch[-1]["text"].endswith("j")
    text = client.get("/ai/v1/metrics").text
    assert "antfly_inference_requests_total" in text and 'endpoint="embed"' in text


def test_request_queue_backpressure():
    q = RequestQueue(max_units=1, max_waiting=0)
    q.acquire(1)
    with pytest.raises(QueueFull):
        q.acquire(1, timeout=0.05)
    q.release(1)
    q.acquire(1)


@pytest.mark.parametrize("index_type", ["flat", "hbc", "hnsw"])
def test_table_create_batch_and_hybrid_query(client, index_type):
    t = f"docs_{index_type}"
    r = client.post(f"/db/v1/tables/{t}", json={"embedder": "tiny-embed", "reranker": "tiny-rerank",
                                                 "index_type": index_type})
    assert r.status_code == 200 and r.json()["dimension"] == 128
    assert client.post(f"/db/v1/tables/{t}", json={}).status_code == 409
    texts = ["red apples and green apples", "how to bake an apple pie", "history of the roman empire",
             "roman roads and aqueducts", "a new phone was released", "height of the empire state building"]
    texts += [f"filler document number {i} about topic {i % 7}" for i in range(60)]
    r = client.post(f"/db/v1/tables/{t}/batch", json={"inserts": {f"k{i}": {"text": x, "n": i}
                                                                    for i, x in enumerate(texts)}})
    assert r.status_code == 200 and r.json() == {"inserted": 66, "deleted": 0, "count": 66}
    assert {"name": t, "count": 66} in client.get("/db/v1/tables").json()["tables"]
    # full text + semantic, fused with RRF; documents and per-index scores come back
    r = client.post(f"/db/v1/tables/{t}/query", json={"semantic_search": "roman empire",
                                                       "full_text_search": {"query": "roman empire"}, "limit": 5})
    body = r.json()["responses"][0]
    assert r.status_code == 200 and body["status"] == 200 and body["hits"]["total"] == 5
    top = body["hits"]["hits"][0]
    assert top["_id"] == "k2" and top["_source"]["text"] == texts[2] and "full_text" in top["_index_scores"]
    assert body["hits"]["max_score"] == top["_score"]
    # the document's own embedding finds it first; fields filter the source
    e = client.post("/ai/v1/embed", json={"model": "tiny-embed", "input": texts[1]}).json()["data"][0]["embedding"]
    r = client.post(f"/db/v1/tables/{t}/query", json={"embeddings": {"dense": e}, "limit": 3, "fields": ["n"]})
    h = r.json()["responses"][0]["hits"]["hits"]
    assert h[0]["_id"] == "k1" and h[0]["_source"] == {"n": 1} and set(h[0]["_index_scores"]) == {"dense"}
    # rerank stage, offset paging, deletes
    r = client.post(f"/db/v1/tables/{t}/query", json={"full_text_search": "apple", "limit": 2,
                                                       "reranker": {"query": "apple pie recipe"}})
    assert all("reranker" in x["_index_scores"] for x in r.json()["responses"][0]["hits"]["hits"])
    a = client.post(f"/db/v1/tables/{t}/query", json={"full_text_search": "roman", "limit": 2}).json()
    b = client.post(f"/db/v1/tables/{t}/query", json={"full_text_search": "roman", "limit": 1, "offset": 1}).json()
    assert b["responses"][0]["hits"]["hits"][0]["_id"] == a["responses"][0]["hits"]["hits"][1]["_id"]
    r = client.post(f"/db/v1/tables/{t}/batch", json={"deletes": ["k2", "nope"]})
    assert r.json()["deleted"] == 1 and r.json()["count"] == 65
    ids = [x["_id"] for x in client.post(f"/db/v1/tables/{t}/query", json={
        "semantic_search": "roman empire", "full_text_search": "roman empire", "limit": 10}).json()[
        "responses"][0]["hits"]["hits"]]
    assert "k2" not in ids
    assert client.post("/db/v1/tables/missing/query", json={"full_text_search": "x"}).status_code == 404
    assert client.post(f"/db/v1/tables/{t}/query", json={"limit": 0}).status_code == 400


def _write_bert(dirpath, num_labels, id2label, seed):
    import torch

    from antfly_b200.formats import safetensors_io as st
    from antfly_b200.models.bert import BertConfig, BertModel

    dirpath.mkdir(parents=True)
    cfg = BertConfig(hidden_size=64, num_hidden_layers=1, num_attention_heads=4, intermediate_size=128, vocab_size=300,
                     num_labels=num_labels)
    m = BertModel.random_init(cfg, device="cpu", seed=seed)
    if num_labels:
        m.w["cls.w"] = m.w["cls.w"] * 40.0               # decisive heads: random init gives near-uniform labels
    st.save_file(m.state_dict_hf(), str(dirpath / "model.safetensors"))
    (dirpath / "config.json").write_text(json.dumps({
        "model_type": "bert", "hidden_size": 64, "num_hidden_layers": 1, "num_attention_heads": 4,
        "intermediate_size": 128, "vocab_size": 300, "max_position_embeddings": 512, "num_labels": num_labels,
        "id2label": {str(i): l for i, l in enumerate(id2label)}}))


def _write_t5(dirpath):
    import torch

    from antfly_b200.formats import safetensors_io as st

    dirpath.mkdir(parents=True)
    g = torch.Generator().manual_seed(0)
    sd = {"shared.weight": torch.randn(300, 64, generator=g)}
    for stack, ff in (("encoder", 1), ("decoder", 2)):
        for l in range(2):
            s = f"{stack}.block.{l}.layer."
            for n in "qkvo":
                sd[s + f"0.SelfAttention.{n}.weight"] = torch.randn(64, 64, generator=g) * 0.2
                if stack == "decoder":
                    sd[s + f"1.EncDecAttention.{n}.weight"] = torch.randn(64, 64, generator=g) * 0.2
            sd[s + "0.layer_norm.weight"] = torch.ones(64)
            if stack == "decoder":
                sd[s + "1.layer_norm.weight"] = torch.ones(64)
            sd[s + f"{ff}.DenseReluDense.wi.weight"] = torch.randn(128, 64, generator=g) * 0.2
            sd[s + f"{ff}.DenseReluDense.wo.weight"] = torch.randn(64, 128, generator=g) * 0.2
            sd[s + f"{ff}.layer_norm.weight"] = torch.ones(64)
        sd[f"{stack}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"] = torch.randn(8, 4, generator=g)
        sd[f"{stack}.final_layer_norm.weight"] = torch.ones(64)
    st.save_file({k: v.contiguous() for k, v in sd.items()}, str(dirpath / "model.safetensors"))
    (dirpath / "config.json").write_text(json.dumps({
        "model_type": "t5", "vocab_size": 300, "d_model": 64, "d_kv": 16, "d_ff": 128, "num_layers": 2,
        "num_heads": 4, "relative_attention_num_buckets": 8, "relative_attention_max_distance": 20,
        "feed_forward_proj": "relu", "eos_token_id": 2, "decoder_start_token_id": 0}))


def test_rewrite_and_extract_endpoints(tmp_path):
    _write_t5(tmp_path / "rewriters" / "tiny-t5")
    _write_bert(tmp_path / "recognizers" / "tiny-ner", 5, ["O", "B-PER", "I-PER", "B-LOC", "I-LOC"], 1)
    _write_bert(tmp_path / "classifiers" / "tiny-clf", 3, ["negative", "neutral", "positive"], 2)
    c = TestClient(create_app(ModelManager(models_dir=str(tmp_path), device="cpu")))
    # rewrite: one object per input, usage accounting, greedy = deterministic
    r = c.post("/ai/v1/rewrite", json={"model": "tiny-t5", "inputs": ["translate: hello", "paraphrase: cats"],
                                      "max_tokens": 8})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "list" and body["model"] == "tiny-t5"
    assert [d["index"] for d in body["data"]] == [0, 1] and all(d["object"] == "rewrite" and len(d["texts"]) == 1
                                                               for d in body["data"])
    u = body["usage"]
    assert u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"] and 0 < u["completion_tokens"] <= 16
    assert c.post("/ai/v1/rewrite", json={"model": "tiny-t5", "inputs": ["translate: hello"],
                                         "max_tokens": 8}).json()["data"][0]["texts"] == body["data"][0]["texts"]
    assert c.post("/ai/v1/rewrite", json={"model": "nope", "inputs": ["x"]}).status_code == 404
    # extract: entities restricted to the schema's labels, spans index the input text, classifications per task
    text = "alice met bob in paris and then flew to rome"
    r = c.post("/ai/v1/extract", json={"model": "tiny-ner", "inputs": [{"id": "d1", "content": text}],
                                      "schema": {"entities": ["PER", "LOC"]}})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "extraction" and body["data"][0]["id"] == "d1"
    ents = body["data"][0]["entities"]
    assert ents and all(e["label"] in ("PER", "LOC") and 0 <= e["score"] <= 1 for e in ents)
    assert all(text[e["start"]:e["end"]] == e["text"] for e in ents if "start" in e)
    only = c.post("/ai/v1/extract", json={"model": "tiny-ner", "inputs": [{"content": text}],
                                         "schema": {"entities": ["LOC"]}}).json()["data"][0]["entities"]
    assert all(e["label"] == "LOC" for e in only) and len(only) <= len(ents)
    hi = c.post("/ai/v1/extract", json={"model": "tiny-ner", "inputs": [{"content": text}],
                                       "schema": {"entities": ["PER", "LOC"]}, "options": {"threshold": 1.1}})
    assert hi.json()["data"][0]["entities"] == []
    r = c.post("/ai/v1/extract", json={"model": "tiny-clf", "inputs": [{"content": "great movie"},
                                                                      {"content": [{"type": "text", "text": "bad"}]}],
                                      "schema": {"classifications": [{"name": "sentiment",
                                                                      "labels": ["negative", "positive"]}]}})
    cls = [d["classifications"] for d in r.json()["data"]]
    assert r.status_code == 200 and all(len(x) == 1 and x[0]["name"] == "sentiment" and
                                        x[0]["label"] in ("negative", "positive") for x in cls)
    assert c.post("/ai/v1/extract", json={"model": "tiny-clf", "inputs": [{"content": "x"}], "schema": {
        "classifications": [{"name": "t", "labels": ["sarcastic"]}]}}).status_code == 400
    assert c.post("/ai/v1/extract", json={"model": "tiny-clf", "inputs": [{"content": "x"}],
                                         "schema": {}}).status_code == 400
    # a model with entailment / contradiction labels classifies against labels it never saw (zero-shot)
    _write_bert(tmp_path / "classifiers" / "tiny-nli", 3, ["contradiction", "neutral", "entailment"], 4)
    r = c.post("/ai/v1/extract", json={"model": "tiny-nli", "inputs": [{"content": "the team won"}, {"content": "y"}],
                                      "schema": {"classifications": [
                                          {"name": "topic", "labels": ["sports", "politics", "cooking"]},
                                          {"name": "tone", "labels": ["happy", "sad"], "multi_label": True}]}})
    assert r.status_code == 200, r.text
    for d in r.json()["data"]:
        topic = [x for x in d["classifications"] if x["name"] == "topic"]
        tone = [x for x in d["classifications"] if x["name"] == "tone"]
        assert len(topic) == 1 and topic[0]["label"] in ("sports", "politics", "cooking") and 0 < topic[0]["score"] <= 1
        assert all(x["label"] in ("happy", "sad") and 0 <= x["score"] <= 1 for x in tone) and len(tone) == 2


def test_anthropic_messages_and_openai_path_compat(client):
    """Messages-API wire format over the native generate handler (request translation, content blocks, stop reasons,
    usage, named streaming events, error envelope) and the /openai/v1 path aliases."""
    from antfly_b200.api.compat import anthropic_to_generate

    body = {"model": "tiny-gen", "max_tokens": 6, "system": [{"type": "text", "text": "be brief"}],
            "messages": [{"role": "user", "content": [{"type": "text", "text": "hi there"}]}], "temperature": 0}
    g = anthropic_to_generate(body)
    assert g["messages"][0] == {"role": "system", "content": "be brief"} and g["messages"][1]["content"] == "hi there"
    t = anthropic_to_generate({"model": "m", "max_tokens": 5, "messages": [
        {"role": "user", "content": "weather?"},
        {"role": "assistant", "content": [{"type": "tool_use", "id": "toolu_1", "name": "get", "input": {"c": "x"}}]},
        {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "toolu_1", "content": "sunny"}]}],
        "tools": [{"name": "get", "description": "d", "input_schema": {"type": "object"}}],
        "tool_choice": {"type": "any"}, "stop_sequences": ["END"]})
    assert [m["role"] for m in t["messages"]] == ["user", "assistant", "tool"]
    assert t["messages"][1]["tool_calls"][0]["function"] == {"name": "get", "arguments": '{"c": "x"}'}
    assert t["messages"][2] == {"role": "tool", "tool_call_id": "toolu_1", "content": "sunny"}
    assert t["tools"][0]["function"]["name"] == "get" and t["tool_choice"] == "required" and t["stop"] == ["END"]

    r = client.post("/anthropic/v1/messages", json=body)
    m = r.json()
    assert r.status_code == 200 and m["type"] == "message" and m["role"] == "assistant" and m["model"] == "tiny-gen"
    assert m["id"].startswith("msg_") and m["stop_reason"] in ("max_tokens", "end_turn") and m["stop_sequence"] is None
    assert m["usage"]["input_tokens"] > 0 and 0 < m["usage"]["output_tokens"] <= 6
    assert all(b["type"] == "text" for b in m["content"])
    # same tokens as the native endpoint (greedy)
    n = client.post("/ai/v1/generate", json={"model": "tiny-gen", "max_tokens": 6, "temperature": 0, "messages": [
        {"role": "system", "content": "be brief"}, {"role": "user", "content": "hi there"}]}).json()
    assert (m["content"][0]["text"] if m["content"] else None) == n["choices"][0]["message"]["content"]
    # streaming: named events in order, text deltas concatenate to the non-streamed text
    with client.stream("POST", "/anthropic/v1/messages", json={**body, "stream": True}) as s:
        raw = "".join(s.iter_text())
    events = [blk.split("\n") for blk in raw.strip().split("\n\n")]
    names = [e[0].split(": ", 1)[1] for e in events]
    assert names[0] == "message_start" and names[-2:] == ["message_delta", "message_stop"] and "[DONE]" not in raw
    datas = [json.loads(e[1].split(": ", 1)[1]) for e in events]
    text = "".join(d["delta"]["text"] for d in datas if d["type"] == "content_block_delta")
    assert text == (m["content"][0]["text"] if m["content"] else "")
    if text:
        assert names.count("content_block_start") == names.count("content_block_stop") == 1
    md = datas[names.index("message_delta")]
    assert md["delta"]["stop_reason"] == m["stop_reason"] and md["usage"]["output_tokens"] == m["usage"]["output_tokens"]
    # errors use the Messages-API envelope
    e = client.post("/anthropic/v1/messages", json={"model": "tiny-gen", "messages": [{"role": "user", "content": "x"}]})
    assert e.status_code == 400 and e.json()["type"] == "error" and e.json()["error"]["type"] == "invalid_request_error"
    e = client.post("/anthropic/v1/messages", json={**body, "model": "missing"})
    assert e.status_code == 404 and e.json()["error"]["type"] == "not_found_error"
    # OpenAI path aliases
    o = client.post("/openai/v1/chat/completions", json={"model": "tiny-gen", "max_tokens": 4, "temperature": 0,
                                                         "messages": [{"role": "user", "content": "hi"}]})
    assert o.status_code == 200 and o.json()["object"] == "chat.completion"
    ids = [x["id"] for x in client.get("/openai/v1/models").json()["data"]]
    assert "tiny-gen" in ids and "tiny-embed" in ids
    assert client.post("/openai/v1/embeddings", json={"model": "tiny-embed", "input": "x"}).status_code == 200


def test_result_cache_serves_repeated_texts_and_expires():
    from antfly_b200.api.cache import ResultCache

    now = [0.0]
    c = ResultCache(ttl_s=120, max_entries=3, clock=lambda: now[0])
    k = ResultCache.key("embed", "m", None, None, "text")
    assert k != ResultCache.key("embed", "m", None, None, "text ") and c.get(k) is None
    c.put(k, [1.0])
    now[0] = 119
    assert c.get(k) == [1.0]
    now[0] = 121
    assert c.get(k) is None and len(c) == 0 and (c.hits, c.misses) == (1, 2)
    for i in range(5):
        c.put(i, i)
    assert len(c) == 3 and c.get(0) is None and c.get(4) == 4          # bounded, oldest evicted

    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register_random("e", "embedder")
    mgr.register_random("r", "reranker")
    cl = TestClient(create_app(mgr))
    a = cl.post("/ai/v1/embed", json={"model": "e", "input": ["alpha", "beta"]}).json()
    b = cl.post("/ai/v1/embed", json={"model": "e", "input": ["beta", "gamma", "alpha"]}).json()
    assert b["data"][0]["embedding"] == a["data"][1]["embedding"] and b["data"][2]["embedding"] == a["data"][0]["embedding"]
    assert b["usage"]["prompt_tokens"] > a["usage"]["prompt_tokens"]     # usage counts cached texts too
    s1 = cl.post("/ai/v1/rerank", json={"model": "r", "query": "q", "prompts": ["x", "y"]}).json()
    s2 = cl.post("/ai/v1/rerank", json={"model": "r", "query": "q", "prompts": ["y", "x"]}).json()
    assert s2["data"][0]["score"] == s1["data"][1]["score"]
    assert s2["usage"]["prompt_tokens"] == s1["usage"]["prompt_tokens"]
    m = cl.get("/metrics").text
    assert 'antfly_inference_result_cache_total{endpoint="embed",outcome="hit"} 2.0' in m
    assert 'antfly_inference_result_cache_total{endpoint="rerank",outcome="hit"} 2.0' in m


def test_required_tool_choice_always_yields_a_valid_call(client):
    tools = [{"type": "function", "function": {"name": "set_flag", "parameters": {
        "type": "object", "properties": {"on": {"type": "boolean"}}, "required": ["on"]}}}]
    r = client.post("/ai/v1/chat/completions", json={
        "model": "tiny-gen", "messages": [{"role": "user", "content": "do it"}], "max_tokens": 120, "temperature": 0,
        "tools": tools, "tool_choice": "required"})
    assert r.status_code == 200, r.text
    ch = r.json()["choices"][0]
    if ch["finish_reason"] == "tool_calls":     # (random weights may spend the budget on optional whitespace)
        call = ch["message"]["tool_calls"][0]["function"]
        assert call["name"] == "set_flag" and isinstance(json.loads(call["arguments"])["on"], bool)
    else:
        assert ch["finish_reason"] == "length"
    r = client.post("/ai/v1/chat/completions", json={
        "model": "tiny-gen", "messages": [{"role": "user", "content": "x"}], "tools": tools,
        "tool_choice": {"type": "function", "function": {"name": "missing"}}})
    assert r.status_code == 400


def test_api_key_guards_everything_but_the_probes():
    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register_random("e", "embedder")
    c = TestClient(create_app(mgr, api_key="s3cret"))
    assert c.get("/healthz").status_code == 200 and c.get("/readyz").status_code == 200
    r = c.post("/ai/v1/embed", json={"model": "e", "input": "x"})
    assert r.status_code == 401 and r.json()["error"] == "unauthorized"
    assert c.get("/ai/v1/models", headers={"Authorization": "Bearer wrong"}).status_code == 401
    assert c.post("/ai/v1/embed", json={"model": "e", "input": "x"},
                  headers={"Authorization": "Bearer s3cret"}).status_code == 200
    assert c.get("/metrics", headers={"X-API-Key": "s3cret"}).status_code == 200


def test_read_endpoint_with_a_tiny_vision_encoder_decoder(tmp_path):
    """/ai/v1/read: data-URL image -> device preprocessing -> ViT -> TrOCR decoder -> text."""
    import base64
    import io

    import numpy as np
    import torch

    transformers = pytest.importorskip("transformers")
    pil = pytest.importorskip("PIL.Image")
    from antfly_b200.formats import safetensors_io as st

    torch.manual_seed(0)
    enc = transformers.ViTConfig(hidden_size=48, num_hidden_layers=1, num_attention_heads=4, intermediate_size=96,
                                 image_size=32, patch_size=8)
    dec = transformers.TrOCRConfig(vocab_size=300, d_model=64, decoder_layers=1, decoder_attention_heads=4,
                                   decoder_ffn_dim=128, max_position_embeddings=40, cross_attention_hidden_size=48,
                                   decoder_start_token_id=2, eos_token_id=2, pad_token_id=1)
    hf_cfg = transformers.VisionEncoderDecoderConfig.from_encoder_decoder_configs(enc, dec)
    hf = transformers.VisionEncoderDecoderModel(hf_cfg)
    d = tmp_path / "readers" / "tiny-ocr"
    d.mkdir(parents=True)
    st.save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(hf_cfg.to_dict(), default=str))
    (d / "preprocessor_config.json").write_text(json.dumps({"image_mean": [0.5, 0.5, 0.5], "image_std": [0.5, 0.5, 0.5],
                                                            "resample": 2, "size": {"height": 32, "width": 32}}))
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")
    c = TestClient(create_app(mgr))
    buf = io.BytesIO()
    img = np.random.default_rng(0).integers(0, 256, size=(20, 90, 3), dtype=np.uint8)
    pil.fromarray(img).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    r = c.post("/ai/v1/read", json={"model": "tiny-ocr", "images": [{"url": url}, url], "max_tokens": 5})
    body = r.json()
    assert r.status_code == 200, r.text
    assert body["object"] == "list" and [x["index"] for x in body["data"]] == [0, 1]
    assert body["data"][0]["text"] == body["data"][1]["text"] and body["usage"]["completion_tokens"] <= 10
    # same tokens as driving the model directly on the same preprocessed pixels
    pipe = mgr.get("tiny-ocr", "reader").pipeline
    direct = pipe.model.read_ids(pipe.preprocess(torch.from_numpy(img)), 5)
    assert pipe.read([torch.from_numpy(img)], 5)[0].token_ids == direct
    assert c.post("/ai/v1/read", json={"model": "tiny-ocr", "images": ["http://x/y.png"]}).status_code == 400
    assert c.post("/ai/v1/read", json={"model": "tiny-ocr", "images": []}).status_code == 400
    assert c.post("/ai/v1/read", json={"model": "nope", "images": [url]}).status_code == 404


def test_neural_chunker_splits_at_predicted_boundaries(tmp_path):
    """A token-classification chunker model: chunks cover the text in order, respect the token cap, and are cut
    where the model says so."""
    import torch

    from antfly_b200.pipelines.chunking import NeuralChunker

    _write_bert(tmp_path / "chunkers" / "tiny-chunker", 2, ["O", "separator"], 5)
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")
    tagger = mgr.get("tiny-chunker", "chunker").pipeline
    text = "First sentence here. Second one follows! And a third, somewhat longer, closes the paragraph.\n\nNew part."
    ch = NeuralChunker(tagger).chunk(text, max_tokens=30, min_tokens=4)
    assert ch and ch[0]["start_char"] == 0 and ch[-1]["end_char"] == len(text)
    assert all(c["tokens"] <= 30 and c["text"] == text[c["start_char"]:c["end_char"]] for c in ch)
    assert all(a["end_char"] <= b["start_char"] for a, b in zip(ch, ch[1:]))
    assert "".join(c["text"] for c in ch).replace(" ", "") in text.replace(" ", "") or len(ch) > 1
    # boundaries come from the model: forcing every token to be a separator yields chunks of exactly min_tokens
    class Always:
        tokenizer = tagger.tokenizer

        def tag_ids(self, seqs):
            return [(["separator"] * len(s), [1.0] * len(s)) for s in seqs]

    every = NeuralChunker(Always()).chunk(text, max_tokens=30, min_tokens=5)
    assert all(c["tokens"] == 5 for c in every[:-1]) and len(every) > 5
    none = NeuralChunker(Always(), boundary_labels=("never",)).chunk(text, max_tokens=30)
    assert all(c["tokens"] == 30 for c in none[:-1])
    c = TestClient(create_app(mgr))
    r = c.post("/ai/v1/chunk", json={"text": text, "model": "tiny-chunker", "target_tokens": 30})
    assert r.status_code == 200 and r.json()["chunks"][0]["start_char"] == 0
    assert c.post("/ai/v1/chunk", json={"text": text, "model": "missing"}).status_code == 404
    assert c.post("/ai/v1/chunk", json={"text": "a b c d", "target_tokens": 2, "overlap_tokens": 0}).json()[
        "chunks"][0]["text"] == "a b"


def test_generate_with_draft_model_and_cache_dtype_per_request():
    """``draft_model`` loads a second generator as the speculative draft (own KV cache), ``speculative_k`` sets the
    round length, ``cache_dtype`` selects the KV-cache codec; greedy output never depends on the draft, and the
    speculative stats show up in the metrics."""
    mgr = ModelManager(models_dir="/nonexistent", device="cpu", kv_blocks=128, max_batch=4)
    mgr.register_random("target", "generator", seed=0)
    mgr.register_random("small", "generator", seed=7)
    c = TestClient(create_app(mgr))
    base = {"model": "target", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 9, "temperature": 0}
    plain = c.post("/ai/v1/chat/completions", json=base).json()["choices"][0]["message"]["content"]
    r = c.post("/ai/v1/chat/completions", json=dict(base, draft_model="small", speculative_k=3))
    assert r.status_code == 200, r.text
    assert r.json()["choices"][0]["message"]["content"] == plain
    variant = mgr.get_generator("target", "small", None)
    assert variant.pipeline.engine.draft_cache is not None and variant.pipeline.engine.spec.rounds > 0
    assert variant.pipeline.engine.model is mgr.get("target", "generator").pipeline.engine.model   # weights shared
    # quantised caches: served, and a different engine per dtype
    for dt in ("fp8", "int8", "int4", "f16", "f32"):
        r = c.post("/ai/v1/chat/completions", json=dict(base, cache_dtype=dt))
        assert r.status_code == 200, (dt, r.text)
    assert mgr.get_generator("target", None, "int8").pipeline.engine.cache.codec == "int8"
    assert mgr.get_generator("target", None, "f16") is mgr.get("target", "generator")
    # errors: unknown draft model, draft equal to the target
    assert c.post("/ai/v1/chat/completions", json=dict(base, draft_model="nope")).status_code == 404
    assert c.post("/ai/v1/chat/completions", json=dict(base, draft_model="target")).status_code == 400
    assert c.post("/ai/v1/chat/completions", json=dict(base, cache_dtype="int3")).status_code in (400, 422)


def test_classify_and_recognize_endpoints(tmp_path):
    """/ai/v1/classify over a trained head (its own labels, optionally restricted) and /ai/v1/recognize over a token
    classifier and over a zero-shot span model with relations and a resolver section."""
    from antfly_b200.pipelines import gliner as G

    _write_bert(tmp_path / "classifiers" / "clf", 3, ["negative", "neutral", "positive"], 2)
    _write_bert(tmp_path / "recognizers" / "ner", 3, ["O", "B-PER", "I-PER"], 1)
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")

    class Fake:
        def recognize(self, texts, labels, threshold=None):
            E = G.GlinerEntity
            return [[E("Zoë", "person", 0, 4, 0.9), E("Paris", "city", 14, 19, 0.8)], [E("zoë", "person", 0, 4, 0.7)]][: len(texts)]

        def extract_relations(self, texts, ents, rels):
            e = self.recognize(texts, ents)
            return e, [[G.GlinerRelation(e[0][0], e[0][1], rels[0], 0.6)], []][: len(texts)]

        def classify(self, text, labels, threshold=0.0, multi_label=False):
            return [(labels[0], 0.75)] + [(l, 0.1) for l in labels[1:]]

    mgr.register("span", "recognizer", Fake(), None)
    mgr.register("span", "classifier", Fake(), None)
    c = TestClient(create_app(mgr))
    r = c.post("/ai/v1/classify", json={"model": "clf", "texts": ["good", "bad"]})
    assert r.status_code == 200, r.text
    body = r.json()
    assert body["object"] == "list" and [d["index"] for d in body["data"]] == [0, 1]
    row = body["data"][0]["classifications"]
    assert body["data"][0]["object"] == "classification" and {x["label"] for x in row} == {"negative", "neutral", "positive"}
    assert abs(sum(x["score"] for x in row) - 1.0) < 1e-3 and row[0]["score"] >= row[1]["score"]
    r = c.post("/ai/v1/classify", json={"model": "clf", "texts": ["good"], "labels": ["positive"]})
    assert [x["label"] for x in r.json()["data"][0]["classifications"]] == ["positive"]
    r = c.post("/ai/v1/classify", json={"model": "span", "texts": ["good"], "labels": ["a", "b"]})
    assert r.json()["data"][0]["classifications"][0] == {"label": "a", "score": 0.75}
    assert c.post("/ai/v1/classify", json={"model": "span", "texts": ["good"]}).status_code == 400
    assert c.post("/ai/v1/classify", json={"model": "clf", "texts": []}).status_code == 400
    r = c.post("/ai/v1/recognize", json={"model": "ner", "texts": ["alice went home"]})
    assert r.status_code == 200 and r.json()["data"][0]["object"] == "recognition" and "entities" in r.json()["data"][0]
    r = c.post("/ai/v1/recognize", json={"model": "span", "texts": ["Zoë lives in Paris", "zoë again"],
                                         "labels": ["person", "city"], "relation_labels": ["lives_in"],
                                         "resolver": {"similarity_threshold": 0.8}})
    assert r.status_code == 200, r.text
    out = r.json()
    e0 = out["data"][0]["entities"]
    assert e0[0] == {"text": "Zoë", "label": "person", "start": 0, "end": 3, "score": 0.9}       # characters, not bytes
    assert e0[1]["start"] == 13 and e0[1]["end"] == 18
    rel = out["data"][0]["relations"][0]
    assert rel["label"] == "lives_in" and rel["head"]["text"] == "Zoë" and rel["tail"]["text"] == "Paris"
    assert out["data"][1]["relations"] == []
    kg = out["knowledge_graph"]
    assert [e["name"] for e in kg["entities"]] == ["Zoë", "Paris"] and kg["entities"][0]["inputs"] == [0, 1]
    assert kg["relations"][0]["type"] == "lives_in"
    assert "knowledge_graph" not in c.post("/ai/v1/recognize", json={"model": "span", "texts": ["x"]}).json()
