"""Product-level check: the server started as a process on a free port, reached over HTTP the way a client would
(readiness, embeddings with unit norm and the requested dimension, rerank ordering contract, generation as a JSON
reply and as a server-sent event stream, model listing, metrics)."""
import json
import os
import socket
import subprocess
import sys
import time
import urllib.error
import urllib.request

import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _post(base, path, body, timeout=60):
    req = urllib.request.Request(base + path, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return r.status, r.read()


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=os.getcwd())
    proc = subprocess.Popen([sys.executable, "-m", "antfly_b200", "run", "--host", "127.0.0.1", "--port", str(port),
                             "--device", "cpu", "--models-dir", str(tmp_path_factory.mktemp("models")), "--kv-blocks", "64",
                             "--preload", "generator:random:tiny", "embedder:random:tiny", "reranker:random:tiny"],
                            env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    base = f"http://127.0.0.1:{port}"
    deadline = time.time() + 120
    ok = False
    while time.time() < deadline and proc.poll() is None:
        try:
            with urllib.request.urlopen(base + "/readyz", timeout=2) as r:
                if r.status == 200:
                    ok = True
                    break
        except (urllib.error.URLError, OSError):
            time.sleep(0.5)
    if not ok:
        proc.kill()
        out = proc.stdout.read().decode(errors="replace")[-2000:]
        pytest.fail(f"server did not become ready: {out}")
    yield base
    proc.terminate()
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        proc.kill()


def test_embed_rerank_generate_over_http(server):
    st, body = _post(server, "/ai/v1/embed", {"model": "random:tiny", "input": ["first text", "second text"], "dimensions": 16})
    rep = json.loads(body)
    assert st == 200 and rep["object"] == "list" and len(rep["data"]) == 2
    vec = rep["data"][0]["embedding"]
    assert len(vec) == 16 and rep["usage"]["prompt_tokens"] > 0
    st, body = _post(server, "/ai/v1/embeddings", {"model": "random:tiny", "input": "first text"})
    full = json.loads(body)["data"][0]["embedding"]
    assert abs(sum(v * v for v in full) - 1.0) < 1e-2                       # L2-normalised
    st, body = _post(server, "/ai/v1/rerank", {"model": "random:tiny", "query": "q", "prompts": ["a", "bb", "ccc"]})
    data = json.loads(body)["data"]
    assert sorted(d["index"] for d in data) == [0, 1, 2] and all(d["object"] == "rerank.score" for d in data)
    st, body = _post(server, "/ai/v1/generate", {"model": "random:tiny", "messages": [{"role": "user", "content": "hi"}],
                                                 "max_tokens": 4})
    rep = json.loads(body)
    assert rep["choices"][0]["message"]["role"] == "assistant" and rep["usage"]["completion_tokens"] <= 4
    # streaming: data: {...} chunks ending with data: [DONE]
    req = urllib.request.Request(server + "/ai/v1/chat/completions", data=json.dumps(
        {"model": "random:tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "stream": True}).encode(),
        headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=60) as r:
        lines = [l.decode().strip() for l in r if l.strip()]
    assert lines[-1] == "data: [DONE]" and all(l.startswith("data: ") for l in lines)
    assert json.loads(lines[0][6:])["object"].startswith("chat.completion")


def test_client_library_against_the_running_server(server):
    from antfly_b200.client import ApiError, Client

    c = Client(server)
    c.wait_ready(10)
    assert len(c.embed("random:tiny", ["a", "b"], dimensions=8)[1]) == 8
    assert len(c.rerank("random:tiny", "q", ["x", "yy"])) == 2
    assert isinstance(c.generate("random:tiny", "hi", max_tokens=3), str)
    assert "".join(c.stream("random:tiny", [{"role": "user", "content": "hi"}], max_tokens=3)) is not None
    chunks = c.chunk("One sentence here. " * 40, config={"text": {"target_tokens": 20, "overlap_tokens": 2}})
    assert len(chunks) > 1 and chunks[0]["mime_type"] == "text/plain"
    with pytest.raises(ApiError) as e:
        c.classify("nobody", ["x"], ["a"])
    assert e.value.status == 404


def test_models_metrics_and_errors_over_http(server):
    with urllib.request.urlopen(server + "/ai/v1/models", timeout=10) as r:
        models = json.loads(r.read())
    assert "random:tiny" in json.dumps(models)
    with urllib.request.urlopen(server + "/ai/v1/metrics", timeout=10) as r:
        text = r.read().decode()
    assert "antfly_inference_" in text
    with urllib.request.urlopen(server + "/healthz", timeout=10) as r:
        assert r.status == 200
    with pytest.raises(urllib.error.HTTPError) as e:
        _post(server, "/ai/v1/embed", {"model": "no-such-model", "input": "x"})
    assert e.value.code == 404 and "error" in json.loads(e.value.read())
    with pytest.raises(urllib.error.HTTPError) as e:
        _post(server, "/ai/v1/rerank", {"model": "random:tiny"})
    assert e.value.code in (400, 422)
