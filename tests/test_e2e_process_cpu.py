"""Product-level test: start the real server process on a free port, wait for /readyz, and talk to it over HTTP with
the bundled client -- the shape of the reference's e2e suites (zig/e2e/inference/conftest.py:72-112,
test_embed.py:37-85, test_rerank.py:27-50): embedding dimension and unit norm, rerank ordering contract, chat and
streaming, error envelope, hybrid table round trip, metrics."""
import math
import os
import signal
import socket
import subprocess
import sys
import textwrap

import pytest

from antfly_b200.client import ApiError, Client


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    port = _free_port()
    cfg = tmp_path_factory.mktemp("cfg") / "inference.yaml"
    cfg.write_text(textwrap.dedent(f"""\
        api_url: http://127.0.0.1:{port}
        models_dir: {tmp_path_factory.mktemp("models")}
        keep_alive: 10m
        max_concurrent_requests: 8
        max_queue_size: 16
        preload: ["embedder:random:tiny", "reranker:random:tiny", "generator:random:tiny"]
        log: {{level: info, style: json}}
        """))
    env = {**os.environ, "PYTHONPATH": os.path.dirname(os.path.dirname(os.path.abspath(__file__)))}
    proc = subprocess.Popen([sys.executable, "-m", "antfly_b200", "run", "--config", str(cfg), "--device", "cpu",
                             "--kv-blocks", "128"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    c = Client(f"http://127.0.0.1:{port}")
    try:
        c.wait_ready(180)
    except Exception:
        proc.kill()
        out, err = proc.communicate(timeout=10)
        raise AssertionError("server did not start:\n" + err.decode()[-3000:])
    yield c, proc
    proc.send_signal(signal.SIGTERM)
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        proc.kill()


def test_process_level_round_trips(server):
    c, proc = server
    m = c.models()
    assert "random:tiny" in m["embedders"] and "random:tiny" in m["generators"]
    emb = c.embed("random:tiny", ["the cat sat", "a dog ran", "the cat sat"])
    assert len(emb) == 3 and len(emb[0]) == 128 and emb[0] == emb[2]
    assert all(abs(math.sqrt(sum(x * x for x in e)) - 1.0) < 1e-2 for e in emb)
    assert len(c.embed("random:tiny", "one", dimensions=16)[0]) == 16
    scores = c.rerank("random:tiny", "query", ["doc one", "doc two", "doc three"])
    assert len(scores) == 3 and all(0.0 <= s <= 1.0 for s in scores)
    text = c.generate("random:tiny", "hello", max_tokens=6, temperature=0)
    streamed = "".join(c.stream("random:tiny", [{"role": "user", "content": "hello"}], max_tokens=6, temperature=0))
    assert streamed and text.startswith(streamed)      # deltas hold back incomplete UTF-8 tails (random bytes)
    with pytest.raises(ApiError) as e:
        c.embed("no-such-model", "x")
    assert e.value.status == 404 and e.value.code == "model_not_found"
    c.create_table("docs", embedder="random:tiny")
    c.upsert("docs", {f"k{i}": {"text": t} for i, t in enumerate(["red apples", "green pears", "roman roads"])})
    hits = c.query("docs", full_text_search="roman", semantic_search="roman roads", limit=2)
    assert hits[0]["_id"] == "k2" and set(hits[0]["_index_scores"]) == {"dense", "full_text"}
    metrics = c.s.get(c.base + "/metrics").text
    assert 'antfly_inference_requests_total{endpoint="embed",status="200"}' in metrics
    assert proc.poll() is None
