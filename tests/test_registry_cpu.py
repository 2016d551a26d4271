"""Model references, file selection per variant, pull from a mirror directory and from an HTTP hub (a server on the
loopback interface), resume, checksum, manifest synthesis, discovery."""
import hashlib
import http.server
import json
import os
import threading

import pytest

from antfly_b200 import registry as R


def F(*names):
    return [R.HubFile(n, 10) for n in names]


def test_model_ref_forms():
    assert R.ModelRef.parse("hf:BAAI/bge-small-en-v1.5") == R.ModelRef("BAAI", "bge-small-en-v1.5", "auto")
    assert R.ModelRef.parse("unsloth/Qwen3-8B-GGUF:gguf:Q4_K_M").variant == "gguf:Q4_K_M"
    assert R.ModelRef.parse("a/b:safetensors").variant == "safetensors"
    for bad in ("nameonly", "/b", "a/", "a/b:"):
        with pytest.raises(R.RegistryError):
            R.ModelRef.parse(bad)


def test_gguf_selection_prefers_small_quants_and_whole_tags():
    files = F("config.json", "m-Q8_0.gguf", "m-Q4_K_M.gguf", "m-Q4_K_S.gguf", "m-F16.gguf", "mmproj-m-f16.gguf")
    names = lambda fs: [f.name for f in fs]
    assert names(R.select_gguf(files, None)) == ["m-Q4_K_S.gguf"]
    assert names(R.select_gguf(files, "Q8_0")) == ["m-Q8_0.gguf"]
    assert names(R.select_gguf(files, "q4_k_m")) == ["m-Q4_K_M.gguf"]
    assert R.select_gguf(files, "Q4_K") == []                       # a prefix of other tags is not a match
    assert R.select_gguf(files, "Q5_K_M") == []
    assert names(R.select_gguf(F("x.F16.gguf", "x.BF16.gguf"), None)) == ["x.BF16.gguf"]   # nothing preferred: first by name
    assert names(R.select_projector(files)) == ["mmproj-m-f16.gguf"]
    split = F("big-Q4_K_M-00001-of-00002.gguf", "big-Q4_K_M-00002-of-00002.gguf", "big-Q8_0-00001-of-00001.gguf")
    assert names(R.select_gguf(split, "Q4_K_M")) == ["big-Q4_K_M-00001-of-00002.gguf", "big-Q4_K_M-00002-of-00002.gguf"]


def test_variant_file_sets():
    files = F("config.json", "tokenizer.json", "README.md", "model.onnx", "onnx/model_quantized.onnx",
              "model.safetensors.index.json", "model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors",
              "extra.safetensors", "w-Q4_K_M.gguf", "mmproj-w-f16.gguf", "adapter_config.json")
    shards = lambda idx: ["model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors",
                          "model-00001-of-00002.safetensors"]
    names = lambda v: [f.name for f in R.select_files(files, v, shards)]
    st = ["model.safetensors.index.json", "model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"]
    base = ["config.json", "tokenizer.json", "adapter_config.json"]
    assert names("safetensors") == base + st
    assert names("gguf") == base + ["w-Q4_K_M.gguf"]
    assert names("auto") == base + ["w-Q4_K_M.gguf"] + st
    assert names("mmproj") == ["mmproj-w-f16.gguf"]
    assert names("onnx") == base + st                               # no ONNX lane: the safetensors fallback
    assert not any(n.endswith(".onnx") or n == "README.md" for v in ("auto", "onnx", "hybrid") for n in names(v))
    with pytest.raises(R.RegistryError):
        names("gguf:Q2_K")
    with pytest.raises(R.RegistryError):
        names("tflite")
    with pytest.raises(R.RegistryError):
        R.select_files(F("config.json", "model.onnx"), "onnx")
    with pytest.raises(R.RegistryError):                            # an index naming a shard the hub does not have
        R.select_files(F("model.safetensors.index.json"), "safetensors", lambda idx: ["gone.safetensors"])


def _repo(root, owner, name, files):
    d = os.path.join(root, owner, name)
    for rel, data in files.items():
        p = os.path.join(d, rel)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        with open(p, "wb") as f:
            f.write(data)
    return d


CONFIG = json.dumps({"architectures": ["LlamaForCausalLM"], "model_type": "llama"}).encode()


def test_pull_from_mirror_directory_writes_manifest_and_discovers(tmp_path):
    mirror, models = str(tmp_path / "mirror"), str(tmp_path / "models")
    idx = json.dumps({"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}})
    _repo(mirror, "acme", "tiny", {"config.json": CONFIG, "tokenizer.json": b"{}", "notes.txt": b"skip me",
                                    "tokenizer_config.json": json.dumps({"chat_template": "{{ messages }}"}).encode(),
                                    "model.safetensors.index.json": idx.encode(),
                                    "model-00001-of-00002.safetensors": b"A" * 100,
                                    "model-00002-of-00002.safetensors": b"B" * 50,
                                    "1_Pooling/config.json": b"{}"})
    seen = []
    dest = R.pull("hf:acme/tiny:safetensors", models, R.Hub("file://" + mirror),
                  progress=lambda n, done, total: seen.append((n, done, total)))
    assert dest == os.path.join(os.path.realpath(models), "acme", "tiny")
    got = sorted(os.path.relpath(os.path.join(d, n), dest) for d, _, ns in os.walk(dest) for n in ns)
    assert got == ["1_Pooling/config.json", "config.json", "model-00001-of-00002.safetensors",
                   "model-00002-of-00002.safetensors", "model.safetensors.index.json", "model_manifest.json",
                   "tokenizer.json", "tokenizer_config.json"]
    man = json.load(open(os.path.join(dest, "model_manifest.json")))
    assert man == {"type": "generator", "tasks": ["generate"], "capabilities": ["chat"]}
    assert ("model-00001-of-00002.safetensors", 100, 100) in seen
    # a second pull with tasks rewrites the manifest; the files already there are not copied again
    seen.clear()
    R.pull("acme/tiny:safetensors", models, R.Hub(mirror), tasks="embed, rerank", capabilities="long_context")
    man = json.load(open(os.path.join(dest, "model_manifest.json")))
    assert man["type"] == "reranker" and man["tasks"] == ["embed", "rerank"] and "long_context" in man["capabilities"]
    _repo(models, "rerankers", "bare", {"config.json": b"{}", "model.safetensors": b"x"})
    ents = {e.name: e for e in R.discover(models)}
    assert ents["acme/tiny"].kind == "reranker" and ents["acme/tiny"].variant == "safetensors"
    assert ents["bare"].kind == "reranker"
    assert R.resolve_variant(models, "hf:acme/tiny:safetensors") == os.path.join(models, "acme", "tiny")
    with pytest.raises(R.RegistryError):
        R.pull("acme/absent", models, R.Hub(mirror))


class _Handler(http.server.BaseHTTPRequestHandler):
    repo = {}
    ranges = []
    truncate = {}

    def log_message(self, *a):
        pass

    def do_GET(self):
        path = self.path.split("?")[0]
        if path == "/api/models/acme/web":
            sib = []
            for n, data in self.repo.items():
                e = {"rfilename": n}
                if n.endswith(".gguf"):
                    e["lfs"] = {"size": len(data), "sha256": hashlib.sha256(data).hexdigest()}
                else:
                    e["size"] = len(data)
                sib.append(e)
            body = json.dumps({"siblings": sib}).encode()
            self.send_response(200); self.send_header("Content-Length", str(len(body))); self.end_headers()
            self.wfile.write(body)
            return
        pre = "/acme/web/resolve/main/"
        if path.startswith(pre) and path[len(pre):] in self.repo:
            if self.headers.get("Authorization") != "Bearer s3cret":
                self.send_response(401); self.end_headers(); return
            name = path[len(pre):]
            data = self.repo[name]
            rng = self.headers.get("Range")
            start = 0
            if rng:
                start = int(rng.split("=")[1].split("-")[0])
                type(self).ranges.append((name, start))
                self.send_response(206)
            else:
                self.send_response(200)
            body = data[start:]
            cut = type(self).truncate.pop(name, None)
            if cut is not None:
                body = body[:cut]
            self.send_header("Content-Length", str(len(body))); self.end_headers()
            self.wfile.write(body)
            return
        self.send_response(404); self.end_headers()


def test_pull_over_http_with_token_resume_and_checksum(tmp_path):
    weights = bytes(range(256)) * 40
    _Handler.repo = {"config.json": CONFIG, "w-Q4_K_M.gguf": weights, "w-Q8_0.gguf": b"big" * 10, "model.onnx": b"o"}
    _Handler.ranges, _Handler.truncate = [], {"w-Q4_K_M.gguf": 1000}
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _Handler)
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    try:
        base = f"http://127.0.0.1:{srv.server_address[1]}"
        models = str(tmp_path / "models")
        with pytest.raises(R.RegistryError, match="access denied"):
            R.pull("acme/web:gguf", models, R.Hub(base, token="wrong"))
        hub = R.Hub(base, token="s3cret")
        with pytest.raises(R.RegistryError, match="resume"):          # the server cut the first transfer short
            R.pull("acme/web:gguf", models, hub)
        dest = os.path.join(os.path.realpath(models), "acme", "web")
        assert os.path.getsize(os.path.join(dest, "w-Q4_K_M.gguf.part")) == 1000
        R.pull("acme/web:gguf", models, hub)
        assert ("w-Q4_K_M.gguf", 1000) in _Handler.ranges              # resumed, not restarted
        assert open(os.path.join(dest, "w-Q4_K_M.gguf"), "rb").read() == weights
        assert sorted(os.listdir(dest)) == ["config.json", "model_manifest.json", "w-Q4_K_M.gguf"]
        # a corrupted payload is refused by its checksum and leaves nothing behind
        os.remove(os.path.join(dest, "w-Q4_K_M.gguf"))
        good = _Handler.repo["w-Q4_K_M.gguf"]
        listing = hub.list_files(R.ModelRef("acme", "web"))
        _Handler.repo["w-Q4_K_M.gguf"] = good[:-1] + b"\x00"
        f = [x for x in listing if x.name == "w-Q4_K_M.gguf"][0]
        with pytest.raises(R.RegistryError, match="sha256"):
            hub.fetch(R.ModelRef("acme", "web"), f, os.path.join(dest, "w-Q4_K_M.gguf"))
        assert not os.path.exists(os.path.join(dest, "w-Q4_K_M.gguf.part"))
        with pytest.raises(R.RegistryError, match="not found"):
            R.pull("acme/none", models, hub)
    finally:
        srv.shutdown()
        srv.server_close()


def test_unreachable_hub_is_a_registry_error(tmp_path):
    with pytest.raises(R.RegistryError):
        R.pull("a/b", str(tmp_path), R.Hub("http://127.0.0.1:9", timeout=2.0))


def test_registry_form_names_resolve_to_the_pulled_directory(tmp_path):
    from antfly_b200.formats.manifest import resolve_model_path

    (tmp_path / "acme" / "tiny").mkdir(parents=True)
    want = str(tmp_path / "acme" / "tiny")
    assert resolve_model_path("acme/tiny", str(tmp_path)) == want
    assert resolve_model_path("hf:acme/tiny:gguf:Q4_K_M", str(tmp_path)) == want
    assert resolve_model_path("acme/none:gguf", str(tmp_path)) is None
