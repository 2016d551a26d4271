"""Configuration file / environment / flag precedence, Go-style durations, and the model manager's unloading rules
(keep-alive idleness, maximum loaded models, advisory memory budget, eager pinning)."""
import json

import pytest
import torch

from antfly_b200.api.model_manager import ModelManager
from antfly_b200.config import Config, load_config, parse_duration
from antfly_b200.formats import safetensors_io as st
from antfly_b200.models.bert import BertConfig, BertModel


def test_durations():
    assert parse_duration("5m") == 300 and parse_duration("1h30m") == 5400 and parse_duration("250ms") == 0.25
    assert parse_duration("0") == 0 and parse_duration(0) == 0 and parse_duration("30s") == 30
    assert parse_duration("1.5h") == 5400 and parse_duration("45") == 45
    for bad in ("5 minutes", "m5", "5x", "1h,30m"):
        with pytest.raises(ValueError):
            parse_duration(bad)


def test_defaults_match_the_documented_schema():
    c = Config()
    assert c.keep_alive == "5m" and c.keep_alive_s == 300 and c.max_loaded_models == 0 and c.pool_size == 1
    assert c.max_concurrent_requests == 0 and c.max_queue_size == 0 and c.request_timeout_s == 0
    assert c.max_memory_mb == 0 and c.preload == [] and c.strategy("any") == "lazy"
    assert c.host_port == ("localhost", 8080)


def test_file_env_and_override_precedence(tmp_path):
    p = tmp_path / "inference.yaml"
    p.write_text("api_url: http://0.0.0.0:9090\nmodels_dir: /models\nkeep_alive: 10m\nmax_loaded_models: 3\n"
                 "preload: [BAAI/bge-small-en-v1.5]\nmodel_strategies: {big: eager}\nlog: {level: debug, style: json}\n"
                 "backend_priority: [onnx, 'native:cpu']\n")
    c = load_config(str(p), env={})
    assert c.host_port == ("0.0.0.0", 9090) and c.models_dir == "/models" and c.keep_alive_s == 600
    assert c.max_loaded_models == 3 and c.preload == ["BAAI/bge-small-en-v1.5"] and c.strategy("big") == "eager"
    assert c.strategy("other") == "lazy" and c.log.level == "debug" and c.log.style == "json"
    assert c.device() == "cpu"                        # onnx is not a backend of this build; native:cpu is
    c = load_config(str(p), env={"ANTFLY_INFERENCE_KEEP_ALIVE": "0", "TERMITE_MAX_LOADED_MODELS": "7",
                                 "ANTFLY_INFERENCE_PRELOAD": "a, b"})
    assert c.keep_alive_s == 0 and c.strategy("other") == "eager" and c.max_loaded_models == 7
    assert c.preload == ["a", "b"]
    c = load_config(str(p), env={"TERMITE_MAX_LOADED_MODELS": "7"}, max_loaded_models=2)
    assert c.max_loaded_models == 2
    j = tmp_path / "c.json"
    j.write_text(json.dumps({"api_url": "http://[::1]:7000", "request_timeout": "30s"}))
    c = load_config(str(j), env={})
    assert c.host_port == ("::1", 7000) and c.request_timeout_s == 30
    assert load_config(None, env={}).to_dict()["keep_alive"] == "5m"


def test_bad_configuration_is_rejected(tmp_path):
    p = tmp_path / "bad.yaml"
    p.write_text("api_url: http://localhost:1\nno_such_key: 1\n")
    with pytest.raises(ValueError, match="unknown configuration key"):
        load_config(str(p), env={})
    for kw in ({"keep_alive": "soon"}, {"pool_size": 0}, {"max_queue_size": -1}, {"content_security": {"download_timeout_seconds": 0}},
               {"model_strategies": {"m": "sometimes"}}):
        with pytest.raises(ValueError):
            load_config(None, env={}, **kw)


def _model_dirs(root, names):
    for i, n in enumerate(names):
        d = root / "embedders" / n
        d.mkdir(parents=True)
        cfg = BertConfig(hidden_size=64, num_hidden_layers=1, num_attention_heads=4, intermediate_size=128,
                         vocab_size=300)
        st.save_file(BertModel.random_init(cfg, device="cpu", seed=i).state_dict_hf(), str(d / "model.safetensors"))
        (d / "config.json").write_text(json.dumps({"model_type": "bert", "hidden_size": 64, "num_hidden_layers": 1,
                                                   "num_attention_heads": 4, "intermediate_size": 128,
                                                   "vocab_size": 300, "max_position_embeddings": 512}))


def test_keep_alive_limits_and_pinning(tmp_path):
    _model_dirs(tmp_path, ["a", "b", "c"])
    now = [1000.0]
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu", max_loaded_models=0, keep_alive_s=300,
                       strategies={"c": "eager"}, clock=lambda: now[0])
    la = mgr.get("a", "embedder")
    assert la.bytes > 0 and not la.pinned
    mgr.get("c", "embedder")
    now[0] += 200
    mgr.get("b", "embedder")
    assert mgr.loaded_count() == 3
    now[0] += 150                                     # a idle 350 s, b 150 s, c pinned
    assert mgr.evict_idle() == 1 and mgr.loaded_count() == 2
    assert mgr.get("a", "embedder") is not la         # reloaded on demand
    now[0] += 1000
    mgr.get("b", "embedder")                          # access evicts idle a, keeps pinned c and refreshes b
    assert {k.split(":")[1] for k in mgr._models} == {"b", "c"} and mgr.evictions == 2

    lim = ModelManager(models_dir=str(tmp_path), device="cpu", max_loaded_models=2)
    for n in "abc":
        lim.get(n, "embedder")
    assert [k.split(":")[1] for k in lim._models] == ["b", "c"]          # least recently used went first
    lim.get("b", "embedder"); lim.get("a", "embedder")
    assert [k.split(":")[1] for k in lim._models] == ["b", "a"]

    one = ModelManager(models_dir=str(tmp_path), device="cpu", max_loaded_models=0)
    size_mb = one.get("a", "embedder").bytes / (1 << 20)
    mem = ModelManager(models_dir=str(tmp_path), device="cpu", max_loaded_models=0,
                       max_memory_mb=max(1, int(size_mb * 2.5)))
    if size_mb * 3 > max(1, int(size_mb * 2.5)):      # three models exceed the budget, two fit
        for n in "abc":
            mem.get(n, "embedder")
        assert mem.loaded_count() == 2 and "embedder:a" not in mem._models
    assert one.unload("a", "embedder") and not one.unload("a", "embedder")


def test_structured_logging_text_and_json():
    import io
    import logging

    from antfly_b200.utils import logs

    buf = io.StringIO()
    lg = logs.setup("debug", "json", buf)
    logs.event(logs.get("server"), logging.INFO, "request", endpoint="embed", units=3, duration_ms=1.5)
    rec = json.loads(buf.getvalue().strip())
    assert rec["msg"] == "request" and rec["endpoint"] == "embed" and rec["units"] == 3 and rec["level"] == "info"
    assert rec["logger"] == "antfly_b200.server" and rec["ts"].endswith("Z")
    buf = io.StringIO()
    logs.setup("warning", "text", buf)
    logs.event(logs.get("x"), logging.INFO, "hidden")
    logs.event(logs.get("x"), logging.WARNING, "queue full", endpoint="generate", note="retry later")
    line = buf.getvalue().strip()
    assert "hidden" not in line and "warn" in line and "queue full endpoint=generate" in line
    assert 'note="retry later"' in line and len(lg.handlers) == 1
    logs.setup("info", "text", io.StringIO())
