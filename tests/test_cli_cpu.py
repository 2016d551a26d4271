"""CLI smoke on the CPU path."""
import json

from antfly_b200.cli import main


def test_cli_embed_rerank_generate_list(capsys, tmp_path):
    assert main(["embed", "--model", "random:tiny", "--device", "cpu", "--text", "hello", "world", "--dimensions", "8"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert len(lines) == 2 and len(lines[0]["embedding"]) == 8
    assert main(["rerank", "--model", "random:tiny", "--device", "cpu", "--query", "q", "--doc", "a", "bb"]) == 0
    out = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert {o["index"] for o in out} == {0, 1} and out[0]["score"] >= out[1]["score"]
    assert main(["generate", "--model", "random:tiny", "--device", "cpu", "--kv-blocks", "64", "--prompt", "hi",
                 "--max-tokens", "4", "--print-timing", "--print-finish-reason", "--draft-layers", "1",
                 "--speculative-k", "2"]) == 0
    cap = capsys.readouterr()
    assert "generate_timing_ms:" in cap.err and "speculative: rounds=" in cap.err and "finish_reason:" in cap.err
    assert main(["list", "--models-dir", str(tmp_path)]) == 0
    assert "chunkers" in capsys.readouterr().out


def test_cli_export_gguf_roundtrip_and_task_commands(capsys, tmp_path):
    """safetensors -> GGUF (q8_0) -> loaded again by the GGUF reader with HF names; classify / recognize / rewrite /
    compare subcommands over model directories."""
    import torch

    from antfly_b200.formats import gguf as GG
    from antfly_b200.formats import safetensors_io as st
    from tests.test_api_cpu import _write_bert, _write_t5

    src = tmp_path / "generators" / "tiny-llama"
    src.mkdir(parents=True)
    H, F, V, L = 64, 128, 96, 2
    g = torch.Generator().manual_seed(0)
    sd = {"model.embed_tokens.weight": torch.randn(V, H, generator=g), "model.norm.weight": torch.ones(H),
          "lm_head.weight": torch.randn(V, H, generator=g)}
    for l in range(L):
        p = f"model.layers.{l}."
        for n, (o, i) in {"self_attn.q_proj": (H, H), "self_attn.k_proj": (32, H), "self_attn.v_proj": (32, H),
                          "self_attn.o_proj": (H, H), "mlp.gate_proj": (F, H), "mlp.up_proj": (F, H),
                          "mlp.down_proj": (H, F)}.items():
            sd[p + n + ".weight"] = torch.randn(o, i, generator=g) * 0.1
        sd[p + "input_layernorm.weight"] = torch.ones(H)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H)
    st.save_file(sd, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({
        "model_type": "llama", "hidden_size": H, "intermediate_size": F, "num_hidden_layers": L,
        "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": V, "rope_theta": 500000.0,
        "rms_norm_eps": 1e-5}))
    out = tmp_path / "tiny.gguf"
    assert main(["export", "--in", str(src), "--out", str(out), "--quant", "q8_0"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["tensor_types"] == {"8": 15, "1": 1, "0": 5}      # projections + lm_head q8_0, embedding f16, norms f32
    f = GG.GGUFFile(str(out))
    cfg = GG.llama_config_from_gguf(f.metadata)
    assert cfg["num_hidden_layers"] == L and cfg["num_key_value_heads"] == 2 and cfg["rope_theta"] == 500000.0
    assert cfg["vocab_size"] == V
    assert cfg["rope_half_split"] is False                       # llama files store Q / K rows with rotary pairs adjacent
    back = GG.to_hf_row_order({GG.hf_name(n): f.tensor(n) for n in f.tensors}, cfg)
    assert set(back) == set(sd)
    for n, t in sd.items():
        tol = 0.02 * float(t.abs().max()) if t.dim() == 2 else 0.0
        assert float((back[n] - t).abs().max()) <= tol + 1e-3, n

    # planning only, with filters: attention projections quantised, everything else left in f16
    plan = tmp_path / "plan.gguf"
    assert main(["export", "--in", str(src), "--out", str(plan), "--quant", "q5_1", "--dry-run", "--quantize-include",
                 "model.layers.", "--quantize-exclude", "model.layers.0.mlp.,model.layers.1.mlp."]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["dry_run"] and rep["bytes"] is None and not plan.exists()
    assert rep["tensor_types"] == {"7": 4 * L, "1": 3 * L + 2, "0": 5}
    _write_bert(tmp_path / "classifiers" / "clf", 3, ["negative", "neutral", "positive"], 2)
    _write_bert(tmp_path / "recognizers" / "ner", 3, ["O", "B-PER", "I-PER"], 1)
    _write_bert(tmp_path / "embedders" / "emb", 0, [], 3)
    _write_t5(tmp_path / "rewriters" / "t5")
    md = ["--models-dir", str(tmp_path), "--device", "cpu"]
    assert main(["classify", *md, "--model", "clf", "--text", "good", "bad", "--top-k", "2"]) == 0
    rows = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert len(rows) == 2 and len(rows[0]["labels"]) == 2 and rows[0]["labels"][0]["score"] >= rows[0]["labels"][1]["score"]
    assert main(["recognize", *md, "--model", "ner", "--text", "alice went home"]) == 0
    assert "entities" in json.loads(capsys.readouterr().out)
    assert main(["rewrite", *md, "--model", "t5", "--text", "paraphrase: hi", "--max-tokens", "5",
                 "--print-timing"]) == 0
    cap = capsys.readouterr()
    assert json.loads(cap.out)["tokens"] <= 5 and "generate_timing_ms:" in cap.err
    assert main(["compare", "--models-dir", str(tmp_path), "--model", "emb", "--text", "a b c", "hello",
                 "--device-a", "cpu", "--device-b", "cpu"]) == 0
    assert json.loads(capsys.readouterr().out)["min_cosine"] > 0.9999


def test_compile_artifact_is_loaded_instead_of_repacking(capsys, tmp_path):
    """compile-artifact writes the packed layout; the model built from it is bit-identical to the one packed from
    the checkpoint, and the model manager prefers it."""
    import torch

    from antfly_b200.api.model_manager import COMPILED_ARTIFACT, ModelManager
    from antfly_b200.formats import safetensors_io as st
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from tests.test_parallel_cpu import _forward_logits, _hf_llama_state

    cfg = LlamaConfig.tiny(num_hidden_layers=2)
    src = tmp_path / "generators" / "tiny"
    src.mkdir(parents=True)
    st.save_file(_hf_llama_state(cfg), str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({
        "model_type": "llama", "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
        "num_hidden_layers": 2, "num_attention_heads": cfg.num_attention_heads,
        "num_key_value_heads": cfg.num_key_value_heads, "vocab_size": cfg.vocab_size, "rope_theta": cfg.rope_theta,
        "rms_norm_eps": cfg.rms_norm_eps, "head_dim": cfg.head_dim, "tie_word_embeddings": False}))
    assert main(["compile-artifact", "--in", str(src)]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["out"].endswith(COMPILED_ARTIFACT) and rep["bytes"] > 0
    a = LlamaModel.from_artifact(rep["out"], device="cpu")
    b = LlamaModel.from_state_dict(LlamaConfig.from_hf(json.loads((src / "config.json").read_text())),
                                   st.load_model_dir(str(src)), device="cpu")
    assert set(a.w) == set(b.w)
    for k in a.w:
        if hasattr(a.w[k], "q"):
            assert torch.equal(a.w[k].q.view(torch.uint8), b.w[k].q.view(torch.uint8))
            assert torch.equal(a.w[k].scales, b.w[k].scales) and a.w[k].interleaved_swiglu == b.w[k].interleaved_swiglu
        else:
            assert torch.equal(a.w[k], b.w[k])
    assert torch.equal(_forward_logits(a, a.cfg), _forward_logits(b, b.cfg))
    lm = ModelManager(models_dir=str(tmp_path), device="cpu", kv_blocks=32).get("tiny", "generator")
    assert lm.info["weights"] == "compiled"
    with __import__("pytest").raises(ValueError):
        LlamaModel.from_artifact(str(src / "model.safetensors"), device="cpu")
    # run-artifact: the same tokens as the served model, straight from the artifact file
    from antfly_b200.runtime.sampling_params import SamplingParams

    capsys.readouterr()
    assert main(["run-artifact", "--artifact", rep["out"], "--device", "cpu", "--kv-blocks", "32", "--prompt", "hi",
                 "--max-tokens", "5", "--raw-prompt", "--print-timing"]) == 0
    cap = capsys.readouterr()
    want = lm.pipeline.generate("hi", SamplingParams(max_tokens=5), raw_prompt=True).text
    assert cap.out.rstrip("\n") == want and "generate_timing_ms:" in cap.err


def test_cli_extract_answers_a_schema_in_process(capsys, tmp_path):
    from tests.test_api_cpu import _write_bert

    _write_bert(tmp_path / "recognizers" / "tiny-ner", 5, ["O", "B-PER", "I-PER", "B-LOC", "I-LOC"], 1)
    assert main(["extract", "--models-dir", str(tmp_path), "--device", "cpu", "--model", "tiny-ner", "--text",
                 "alice met bob in paris", "--entities", "PER", "LOC", "--compact"]) == 0
    body = json.loads(capsys.readouterr().out)
    assert body["object"] == "extraction" and body["data"][0]["id"] == "0"
    assert all(e["label"] in ("PER", "LOC") for e in body["data"][0]["entities"])
    assert main(["extract", "--models-dir", str(tmp_path), "--device", "cpu", "--model", "nope", "--text", "x",
                 "--entities", "PER", "--compact"]) == 2
    capsys.readouterr()


def test_cli_bench_forwards_to_the_bench_script(capfd):
    assert main(["bench", "--impl", "reference", "--workload", "cpu"]) == 0
    line = [l for l in capfd.readouterr().out.splitlines() if l.startswith("{")][-1]
    assert json.loads(line)["impl"] == "reference" and "unavailable" in json.loads(line)


def test_cli_dequant_and_cuda_info(capsys, tmp_path):
    import numpy as np
    import torch

    raw = bytearray()
    for b in range(3):
        raw += np.float16(0.5 * (b + 1)).tobytes() + bytes((np.arange(32, dtype=np.int8) - 16 + b).view(np.uint8))
    (tmp_path / "in.bin").write_bytes(bytes(raw))
    assert main(["dequant", "q8_0", "--input", str(tmp_path / "in.bin"), "--output", str(tmp_path / "out.bin")]) == 0
    out = np.frombuffer((tmp_path / "out.bin").read_bytes(), dtype="<f4")
    want = np.concatenate([0.5 * (b + 1) * (np.arange(32) - 16 + b) for b in range(3)]).astype(np.float32)
    assert np.array_equal(out, want)
    assert main(["dequant", "8", "--input", str(tmp_path / "in.bin"), "--output", str(tmp_path / "o2.bin")]) == 0
    assert (tmp_path / "o2.bin").read_bytes() == (tmp_path / "out.bin").read_bytes()
    (tmp_path / "bad.bin").write_bytes(b"123")
    assert main(["dequant", "q8_0", "--input", str(tmp_path / "bad.bin")]) == 2
    assert main(["dequant", "no_such_format", "--input", str(tmp_path / "in.bin")]) == 2
    capsys.readouterr()
    rc = main(["cuda-info"])
    text = capsys.readouterr().out
    if torch.cuda.is_available():
        assert rc == 0 and "device_name:" in text and "compute_capability: sm_" in text
    else:
        assert rc == 1 and text.startswith("cuda: unavailable")


def test_cli_pull_from_a_mirror_directory(capsys, tmp_path):
    import os

    repo = tmp_path / "mirror" / "acme" / "enc"
    repo.mkdir(parents=True)
    (repo / "config.json").write_text(json.dumps({"architectures": ["BertModel"], "model_type": "bert"}))
    (repo / "model.safetensors").write_bytes(b"\0" * 16)
    (repo / "model.onnx").write_bytes(b"\0" * 16)
    models = tmp_path / "models"
    assert main(["pull", "hf:acme/enc", "--hub", str(tmp_path / "mirror"), "--models-dir", str(models)]) == 0
    cap = capsys.readouterr()
    dest = cap.out.strip().splitlines()[-1]
    assert dest.endswith("acme/enc") and "model.safetensors" in cap.err
    assert sorted(os.listdir(dest)) == ["config.json", "model.safetensors", "model_manifest.json"]
    assert json.load(open(os.path.join(dest, "model_manifest.json")))["tasks"] == ["embed"]
    assert main(["pull", "acme/gone", "--hub", str(tmp_path / "mirror"), "--models-dir", str(models)]) == 1
    assert "pull failed" in capsys.readouterr().err
