"""Low-rank adapters in the PEFT layout merged at load time: the arithmetic, the key forms, adapter selection, and an
embedder served with an adapter equal to one whose weights were merged by hand."""
import json
import math
import os

import pytest
import torch

from antfly_b200.formats import lora as LORA
from antfly_b200.formats import safetensors_io as ST


def _adapter(sd, targets, r, seed, prefix="base_model.model.", named=False):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for mod in targets:
        o, i = sd[mod + ".weight"].shape
        tag = ".default" if named else ""
        out[f"{prefix}{mod}.lora_A{tag}.weight"] = torch.randn(r, i, generator=g) * 0.1
        out[f"{prefix}{mod}.lora_B{tag}.weight"] = torch.randn(o, r, generator=g) * 0.1
    return out


def test_merge_adds_scaled_low_rank_product():
    g = torch.Generator().manual_seed(0)
    sd = {"encoder.layer.0.attention.self.query.weight": torch.randn(8, 6, generator=g),
          "encoder.layer.0.attention.self.value.weight": torch.randn(8, 6, generator=g).to(torch.bfloat16),
          "pooler.dense.weight": torch.randn(6, 6, generator=g)}
    before = {k: v.clone() for k, v in sd.items()}
    mods = ["encoder.layer.0.attention.self.query", "encoder.layer.0.attention.self.value"]
    ad = _adapter(sd, mods, r=2, seed=1, named=True)
    merged = LORA.merge_lora(sd, ad, {"r": 2, "lora_alpha": 8})
    assert sorted(merged) == sorted(m + ".weight" for m in mods)
    for m in mods:
        a, b = ad[f"base_model.model.{m}.lora_A.default.weight"], ad[f"base_model.model.{m}.lora_B.default.weight"]
        want = before[m + ".weight"].float() + 4.0 * (b @ a)
        assert sd[m + ".weight"].dtype == before[m + ".weight"].dtype
        torch.testing.assert_close(sd[m + ".weight"].float(), want.to(before[m + ".weight"].dtype).float())
    assert torch.equal(sd["pooler.dense.weight"], before["pooler.dense.weight"])
    assert LORA.adapter_scale({"r": 16, "lora_alpha": 32}) == 2.0
    assert LORA.adapter_scale({"r": 16, "lora_alpha": 32, "use_rslora": True}) == 32 / math.sqrt(16)
    assert LORA.adapter_scale({"r": 4}) == 1.0
    with pytest.raises(ValueError):
        LORA.adapter_scale({"r": 0})


def test_prefixes_missing_targets_and_saved_modules():
    g = torch.Generator().manual_seed(0)
    sd = {"bert.encoder.layer.0.output.dense.weight": torch.randn(4, 8, generator=g),
          "classifier.weight": torch.zeros(2, 4), "classifier.bias": torch.zeros(2)}
    # the adapter was trained on the bare encoder: its names lack the checkpoint's "bert." prefix
    ad = {"base_model.model.encoder.layer.0.output.dense.lora_A.weight": torch.ones(1, 8),
          "base_model.model.encoder.layer.0.output.dense.lora_B.weight": torch.ones(4, 1),
          "base_model.model.classifier.modules_to_save.default.weight": torch.full((2, 4), 3.0),
          "base_model.model.classifier.modules_to_save.default.bias": torch.full((2,), 5.0)}
    w0 = sd["bert.encoder.layer.0.output.dense.weight"].clone()
    merged = LORA.merge_lora(sd, ad, {"r": 1, "lora_alpha": 2})
    torch.testing.assert_close(sd["bert.encoder.layer.0.output.dense.weight"], w0 + 2.0)
    assert float(sd["classifier.weight"][0, 0]) == 3.0 and float(sd["classifier.bias"][1]) == 5.0
    assert "classifier.weight" in merged
    with pytest.raises(KeyError):
        LORA.merge_lora(sd, {"base_model.model.nowhere.lora_A.weight": torch.ones(1, 8),
                             "base_model.model.nowhere.lora_B.weight": torch.ones(4, 1)}, {"r": 1})
    with pytest.raises(ValueError):
        LORA.merge_lora(sd, {"base_model.model.classifier.lora_A.weight": torch.ones(1, 4)}, {"r": 1})
    with pytest.raises(ValueError):                                  # factors of the wrong shape
        LORA.merge_lora(sd, {"base_model.model.classifier.lora_A.weight": torch.ones(1, 5),
                             "base_model.model.classifier.lora_B.weight": torch.ones(2, 1)}, {"r": 1})


def test_adapter_selection(tmp_path):
    d = tmp_path / "m"
    (d / "adapters" / "retrieval").mkdir(parents=True)
    (d / "adapters" / "clustering").mkdir()
    assert LORA.find_adapter(str(d)) is None
    for sub in ("retrieval", "clustering"):
        (d / "adapters" / sub / "adapter_config.json").write_text("{}")
        (d / "adapters" / sub / "adapter_model.safetensors").write_bytes(b"")
    assert LORA.find_adapter(str(d)).endswith("adapters/retrieval")
    assert LORA.find_adapter(str(d), "clustering").endswith("adapters/clustering")
    with pytest.raises(FileNotFoundError):
        LORA.find_adapter(str(d), "absent")
    (d / "adapter_config.json").write_text("{}")
    with pytest.raises(ValueError):                                  # half an adapter in the model directory
        LORA.find_adapter(str(d))
    (d / "adapter_model.safetensors").write_bytes(b"")
    assert LORA.find_adapter(str(d)) == str(d)


def test_embedder_served_with_an_adapter_equals_hand_merged_weights(tmp_path):
    from antfly_b200.api.model_manager import ModelManager
    from tests.test_api_cpu import _write_bert

    for name in ("plain", "adapted", "merged"):
        _write_bert(tmp_path / "embedders" / name, 0, [], 3)
    base = ST.load_file(str(tmp_path / "embedders" / "plain" / "model.safetensors"))
    mods = [k[:-7] for k in base if k.endswith(("query.weight", "value.weight", "intermediate.dense.weight"))]
    assert len(mods) == 3
    ad = _adapter(base, mods, r=4, seed=9)
    ad = {k: v * 3 for k, v in ad.items()}                          # large enough to move the embedding
    cfg = {"r": 4, "lora_alpha": 16, "target_modules": ["query", "value", "dense"], "peft_type": "LORA"}
    adir = tmp_path / "embedders" / "adapted" / "adapters" / "retrieval"
    adir.mkdir(parents=True)
    ST.save_file(ad, str(adir / "adapter_model.safetensors"))
    (adir / "adapter_config.json").write_text(json.dumps(cfg))
    hand = {k: v.clone() for k, v in base.items()}
    LORA.merge_lora(hand, ad, cfg)
    ST.save_file(hand, str(tmp_path / "embedders" / "merged" / "model.safetensors"))
    mm = ModelManager(models_dir=str(tmp_path), device="cpu")
    texts = ["low rank adapters", "merged at load time"]
    emb = {n: mm.get(n, "embedder").pipeline.embed(texts)[0] for n in ("plain", "adapted", "merged")}
    torch.testing.assert_close(emb["adapted"], emb["merged"])
    assert float((emb["adapted"] - emb["plain"]).abs().max()) > 1e-2
    info = mm.get("adapted", "embedder").info["adapter"]
    assert info == {"rank": 4, "scale": 4.0, "merged": 3, "name": "retrieval"}
    assert "adapter" not in mm.get("plain", "embedder").info
    # a named adapter that the model does not have is refused at load
    with pytest.raises(FileNotFoundError):
        ModelManager(models_dir=str(tmp_path), device="cpu", adapters={"adapted": "absent"}).get("adapted", "embedder")
