"""Fine-tuning: networks against transformers, adapters, NF4, losses, packing, the training loop (resume, gradient
accumulation, data parallel on gloo ranks) and the recipe runner end to end on tiny checkpoints."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

from antfly_b200.finetune import data as D
from antfly_b200.finetune import lora as L
from antfly_b200.finetune import losses as LS
from antfly_b200.finetune import recipes as R
from antfly_b200.finetune.nets import DecoderNet
from antfly_b200.finetune.trainer import TrainConfig, Trainer, adapters_disabled, lr_at
from antfly_b200.formats import safetensors_io as ST
from antfly_b200.models.llama import LlamaConfig

transformers = pytest.importorskip("transformers")


def _tiny_llama(path, seed=0, vocab=300, tie=False):
    torch.manual_seed(seed)
    cfg = transformers.LlamaConfig(vocab_size=vocab, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                   tie_word_embeddings=tie)
    hf = transformers.LlamaForCausalLM(cfg).eval().float()
    with torch.no_grad():        # a trained model's output matrix is far from the 0.02 initialisation: with it frozen
        hf.lm_head.weight.mul_(10.0)   # at that scale no hidden state could raise a token's probability above ~1 %
    os.makedirs(path, exist_ok=True)
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    if tie:
        sd.pop("lm_head.weight", None)
    ST.save_file(sd, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    return cfg, hf


def _jsonl(path, rows):
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    return str(path)


def test_nf4_round_trip_and_lora_linear_starts_at_the_base():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(48, 80, generator=g) * 0.05
    codes, absmax = L.nf4_quantize(w)
    assert codes.numel() == 48 * 80 // 2 and absmax.numel() == 48 * 80 // 64
    back = L.nf4_dequantize(codes, absmax, w.shape)
    err = (back - w).abs()
    assert float(err.max()) <= float(absmax.max()) * 0.16 and float(err.mean()) < 0.1 * float(w.abs().mean()) * 1.5
    assert torch.equal(L.nf4_dequantize(*L.nf4_quantize(back), w.shape), back)          # codes are a fixed point
    x = torch.randn(5, 80, generator=g)
    lin = L.LoraLinear(w, torch.zeros(48), rank=4, alpha=8, generator=g)
    torch.testing.assert_close(lin(x), x @ w.t())
    with torch.no_grad():
        lin.lora_B.normal_(0, 0.1, generator=g)
    want = x @ w.t() + 2.0 * (x @ lin.lora_A.t()) @ lin.lora_B.t()
    torch.testing.assert_close(lin(x), want)
    q = L.LoraLinear(w, None, rank=4, alpha=8, nf4=True, generator=g)
    torch.testing.assert_close(q(x), x @ back.t())
    with pytest.raises(ValueError):
        L.target_names("moe-experts", None)
    with pytest.raises(ValueError):
        L.target_names("everything", None)


def test_chunked_cross_entropy_equals_the_plain_one_and_packing_equals_separate_rows(tmp_path):
    cfg_hf, hf = _tiny_llama(str(tmp_path / "m"))
    net = DecoderNet(LlamaConfig.from_hf(cfg_hf.to_dict()), hf.state_dict())
    g = torch.Generator().manual_seed(1)
    a, b = torch.randint(3, 300, (9,), generator=g).tolist(), torch.randint(3, 300, (6,), generator=g).tolist()
    ex = [D.TokenExample(a, [0] * 3 + [1] * 6), D.TokenExample(b, [0] * 2 + [1] * 4)]
    rows = D.pack_examples(ex, 16, pad_id=0)
    assert len(rows) == 1 and rows[0]["doc_ids"] == [0] * 9 + [1] * 6 + [2] and rows[0]["examples"] == [0, 1]
    ids = torch.tensor([rows[0]["ids"]])
    lm = torch.tensor([rows[0]["loss_mask"]]).bool()
    doc = torch.tensor([rows[0]["doc_ids"]])
    packed, n = LS.causal_lm_loss(net, net(ids, doc_ids=doc), ids, lm, doc, chunk=4)
    assert n == 6 + 4
    tot = 0.0
    for e in ex:
        i = torch.tensor([e.ids])
        logits = hf(i).logits[0, :-1]
        lp = torch.log_softmax(logits, -1).gather(-1, i[0, 1:, None])[:, 0]
        tot += float(-(lp * torch.tensor(e.loss_mask[1:])).sum())
    assert abs(float(packed) - tot / 10) < 1e-4
    # gradients flow through the chunked (recomputed) projection
    L.inject(net, rank=2, alpha=4)
    with torch.no_grad():
        for m in net.modules():
            if isinstance(m, L.LoraLinear):
                m.lora_B.normal_(0, 0.02, generator=g)
    loss, _ = LS.causal_lm_loss(net, net(ids, doc_ids=doc), ids, lm, doc, chunk=4)
    loss.backward()
    grads = [p.grad for n_, p in net.named_parameters() if p.requires_grad]
    assert all(g_ is not None and torch.isfinite(g_).all() for g_ in grads) and any(float(g_.abs().sum()) > 0 for g_ in grads)
    with pytest.raises(ValueError):
        D.pack_examples([D.TokenExample(list(range(20)), [1] * 20)], 16)


def test_preference_and_group_losses():
    pc, pr = torch.tensor([-1.0, -3.0]), torch.tensor([-2.0, -2.5])
    rc, rr = torch.tensor([-1.2, -2.8]), torch.tensor([-1.8, -2.6])
    loss, m = LS.dpo_loss(pc, pr, rc, rr, beta=0.5)
    margin = torch.tensor([(-1 + 2) - (-1.2 + 1.8), (-3 + 2.5) - (-2.8 + 2.6)])
    assert abs(float(loss) - float(-torch.nn.functional.logsigmoid(0.5 * margin).mean())) < 1e-6
    assert m["accuracy"] == 0.5
    adv = LS.grpo_advantages(torch.tensor([1.0, 0.0, 0.0, 1.0, 1.0, 1.0]), 3)
    assert abs(float(adv[:3].sum())) < 1e-5 and float(adv[0]) > 0 > float(adv[1]) and float(adv[3:].abs().max()) < 1e-3
    new = torch.tensor([[-0.35, -0.65]], requires_grad=True)
    old, ref = torch.tensor([[-0.4, -0.6]]), torch.tensor([[-0.5, -0.7]])
    loss, m = LS.grpo_loss(new, old, ref, torch.tensor([1.0]), torch.ones(1, 2).bool(), 0.2, 0.04)
    ratio = torch.exp(new.detach() - old)
    d = ref - new.detach()
    want = -(torch.minimum(ratio, ratio.clamp(0.8, 1.2)) - 0.04 * (torch.exp(d) - d - 1)).mean()
    assert abs(float(loss) - float(want)) < 1e-6 and m["kl"] > 0 and m["clip_fraction"] == 0.0
    q = torch.nn.functional.normalize(torch.eye(3) + 0.01, dim=-1)
    loss, m = LS.info_nce(q, q.clone(), temperature=0.05)
    assert m["accuracy"] == 1.0 and float(loss) < 1e-3
    s, y, grp = torch.tensor([2.0, -1.0, 0.5, 0.2]), torch.tensor([1.0, 0.0, 0.0, 1.0]), torch.tensor([0, 0, 1, 1])
    pw = LS.reranker_loss(s, y, grp, "pairwise")
    want = -(torch.nn.functional.logsigmoid(torch.tensor(3.0)) + torch.nn.functional.logsigmoid(torch.tensor(-0.3))) / 2
    assert abs(float(pw) - float(want)) < 1e-6
    assert R.reward(" Yes ", "yes", "exact-match-ci") == 1.0 and R.reward("Yes", "yes", "exact-match") == 0.0
    assert R.reward("yes, sure", "yes", "prefix-match") == 1.0


def test_schedule_and_recipe_validation(tmp_path):
    cfg = TrainConfig(learning_rate=1.0, warmup_ratio=0.1, schedule="cosine")
    assert lr_at(0, 100, cfg) == 0.1 and lr_at(9, 100, cfg) == 1.0 and abs(lr_at(55, 100, cfg) - 0.5) < 1e-6
    assert lr_at(99, 100, TrainConfig(learning_rate=1.0, warmup_ratio=0.0, schedule="linear")) == pytest.approx(0.01)
    base = {"recipe": "lora-sft", "model": {"path": str(tmp_path / "m")}, "dataset": {"path": "x.jsonl"}}
    r = R.normalize(base)
    assert r["adapter"]["rank"] == 16 and r["adapter"]["alpha"] == 32 and r["dataset"]["max_seq_len"] == 512
    assert R.normalize({**base, "recipe": "grpo"})["adapter"]["rank"] == 8
    assert [s["name"] for s in R.plan({**base, "dataset": {"path": "x", "eval_path": "y"},
                                       "artifacts": {"materialized_dir": "z"}})] == ["prepare", "train", "eval", "materialize"]
    for bad in ({**base, "recipe": "rlhf"}, {**base, "model": {}}, {**base, "dataset": {}},
                {**base, "adapter": {"scaling": "dora"}}, {**base, "adapter": {"target_preset": "moe-experts"}},
                {**base, "recipe": "grpo", "grpo": {"reward_mode": "bleu"}}):
        with pytest.raises(ValueError):
            R.normalize(bad)


def _sft_recipe(tmp_path, name="lora-sft", **over):
    rows = [{"prompt": "ab", "completion": "xyz"}, {"prompt": "cd", "completion": "uvw"},
            {"messages": [{"role": "user", "content": "ef"}, {"role": "assistant", "content": "rst"}]},
            {"text": "plain text row"}] * 2
    rec = {"recipe": name, "model": {"path": str(tmp_path / "m")},
           "dataset": {"path": _jsonl(tmp_path / "train.jsonl", rows), "eval_path": _jsonl(tmp_path / "eval.jsonl", rows[:3]),
                       "max_seq_len": 96},
           "adapter": {"rank": 4, "alpha": 8},
           "optimizer": {"learning_rate": 1e-2, "epochs": 20, "batch_size": 1, "gradient_accumulation_steps": 2,
                         "warmup_ratio": 0.0, "schedule": "constant"},
           "artifacts": {"root": str(tmp_path / "run"), "materialized_dir": str(tmp_path / "merged")}}
    for k, v in over.items():
        rec[k] = {**rec.get(k, {}), **v} if isinstance(v, dict) else v
    return rec


@pytest.mark.parametrize("name", ["lora-sft", "qlora-sft", "sft"])
def test_sft_recipes_learn_write_artifacts_and_serve(tmp_path, name):
    _tiny_llama(str(tmp_path / "m"))
    seen = []
    over = {"optimizer": {"learning_rate": 2e-3}} if name == "sft" else {}
    rep = R.run_recipe(_sft_recipe(tmp_path, name, **over), log=seen.append)
    assert rep["status"] == "succeeded" and rep["train"]["final_loss"] < 0.6 * rep["train"]["first_loss"]
    assert rep["packing"]["rows"] < rep["packing"]["examples"] and len(seen) == rep["train"]["optimizer_steps"]
    assert rep["eval"]["loss"] < rep["train"]["first_loss"]
    root = tmp_path / "run"
    man = json.load(open(root / "recipe_run_manifest.json"))
    assert man["schema"] == R.SCHEMA and man["status"] == "succeeded"
    assert [s["status"] for s in man["steps"]] == ["succeeded"] * 4
    assert os.path.exists(root / "training_config.json") and os.path.exists(root / "training_report.json")
    out = root / "adapter-trained"
    if name == "sft":
        assert os.path.exists(out / "model.safetensors") and rep["train"]["adapted_modules"] == 0
    else:
        cfg = json.load(open(out / "adapter_config.json"))
        assert cfg["r"] == 4 and cfg["lora_alpha"] == 8 and "q_proj" in cfg["target_modules"] and rep["train"]["adapted_modules"] == 14
        assert rep["train"]["trainable_parameters"] < 30000
    if name == "lora-sft":
        # the adapter dropped into the model directory is merged at load; the served model equals the materialised one
        from antfly_b200.api.model_manager import ModelManager
        from antfly_b200.runtime.sampling_params import SamplingParams

        gen = tmp_path / "generators"
        os.makedirs(gen / "adapted")
        for n in os.listdir(tmp_path / "m"):
            os.link(tmp_path / "m" / n, gen / "adapted" / n)
        for n in os.listdir(out):
            os.link(out / n, gen / "adapted" / n)
        os.rename(tmp_path / "merged", gen / "merged")
        mm = ModelManager(models_dir=str(tmp_path), device="cpu")
        sp = SamplingParams(max_tokens=4, ignore_eos=True)
        a = mm.get("adapted", "generator")
        assert a.info["adapter"]["rank"] == 4 and a.info["adapter"]["merged"] == 14
        ta = a.pipeline.generate("ab", sp).token_ids
        tb = mm.get("merged", "generator").pipeline.generate("ab", sp).token_ids
        assert ta == tb
        assert a.tokenizer.decode(ta).startswith("xyz")                 # and it has learned the training pair


def test_resume_reproduces_an_uninterrupted_run(tmp_path):
    _tiny_llama(str(tmp_path / "m"))
    over = {"optimizer": {"epochs": 2, "gradient_accumulation_steps": 1, "checkpoint_every": 3}}
    full = R.run_recipe(_sft_recipe(tmp_path, **over, artifacts={"root": str(tmp_path / "full")}))
    a = ST.load_file(str(tmp_path / "full" / "adapter-trained" / "adapter_model.safetensors"))
    ck = tmp_path / "full" / "checkpoints" / "checkpoint-3"
    assert os.path.exists(ck / "optimizer.safetensors") and json.load(open(ck / "trainer_state.json"))["adam_step"] == 3
    again = R.run_recipe(_sft_recipe(tmp_path, **over, artifacts={"root": str(tmp_path / "again")}), resume_from=str(ck))
    b = ST.load_file(str(tmp_path / "again" / "adapter-trained" / "adapter_model.safetensors"))
    assert again["train"]["optimizer_steps"] == full["train"]["optimizer_steps"]
    for k in a:
        torch.testing.assert_close(a[k], b[k], atol=1e-6, rtol=1e-5)


def test_dpo_and_grpo_recipes(tmp_path):
    _tiny_llama(str(tmp_path / "m"))
    pref = [{"prompt": "pick", "chosen": "good", "rejected": "bad"}, {"prompt": "choose", "chosen": "yes", "rejected": "no"}] * 2
    rec = {"recipe": "dpo", "model": {"path": str(tmp_path / "m")},
           "dataset": {"path": _jsonl(tmp_path / "p.jsonl", pref), "eval_path": _jsonl(tmp_path / "pe.jsonl", pref[:2]),
                       "max_seq_len": 64, "format": "rendered-text-preference"},
           "adapter": {"rank": 4, "alpha": 8}, "preference": {"beta": 0.5},
           "optimizer": {"learning_rate": 5e-3, "epochs": 6, "batch_size": 2, "warmup_ratio": 0.0},
           "artifacts": {"root": str(tmp_path / "dpo")}}
    rep = R.run_recipe(rec)
    assert rep["train"]["final_loss"] < rep["train"]["first_loss"] and rep["eval"]["accuracy"] == 1.0
    assert rep["eval"]["reward_margin"] > 0
    # GRPO: reward for answering "a" (token sampled among a 300-entry vocabulary; a short roll-out makes hits likely
    # enough for the group statistics to carry signal once in a while; the run must be finite and well-formed)
    rows = [{"prompt": "say a", "target": "a"}] * 4
    rec = {"recipe": "grpo", "model": {"path": str(tmp_path / "m")},
           "dataset": {"path": _jsonl(tmp_path / "g.jsonl", rows), "eval_path": _jsonl(tmp_path / "ge.jsonl", rows[:1]),
                       "max_seq_len": 32, "format": "rendered-text-grpo"},
           "grpo": {"group_size": 4, "max_completion_tokens": 2, "reward_mode": "prefix-match"},
           "optimizer": {"learning_rate": 1e-3, "epochs": 1, "batch_size": 2},
           "artifacts": {"root": str(tmp_path / "grpo")}}
    seen = []
    rep = R.run_recipe(rec, log=seen.append)
    assert rep["status"] == "succeeded" and rep["train"]["optimizer_steps"] == 2
    assert all(math.isfinite(s["loss"]) and "reward" in s and "kl" in s for s in seen)
    assert 0.0 <= rep["eval"]["greedy_reward"] <= 1.0
    assert json.load(open(tmp_path / "grpo" / "adapter-trained" / "adapter_config.json"))["r"] == 8


def test_reranker_and_embedder_recipes(tmp_path):
    from tests.test_api_cpu import _write_bert

    _write_bert(tmp_path / "rr", 1, ["relevant"], 2)
    pairs = [{"query": "red fruit", "document": "apple apple", "label": 1}, {"query": "red fruit", "document": "engine oil", "label": 0},
             {"query": "car part", "document": "engine oil", "label": 1}, {"query": "car part", "document": "apple apple", "label": 0}]
    for mode in ("bce", "pairwise"):
        rec = {"recipe": "reranker", "model": {"path": str(tmp_path / "rr")},
               "dataset": {"path": _jsonl(tmp_path / "rr.jsonl", pairs), "eval_path": _jsonl(tmp_path / "rre.jsonl", pairs),
                           "max_seq_len": 32},
               "adapter": {"rank": 4, "alpha": 8},
               "optimizer": {"learning_rate": 1e-2, "epochs": 10, "batch_size": 4, "warmup_ratio": 0.0, "reranker_loss": mode},
               "artifacts": {"root": str(tmp_path / ("rr-" + mode))}}
        rep = R.run_recipe(rec)
        assert rep["train"]["final_loss"] < rep["train"]["first_loss"], mode
    _write_bert(tmp_path / "emb", 0, [], 4)
    triples = [{"query": "red fruit", "positive": "apple apple", "negatives": ["engine oil"]},
               {"query": "car part", "positive": "engine oil", "negatives": ["apple apple"]},
               {"query": "blue sky", "positive": "clouds above", "negatives": ["deep sea"]}]
    rec = {"recipe": "embedder", "model": {"path": str(tmp_path / "emb")},
           "dataset": {"path": _jsonl(tmp_path / "e.jsonl", triples), "eval_path": _jsonl(tmp_path / "ee.jsonl", triples),
                       "max_seq_len": 32},
           "adapter": {"rank": 4, "alpha": 8, "target_preset": "attention-only"},
           "optimizer": {"learning_rate": 2e-2, "epochs": 40, "batch_size": 3, "warmup_ratio": 0.0, "temperature": 0.1,
                         "mrl_dims": [64, 16], "xbm_capacity": 6, "xbm_warmup_steps": 25},
           "artifacts": {"root": str(tmp_path / "emb-run")}}
    rep = R.run_recipe(rec)
    # (the training loss is not comparable across the run: the memory adds candidates once it is switched on)
    assert rep["eval"]["loss"] < 0.6 * rep["train"]["first_loss"] and rep["eval"]["accuracy"] >= 0.66
    cfg = json.load(open(tmp_path / "emb-run" / "adapter-trained" / "adapter_config.json"))
    assert cfg["target_modules"] == ["dense", "key", "query", "value"]
    # a failing run leaves a failed manifest behind
    bad = dict(rec, model={"path": str(tmp_path / "nowhere")}, artifacts={"root": str(tmp_path / "bad")})
    with pytest.raises(Exception):
        R.run_recipe(bad)
    assert json.load(open(tmp_path / "bad" / "recipe_run_manifest.json"))["status"] == "failed"


def test_cli_plan_and_two_rank_data_parallel_equals_one_rank_with_the_global_batch(tmp_path, capsys):
    from antfly_b200.cli import main

    _tiny_llama(str(tmp_path / "m"))
    rows = [{"text": "%s%s%s%s %s" % (a, a, b, b, c)} for a in "abcd" for b in "xy" for c in "pq"]      # equal lengths
    def rec(root, batch):
        return {"recipe": "lora-sft", "model": {"path": str(tmp_path / "m")},
                "dataset": {"path": _jsonl(tmp_path / "t.jsonl", rows), "max_seq_len": 32, "packing": False},
                "adapter": {"rank": 2, "alpha": 4, "target_preset": "attention-only"},
                "optimizer": {"learning_rate": 5e-3, "epochs": 1, "batch_size": batch, "warmup_ratio": 0.0,
                              "schedule": "constant"},
                "artifacts": {"root": str(tmp_path / root)}}
    for name, batch in (("one", 2), ("two", 1)):
        with open(tmp_path / f"{name}.json", "w") as f:
            json.dump(rec(name, batch), f)
    assert main(["finetune", "plan", str(tmp_path / "one.json")]) == 0
    assert [s["name"] for s in json.loads(capsys.readouterr().out)["steps"]] == ["prepare", "train"]
    assert main(["finetune", "run", str(tmp_path / "one.json"), "--dry-run"]) == 0
    capsys.readouterr()
    assert main(["finetune", "run", str(tmp_path / "one.json")]) == 0
    one = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert one["status"] == "succeeded" and one["train"]["optimizer_steps"] == 8
    env = dict(os.environ, PYTHONPATH=os.getcwd())
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29631", "-m", "antfly_b200.cli", "finetune",
                          "run", str(tmp_path / "two.json")], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    two = json.loads([l for l in out.stdout.strip().splitlines() if l.startswith("{")][-1])
    assert two["train"]["optimizer_steps"] == 8
    a = ST.load_file(str(tmp_path / "one" / "adapter-trained" / "adapter_model.safetensors"))
    b = ST.load_file(str(tmp_path / "two" / "adapter-trained" / "adapter_model.safetensors"))
    for k in a:
        torch.testing.assert_close(a[k], b[k], atol=2e-5, rtol=1e-3)
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"recipe": "rlhf"}))
    assert main(["finetune", "run", str(bad)]) == 2


def test_smoke_fast_runs_every_recipe_on_synthetic_checkpoints(tmp_path, capsys):
    from antfly_b200.cli import main

    assert main(["finetune", "smoke-fast", str(tmp_path / "smoke")]) == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summary["ok"] and set(summary["cases"]) == set(R.RECIPES)
    assert all(c["manifest_status"] == "succeeded" for c in summary["cases"].values())
    assert os.path.exists(tmp_path / "smoke" / "fast_smoke_summary.json")


def test_bf16_base_weights_with_activation_checkpointing(tmp_path):
    _tiny_llama(str(tmp_path / "m"))
    rec = _sft_recipe(tmp_path, "qlora-sft", model={"dtype": "bf16"},
                      optimizer={"epochs": 5, "gradient_checkpointing": True, "neftune_alpha": 1.0})
    rep = R.run_recipe(rec)
    assert rep["status"] == "succeeded" and rep["train"]["final_loss"] < 0.7 * rep["train"]["first_loss"]
