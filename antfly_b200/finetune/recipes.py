"""Recipe runner: one JSON file names the algorithm, the model, the data, the adapter, the optimiser and where the
artifacts go; ``finetune run recipe.json`` prepares, trains, evaluates and (optionally) materialises a merged
checkpoint, and leaves a run manifest behind.

The schema and the manifest follow the reference's unified recipes
(zig/pkg/inference/docs/finetuning/FINETUNING.md "Unified Recipes": sections ``recipe / model / dataset / adapter /
optimizer / preference / grpo / eval / artifacts``; recipes ``sft``, ``lora-sft``, ``qlora-sft``, ``dpo``, ``grpo``,
``reranker``; LoRA defaults rank 16 / alpha 32 (GRPO: rank 8); manifest schema
``antfly_inference_finetune_recipe_run/v1`` with run status planned / running / succeeded / failed and per-step
records, plus ``training_config.json`` and ``training_report.json``; ``--dry-run`` prints the plan).  ``embedder``
(contrastive retrieval tuning of a BERT-family encoder) is added to the list; unknown fields are ignored so recipe
files can grow.
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from typing import Dict, List, Optional, Tuple

import torch

from ..formats import lora as MERGE
from ..formats import manifest as MF
from ..formats import safetensors_io as ST
from ..models.bert import BertConfig
from ..models.llama import LlamaConfig
from ..tokenizer import load_tokenizer
from . import data as D
from . import lora as L
from . import losses as LS
from .nets import DecoderNet, EncoderNet
from .trainer import TrainConfig, Trainer, adapters_disabled, sample_completions

RECIPES = ("sft", "lora-sft", "qlora-sft", "dpo", "grpo", "reranker", "embedder")
DECODER_RECIPES = ("sft", "lora-sft", "qlora-sft", "dpo", "grpo")
SCHEMA = "antfly_inference_finetune_recipe_run/v1"


class RecipeError(ValueError):
    pass


def normalize(recipe: dict) -> dict:
    """Validate and fill defaults; returns a new dictionary with every section present."""
    name = str(recipe.get("recipe", "")).lower()
    if name not in RECIPES:
        raise RecipeError(f"unknown recipe {recipe.get('recipe')!r}; expected one of {list(RECIPES)}")
    out = {k: dict(recipe.get(k) or {}) for k in ("model", "dataset", "adapter", "optimizer", "preference", "grpo",
                                                  "eval", "artifacts")}
    out["recipe"], out["backend"] = name, recipe.get("backend", "auto")
    if not out["model"].get("path"):
        raise RecipeError("model.path is required")
    ds = out["dataset"]
    if not (ds.get("path") or ds.get("train_path")):
        raise RecipeError("dataset.path or dataset.train_path is required")
    ds.setdefault("max_seq_len", 512)
    ad = out["adapter"]
    ad.setdefault("rank", 8 if name == "grpo" else 16)
    ad.setdefault("alpha", 32)
    ad.setdefault("target_preset", "all-linear")
    scaling = str(ad.get("scaling", "standard")).lower()
    if scaling not in ("standard", "lora", "rslora", "rank-stabilized"):
        raise RecipeError(f"adapter.scaling {ad.get('scaling')!r} is not supported")
    ad["rslora"] = scaling in ("rslora", "rank-stabilized")
    L.target_names(ad.get("target_preset"), ad.get("target_modules"))          # validates the preset
    op = out["optimizer"]
    op.setdefault("learning_rate", 2e-4)
    op.setdefault("epochs", 1)
    op.setdefault("batch_size", 1)
    op.setdefault("gradient_accumulation_steps", 1)
    op.setdefault("max_grad_norm", 1.0)
    out["preference"].setdefault("beta", 0.1)
    gr = out["grpo"]
    gr.setdefault("group_size", 8)
    gr.setdefault("clip_epsilon", 0.2)
    gr.setdefault("kl_coef", 0.04)
    gr.setdefault("normalize_advantage", True)
    gr.setdefault("max_completion_tokens", 16)
    gr.setdefault("reward_mode", "exact-match")
    if gr["reward_mode"] not in ("exact-match", "exact-match-ci", "prefix-match"):
        raise RecipeError(f"grpo.reward_mode {gr['reward_mode']!r} is not supported")
    art = out["artifacts"]
    art.setdefault("root", os.path.join(os.path.dirname(os.path.abspath(out["model"]["path"])), "finetune-run"))
    art.setdefault("manifest_path", os.path.join(art["root"], "recipe_run_manifest.json"))
    art.setdefault("trained_adapter_dir", os.path.join(art["root"], "adapter-trained"))
    return out


def plan(recipe: dict) -> List[dict]:
    r = normalize(recipe)
    steps = [{"name": "prepare", "what": f"tokenise {r['dataset'].get('train_path') or r['dataset'].get('path')} "
                                         f"(max_seq_len {r['dataset']['max_seq_len']})"},
             {"name": "train", "what": f"{r['recipe']}: rank {r['adapter']['rank']}, alpha {r['adapter']['alpha']}, "
                                       f"lr {r['optimizer']['learning_rate']}, epochs {r['optimizer']['epochs']}"}]
    if r["dataset"].get("eval_path"):
        steps.append({"name": "eval", "what": f"loss / accuracy on {r['dataset']['eval_path']}"})
    if r["artifacts"].get("materialized_dir"):
        steps.append({"name": "materialize", "what": f"merged checkpoint into {r['artifacts']['materialized_dir']}"})
    return steps


def reward(text: str, target: str, mode: str) -> float:
    a, b = text.strip(), target.strip()
    if mode == "exact-match-ci":
        return float(a.lower() == b.lower())
    if mode == "prefix-match":
        return float(a.startswith(b))
    return float(a == b)


# ----------------------------------------------------------------------------------------------------------
class _Run:
    def __init__(self, recipe: dict, dist: Optional[Tuple[int, int]] = None, device: str = "cpu",
                 resume_from: Optional[str] = None, log=None):
        self.r = normalize(recipe)
        self.original, self.dist, self.device, self.resume_from = recipe, dist, torch.device(device), resume_from
        self.lead = dist is None or dist[0] == 0
        self.log = log or (lambda rec: None)
        self.root = self.r["artifacts"]["root"]
        self.steps = [{"name": s["name"], "what": s["what"], "status": "planned"} for s in plan(recipe)]
        self.report: Dict[str, object] = {}

    # -- manifest ------------------------------------------------------------------------------------------
    def _write_manifest(self, status: str, error: Optional[str] = None):
        if not self.lead:
            return
        os.makedirs(self.root, exist_ok=True)
        body = {"schema": SCHEMA, "status": status, "recipe": self.original, "artifact_root": self.root,
                "steps": self.steps, "updated_unix": time.time()}
        if error:
            body["error"] = error
        with open(self.r["artifacts"]["manifest_path"], "w", encoding="utf-8") as f:
            json.dump(body, f, indent=1)

    def _step(self, name: str, fn):
        rec = next((s for s in self.steps if s["name"] == name), None)
        if rec is None:
            return None
        rec["status"] = "running"
        self._write_manifest("running")
        t0 = time.time()
        try:
            out = fn()
        except Exception:
            rec["status"] = "failed"
            raise
        rec["status"], rec["seconds"] = "succeeded", round(time.time() - t0, 3)
        return out

    # -- model ---------------------------------------------------------------------------------------------
    def _load(self):
        r = self.r
        path = r["model"]["path"]
        mf = MF.read_manifest(path)
        if mf.weights != "safetensors":
            raise RecipeError(f"{path}: fine-tuning reads safetensors checkpoints (found {mf.weights})")
        sd = ST.load_model_dir(path)
        self.tok = load_tokenizer(path, mf.config.get("vocab_size", 0))
        self.template = mf.chat_template
        name = r["recipe"]
        ckpt = bool(r["optimizer"].get("gradient_checkpointing", False))
        if name in DECODER_RECIPES:
            self.cfg = LlamaConfig.from_hf(mf.config)
            dtype = {"bf16": torch.bfloat16, "fp32": torch.float32}[r["model"].get("dtype", "fp32")]
            self.net = DecoderNet(self.cfg, sd, dtype=dtype, checkpointing=ckpt)
            self.net.neftune_alpha = float(r["optimizer"].get("neftune_alpha", 0.0))
        else:
            self.cfg = BertConfig.from_hf(mf.config)
            if name == "reranker" and not self.cfg.num_labels:
                raise RecipeError("the reranker recipe needs a checkpoint with a classification head")
            self.net = EncoderNet(self.cfg, sd, checkpointing=ckpt)
        ad = r["adapter"]
        if name == "sft":                                     # full-parameter tuning: everything but embeddings
            for n, p in self.net.named_parameters():
                p.requires_grad_(True)
            self.net.model.embed_tokens.weight.requires_grad_(False)
            if self.cfg.tie_word_embeddings:                  # the output matrix is the (frozen) embedding table
                self.net.lm_head.weight.requires_grad_(False)
            self.adapted = []
        else:
            self.adapted = L.inject(self.net, int(ad["rank"]), float(ad["alpha"]), ad.get("target_preset"),
                                    ad.get("target_modules"), float(ad.get("dropout", 0.0)), nf4=name == "qlora-sft",
                                    rslora=ad["rslora"], seed=int(r["optimizer"].get("seed", 0)))
            if ad.get("path") and os.path.exists(os.path.join(ad["path"], "adapter_model.safetensors")):
                L.load_adapter(self.net, ad["path"])          # continue from a bootstrap adapter
        self.net.to(self.device)

    def _save_weights(self, d: str):
        ad = self.r["adapter"]
        if self.adapted:
            L.save_adapter(self.net, d, int(ad["rank"]), float(ad["alpha"]), self.adapted, ad["rslora"],
                           base_model=self.r["model"]["path"])
        else:
            sd = {k: v.detach().cpu() for k, v in self.net.state_dict().items() if k != "inv_freq"}
            if getattr(self.cfg, "tie_word_embeddings", False):
                sd.pop("lm_head.weight", None)
            ST.save_file(sd, os.path.join(d, "model.safetensors"))

    def _load_weights(self, d: str):
        if self.adapted:
            L.load_adapter(self.net, d)
        else:
            self.net.load_state_dict({k: v.to(self.device) for k, v in ST.load_file(
                os.path.join(d, "model.safetensors")).items()}, strict=False)

    # -- data ----------------------------------------------------------------------------------------------
    def _rows(self, which: str) -> List[dict]:
        ds = self.r["dataset"]
        if which == "train":
            return D.read_jsonl(ds.get("train_path") or ds["path"], int(ds.get("max_examples", 0)))
        return D.read_jsonl(ds["eval_path"], int(ds.get("eval_max_examples") or self.r["eval"].get("max_examples", 0)))

    def _prepare(self):
        r, name = self.r, self.r["recipe"]
        S = int(r["dataset"]["max_seq_len"])
        rows = self._rows("train")
        if not rows:
            raise RecipeError("the training set is empty")
        fmt = str(r["dataset"].get("format", ""))
        if name in DECODER_RECIPES:
            self.dtok = D.DecoderTokenizer(self.tok, self.template, rendered=fmt.startswith("rendered"),
                                           add_bos=not r["dataset"].get("no_bos", False))
        pad = self.tok.special.pad_id or 0
        if name in ("sft", "lora-sft", "qlora-sft"):
            ex = [self.dtok.sft_example(x, S) for x in rows]
            self.items = D.pack_examples(ex, S, pad) if r["dataset"].get("packing", True) else [
                {"ids": e.ids, "loss_mask": e.loss_mask, "doc_ids": None} for e in ex]
            self.report["packing"] = {"examples": len(ex), "rows": len(self.items),
                                      "tokens": sum(len(e) for e in ex), "row_length": S}
        elif name == "dpo":
            self.items = []
            for x in rows:
                p = self.dtok.prompt_ids(x["prompt"])[-(S // 2):]
                c, j = self.dtok.completion_ids(str(x["chosen"])), self.dtok.completion_ids(str(x["rejected"]))
                self.items.append({"prompt": p, "chosen": c[: S - len(p)], "rejected": j[: S - len(p)]})
        elif name == "grpo":
            self.items = [{"prompt": self.dtok.prompt_ids(x["prompt"])[-S:], "target": str(x.get("target", x.get("answer", "")))}
                          for x in rows]
        elif name == "reranker":
            self.items = D.encoder_pairs(self.tok, rows, S)
        else:
            self.items = D.encoder_triples(self.tok, rows, S, r["dataset"].get("query_prefix", ""),
                                           r["dataset"].get("document_prefix", ""))
        return len(self.items)

    # -- recipe steps --------------------------------------------------------------------------------------
    def _sft_step(self, batch):
        dev = self.device
        if batch[0]["doc_ids"] is not None:
            ids = torch.tensor([b["ids"] for b in batch], device=dev)
            lm = torch.tensor([b["loss_mask"] for b in batch], device=dev).bool()
            doc = torch.tensor([b["doc_ids"] for b in batch], device=dev)
            hidden = self.net(ids, doc_ids=doc)
        else:
            ids, att, lm = D.pad_batch([b["ids"] for b in batch], self.tok.special.pad_id or 0,
                                       [b["loss_mask"] for b in batch])
            ids, att, lm, doc = ids.to(dev), att.to(dev), lm.to(dev), None
            hidden = self.net(ids, pad_mask=att)
        loss, n = LS.causal_lm_loss(self.net, hidden, ids, lm, doc)
        return loss, {"tokens": n}

    def _seq_logps(self, prompts, completions):
        seqs = [p + c for p, c in zip(prompts, completions)]
        masks = [[0] * len(p) + [1] * len(c) for p, c in zip(prompts, completions)]
        ids, att, lm = D.pad_batch(seqs, self.tok.special.pad_id or 0, masks)
        ids, att, lm = ids.to(self.device), att.to(self.device), lm.to(self.device)
        return LS.sequence_logps(self.net, self.net(ids, pad_mask=att), ids, lm)

    def _dpo_step(self, batch):
        P = [b["prompt"] for b in batch]
        both = self._seq_logps(P + P, [b["chosen"] for b in batch] + [b["rejected"] for b in batch])
        with torch.no_grad(), adapters_disabled(self.net):
            ref = self._seq_logps(P + P, [b["chosen"] for b in batch] + [b["rejected"] for b in batch])
        n = len(batch)
        return LS.dpo_loss(both[:n], both[n:], ref[:n], ref[n:], float(self.r["preference"]["beta"]))

    def _token_logps(self, prompts, completions):
        """Per-token log-probabilities of the completions -> ([N, T] padded, mask [N, T])."""
        seqs = [p + c for p, c in zip(prompts, completions)]
        ids, att, _ = D.pad_batch(seqs, self.tok.special.pad_id or 0)
        ids, att = ids.to(self.device), att.to(self.device)
        hidden = self.net(ids, pad_mask=att)
        tgt = ids[:, 1:].clone()
        lp = LS.chunked_token_logps(self.net, hidden[:, :-1].reshape(-1, hidden.shape[-1]), tgt.reshape(-1)).view(
            ids.shape[0], -1)
        T = max(len(c) for c in completions)
        out = lp.new_zeros(len(seqs), T)
        mask = torch.zeros(len(seqs), T, dtype=torch.bool, device=self.device)
        for i, (p, c) in enumerate(zip(prompts, completions)):
            out[i, : len(c)] = lp[i, len(p) - 1: len(p) - 1 + len(c)]
            mask[i, : len(c)] = True
        return out, mask

    def _grpo_step(self, batch):
        g = self.r["grpo"]
        G = int(g["group_size"])
        prompts, comps, rewards = [], [], []
        self.net.eval()
        for b in batch:
            outs = sample_completions(self.net, b["prompt"], G, int(g["max_completion_tokens"]),
                                      float(g.get("temperature", 1.0)), self.tok.special.eos_id, self._gen, self.device)
            for o in outs:
                text = self.tok.decode([t for t in o if t != self.tok.special.eos_id])
                prompts.append(b["prompt"])
                comps.append(o if o else [self.tok.special.eos_id or 0])
                rewards.append(reward(text, b["target"], g["reward_mode"]))
        self.net.train()
        rew = torch.tensor(rewards, device=self.device)
        adv = LS.grpo_advantages(rew, G, bool(g["normalize_advantage"]))
        new, mask = self._token_logps(prompts, comps)
        with torch.no_grad():
            old = new.detach()
            with adapters_disabled(self.net):
                ref, _ = self._token_logps(prompts, comps)
        loss, m = LS.grpo_loss(new, old, ref, adv, mask, float(g["clip_epsilon"]), float(g["kl_coef"]))
        m["reward"] = float(rew.mean())
        return loss, m

    def _encode(self, seqs, types=None):
        ids, att, _ = D.pad_batch(seqs, self.tok.special.pad_id or 0)
        tt = None
        if types is not None:
            tt, _, _ = D.pad_batch(types, 0)
            tt = tt.to(self.device)
        ids, att = ids.to(self.device), att.to(self.device)
        return self.net(ids, att.long(), tt), att

    def _reranker_step(self, batch):
        states, _ = self._encode([b["ids"] for b in batch], [b["types"] for b in batch])
        scores = self.net.score(states)[:, 0]
        labels = torch.tensor([b["label"] for b in batch], device=self.device)
        groups = torch.tensor([b["group"] for b in batch], device=self.device)
        return LS.reranker_loss(scores, labels, groups, self.r["optimizer"].get("reranker_loss", "bce")), {}

    def _embedder_step(self, batch):
        """InfoNCE over (query, positive) with in-batch negatives, optional hard negatives, an optional cross-batch
        memory of earlier positives (``optimizer.xbm_capacity``) and Matryoshka prefixes (``optimizer.mrl_dims``: the
        loss is averaged over the embedding truncated to each size and re-normalised), as in the reference's
        contrastive trainer (zig/pkg/inference/docs/finetuning/FINETUNING.md "Cross-Batch Memory", "Matryoshka")."""
        op = self.r["optimizer"]

        def emb(seqs):
            st, att = self._encode(seqs)
            return self.net.pool(st, att, normalize=False)

        q, p = emb([b["query"] for b in batch]), emb([b["positive"] for b in batch])
        n_neg = min((len(b["negatives"]) for b in batch), default=0)
        neg = None
        if n_neg:
            neg = emb([n for b in batch for n in b["negatives"][:n_neg]]).view(len(batch), n_neg, -1)
        dims = [int(d) for d in op.get("mrl_dims") or [q.shape[-1]]]
        bank, bank_ids = getattr(self, "_xbm", None), getattr(self, "_xbm_ids", None)
        self._emb_steps = getattr(self, "_emb_steps", 0) + (1 if self.net.training else 0)
        # the memory assumes embeddings that drift slowly: it is switched on after optimizer.xbm_warmup_steps
        # micro-steps, once the encoder has left its starting point
        warm = self._emb_steps > int(op.get("xbm_warmup_steps", 0))
        use_bank = bank is not None and self.net.training and warm
        ids = torch.tensor([b.get("doc", -1) for b in batch], device=self.device)
        exclude = ids[:, None] == bank_ids[None, :] if use_bank else None
        temp = float(op.get("temperature", 0.05))
        norm = lambda t, d: torch.nn.functional.normalize(t[..., :d], dim=-1)
        total, metrics = 0.0, {}
        for d in dims:
            loss, m = LS.info_nce(norm(q, d), norm(p, d), norm(neg, d) if neg is not None else None, temp,
                                  norm(bank, d) if use_bank else None, exclude)
            total = total + loss / len(dims)
            metrics = m if d == dims[0] else metrics
        cap = int(op.get("xbm_capacity", 0))
        if cap and self.net.training and warm:
            new = p.detach()
            self._xbm = new if bank is None else torch.cat([bank, new], 0)[-cap:]
            self._xbm_ids = ids if bank_ids is None else torch.cat([bank_ids, ids], 0)[-cap:]
        return total, metrics

    def _train(self):
        r, name = self.r, self.r["recipe"]
        op = r["optimizer"]
        known = TrainConfig.__dataclass_fields__
        cfg = TrainConfig(**{k: v for k, v in op.items() if k in known})
        world = self.dist[1] if self.dist else 1
        rank = self.dist[0] if self.dist else 0
        per_epoch = max(len(self.items) // (cfg.batch_size * world), 1)
        total = max(per_epoch * cfg.epochs // cfg.gradient_accumulation_steps, 1)
        if cfg.max_steps:
            total = min(total, cfg.max_steps)
        step_fn = {"sft": self._sft_step, "lora-sft": self._sft_step, "qlora-sft": self._sft_step,
                   "dpo": self._dpo_step, "grpo": self._grpo_step, "reranker": self._reranker_step,
                   "embedder": self._embedder_step}[name]
        self._gen = torch.Generator().manual_seed(cfg.seed + 1000 * rank)
        trainer = Trainer(self.net, cfg, os.path.join(self.root, "checkpoints"), self.dist, self._save_weights,
                          self._load_weights)
        start = 0
        if self.resume_from:
            trainer.resume(self.resume_from)
            start = trainer.step * cfg.gradient_accumulation_steps
        it = (b for _, _, b in D.batches(self.items, cfg.batch_size, cfg.epochs, cfg.seed, rank, world, start))
        hist = trainer.fit(it, step_fn, total, self.log)
        out = r["artifacts"]["trained_adapter_dir"]
        if self.lead:
            os.makedirs(out, exist_ok=True)
            self._save_weights(out)
            trainer.save("final")
        trainable = sum(p.numel() for _, p in trainer.params)
        self.report["train"] = {"optimizer_steps": trainer.step, "first_loss": hist[0]["loss"] if hist else None,
                                "final_loss": hist[-1]["loss"] if hist else None, "trainable_parameters": trainable,
                                "adapted_modules": len(self.adapted),
                                "avg_step_ms": sum(h["step_ms"] for h in hist) / max(len(hist), 1)}
        return self.report["train"]

    @torch.no_grad()
    def _eval(self):
        name = self.r["recipe"]
        rows = self._rows("eval")
        keep, self.items = self.items, None
        S = int(self.r["dataset"]["max_seq_len"])
        self.net.eval()
        try:
            if name in ("sft", "lora-sft", "qlora-sft"):
                ex = [self.dtok.sft_example(x, S) for x in rows]
                tot, cnt = 0.0, 0
                for e in ex:
                    loss, n = self._sft_step([{"ids": e.ids, "loss_mask": e.loss_mask, "doc_ids": None}])[0], sum(e.loss_mask[1:])
                    tot, cnt = tot + float(loss) * n, cnt + n
                res = {"loss": tot / max(cnt, 1), "tokens": cnt}
            elif name == "dpo":
                items = []
                for x in rows:
                    p = self.dtok.prompt_ids(x["prompt"])
                    items.append({"prompt": p, "chosen": self.dtok.completion_ids(str(x["chosen"])),
                                  "rejected": self.dtok.completion_ids(str(x["rejected"]))})
                loss, m = self._dpo_step(items)
                res = {"loss": float(loss), **m}
            elif name == "grpo":
                hits = 0
                for x in rows:
                    out = sample_completions(self.net, self.dtok.prompt_ids(x["prompt"]), 1,
                                             int(self.r["grpo"]["max_completion_tokens"]), 0.0,
                                             self.tok.special.eos_id, None, self.device)[0]
                    text = self.tok.decode([t for t in out if t != self.tok.special.eos_id])
                    hits += reward(text, str(x.get("target", x.get("answer", ""))), self.r["grpo"]["reward_mode"])
                res = {"greedy_reward": hits / max(len(rows), 1)}
            elif name == "reranker":
                items = D.encoder_pairs(self.tok, rows, S)
                loss, _ = self._reranker_step(items)
                res = {"loss": float(loss)}
            else:
                items = D.encoder_triples(self.tok, rows, S)
                loss, m = self._embedder_step(items)
                res = {"loss": float(loss), **m}
        finally:
            self.items = keep
        self.report["eval"] = res
        return res

    def _materialize(self):
        """The base checkpoint with the trained adapter folded in, as a model directory the server loads."""
        out = self.r["artifacts"]["materialized_dir"]
        src = self.r["model"]["path"]
        os.makedirs(out, exist_ok=True)
        sd = ST.load_model_dir(src)
        if self.adapted:
            with open(os.path.join(self.r["artifacts"]["trained_adapter_dir"], "adapter_config.json")) as f:
                cfg = json.load(f)
            MERGE.merge_lora(sd, L.adapter_state(self.net), cfg)
        else:
            sd.update({k: v.detach().cpu() for k, v in self.net.state_dict().items() if k in sd})
        ST.save_file(sd, os.path.join(out, "model.safetensors"))
        for n in os.listdir(src):
            if n.endswith((".json", ".txt", ".model", ".jinja")) and not n.startswith("adapter_"):
                with open(os.path.join(src, n), "rb") as a, open(os.path.join(out, n), "wb") as b:
                    b.write(a.read())
        return out

    def run(self) -> dict:
        self._write_manifest("planned")
        try:
            self._step("prepare", lambda: (self._load(), self._prepare()))
            self._step("train", self._train)
            self._step("eval", self._eval)
            if self.lead:
                self._step("materialize", self._materialize)
        except Exception as e:
            self._write_manifest("failed", f"{type(e).__name__}: {e}")
            raise
        self._write_manifest("succeeded")
        if self.lead:
            ds = self.r["dataset"]
            prints = {k: D.fingerprint(ds[k]) for k in ("path", "train_path", "eval_path") if ds.get(k)}
            with open(os.path.join(self.root, "training_config.json"), "w", encoding="utf-8") as f:
                json.dump({"recipe": self.r, "plan": plan(self.original), "datasets": prints,
                           "torch": torch.__version__, "device": str(self.device)}, f, indent=1)
            sums = {}
            d = self.r["artifacts"]["trained_adapter_dir"]
            for n in sorted(os.listdir(d)):
                with open(os.path.join(d, n), "rb") as f:
                    sums[n] = hashlib.sha256(f.read()).hexdigest()
            self.report.update({"status": "succeeded", "steps": self.steps, "datasets": prints, "artifacts": sums})
            with open(os.path.join(self.root, "training_report.json"), "w", encoding="utf-8") as f:
                json.dump(self.report, f, indent=1)
        return self.report


def run_recipe(recipe: dict, dist: Optional[Tuple[int, int]] = None, device: str = "cpu",
               resume_from: Optional[str] = None, log=None) -> dict:
    return _Run(recipe, dist, device, resume_from, log).run()


# ----------------------------------------------------------------------------------------------------------
# self-check without any downloaded model
# ----------------------------------------------------------------------------------------------------------
def _synthetic_decoder(path: str, seed: int = 0) -> None:
    g = torch.Generator().manual_seed(seed)
    H, F, V, L_, nh, nkv = 32, 64, 300, 1, 4, 2
    D_ = H // nh
    rnd = lambda *s, std=0.05: torch.randn(*s, generator=g) * std
    sd = {"model.embed_tokens.weight": rnd(V, H, std=0.5), "model.norm.weight": torch.ones(H),
          "lm_head.weight": rnd(V, H, std=0.3)}
    for l in range(L_):
        p = f"model.layers.{l}."
        sd.update({p + "self_attn.q_proj.weight": rnd(nh * D_, H), p + "self_attn.k_proj.weight": rnd(nkv * D_, H),
                   p + "self_attn.v_proj.weight": rnd(nkv * D_, H), p + "self_attn.o_proj.weight": rnd(H, nh * D_),
                   p + "mlp.gate_proj.weight": rnd(F, H), p + "mlp.up_proj.weight": rnd(F, H),
                   p + "mlp.down_proj.weight": rnd(H, F), p + "input_layernorm.weight": torch.ones(H),
                   p + "post_attention_layernorm.weight": torch.ones(H)})
    os.makedirs(path, exist_ok=True)
    ST.save_file(sd, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump({"model_type": "llama", "hidden_size": H, "intermediate_size": F, "num_hidden_layers": L_,
                   "num_attention_heads": nh, "num_key_value_heads": nkv, "vocab_size": V, "rope_theta": 10000.0,
                   "rms_norm_eps": 1e-5, "max_position_embeddings": 256, "tie_word_embeddings": False}, f)


def _synthetic_encoder(path: str, num_labels: int, seed: int = 0) -> None:
    from ..models.bert import BertModel

    cfg = BertConfig(hidden_size=32, num_hidden_layers=1, num_attention_heads=4, intermediate_size=64, vocab_size=300,
                     num_labels=num_labels)
    m = BertModel.random_init(cfg, device="cpu", seed=seed)
    os.makedirs(path, exist_ok=True)
    ST.save_file(m.state_dict_hf(), os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump({"model_type": "bert", "hidden_size": 32, "num_hidden_layers": 1, "num_attention_heads": 4,
                   "intermediate_size": 64, "vocab_size": 300, "max_position_embeddings": 512,
                   "num_labels": num_labels}, f)


def smoke_fast(root: str) -> dict:
    """Every recipe once on synthetic checkpoints and a handful of rows (no model or dataset needed): the plan of
    each, a short run of each, and the check that its manifest ends ``succeeded``.  The summary is also written to
    ``<root>/fast_smoke_summary.json`` (the reference's ``finetune smoke-fast``)."""
    os.makedirs(root, exist_ok=True)
    dec, enc, rr = os.path.join(root, "decoder"), os.path.join(root, "encoder"), os.path.join(root, "reranker")
    _synthetic_decoder(dec)
    _synthetic_encoder(enc, 0)
    _synthetic_encoder(rr, 1)

    def write(name, rows):
        p = os.path.join(root, name)
        with open(p, "w", encoding="utf-8") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        return p

    sft = write("sft.jsonl", [{"prompt": "ab", "completion": "xy"}, {"text": "plain row"}] * 2)
    pref = write("pref.jsonl", [{"prompt": "pick", "chosen": "good", "rejected": "bad"}] * 2)
    grpo = write("grpo.jsonl", [{"prompt": "say a", "target": "a"}] * 2)
    pairs = write("pairs.jsonl", [{"query": "q", "document": "yes", "label": 1}, {"query": "q", "document": "no", "label": 0}])
    trip = write("trip.jsonl", [{"query": "q1", "positive": "p1"}, {"query": "q2", "positive": "p2"}])
    cases = {"lora-sft": (dec, sft), "qlora-sft": (dec, sft), "sft": (dec, sft), "dpo": (dec, pref), "grpo": (dec, grpo),
             "reranker": (rr, pairs), "embedder": (enc, trip)}
    summary = {"cases": {}, "ok": True}
    for name, (model, data) in cases.items():
        recipe = {"recipe": name, "model": {"path": model}, "dataset": {"path": data, "max_seq_len": 48},
                  "adapter": {"rank": 2, "alpha": 4}, "grpo": {"group_size": 2, "max_completion_tokens": 2},
                  "optimizer": {"epochs": 1, "batch_size": 2, "learning_rate": 1e-3},
                  "artifacts": {"root": os.path.join(root, "run-" + name)}}
        rec = {"plan": [s["name"] for s in plan(recipe)]}
        try:
            rep = run_recipe(recipe)
            with open(os.path.join(root, "run-" + name, "recipe_run_manifest.json"), encoding="utf-8") as f:
                rec["manifest_status"] = json.load(f)["status"]
            rec["final_loss"] = rep["train"]["final_loss"]
            rec["ok"] = rec["manifest_status"] == "succeeded" and rep["train"]["final_loss"] == rep["train"]["final_loss"]
        except Exception as e:                                  # the suite reports, the caller decides
            rec["ok"], rec["error"] = False, f"{type(e).__name__}: {e}"
        summary["cases"][name] = rec
        summary["ok"] = summary["ok"] and rec["ok"]
    with open(os.path.join(root, "fast_smoke_summary.json"), "w", encoding="utf-8") as f:
        json.dump(summary, f, indent=1)
    return summary
