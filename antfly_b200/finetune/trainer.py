"""Training loop: AdamW with warm-up and cosine / linear decay, gradient accumulation, global-norm clipping, LoRA+
learning-rate ratio, data-parallel gradient averaging, checkpoints that resume exactly.

The reference's loop and its knobs (zig/pkg/inference/docs/finetuning/FINETUNING.md: "Training Loop", "AdamW
Optimizer", "Global Gradient Norm Clipping" --max-grad-norm, "Gradient Accumulation" --grad-accum, "LoRA+"
--lora-plus-ratio, "SafeTensors Checkpoint Format" with adam_m_* / adam_v_* / adam_step optimizer files,
--checkpoint-every / --resume-from; "Distributed Training": N ranks, gradients averaged every step).  Ranks are
``torch.distributed`` processes (NCCL on GPUs, gloo on CPU); only the trainable parameters' gradients cross the
wire, which for adapters is a few megabytes.
"""
from __future__ import annotations

import json
import math
import os
import time
from contextlib import contextmanager
from dataclasses import asdict, dataclass
from typing import Callable, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from ..formats import safetensors_io as ST
from . import lora as L


@dataclass
class TrainConfig:
    learning_rate: float = 2e-4
    epochs: int = 1
    batch_size: int = 1
    gradient_accumulation_steps: int = 1
    max_grad_norm: float = 1.0
    weight_decay: float = 0.0
    warmup_ratio: float = 0.03
    schedule: str = "cosine"            # cosine | linear | constant
    lora_plus_ratio: float = 1.0        # learning rate of the B factors over that of the A factors
    seed: int = 0
    checkpoint_every: int = 0           # optimizer steps; 0: only at the end
    save_optimizer_state: bool = True
    max_steps: int = 0                  # 0: run the epochs out
    log_every: int = 1


def lr_at(step: int, total: int, cfg: TrainConfig) -> float:
    warm = int(round(cfg.warmup_ratio * total))
    if warm and step < warm:
        return cfg.learning_rate * (step + 1) / warm
    if cfg.schedule == "constant" or total <= warm:
        return cfg.learning_rate
    frac = (step - warm) / max(total - warm, 1)
    if cfg.schedule == "linear":
        return cfg.learning_rate * max(0.0, 1.0 - frac)
    return cfg.learning_rate * 0.5 * (1.0 + math.cos(math.pi * min(frac, 1.0)))


@contextmanager
def adapters_disabled(model: nn.Module):
    """The base model's behaviour for the duration of the block (the reference policy of DPO / GRPO when no separate
    reference checkpoint is given)."""
    mods = [m for m in model.modules() if isinstance(m, L.LoraLinear)]
    saved = [m.scale for m in mods]
    for m in mods:
        m.scale = 0.0
    try:
        yield
    finally:
        for m, s in zip(mods, saved):
            m.scale = s


class Trainer:
    """``step_fn(batch) -> (loss, metrics)`` is the recipe; everything else is here.  ``dist`` = (rank, world) of an
    initialised ``torch.distributed`` group, or None."""

    def __init__(self, model: nn.Module, cfg: TrainConfig, out_dir: str, dist: Optional[Tuple[int, int]] = None,
                 save_fn: Optional[Callable[[str], None]] = None, load_fn: Optional[Callable[[str], None]] = None):
        self.model, self.cfg, self.out_dir, self.dist = model, cfg, out_dir, dist
        self.params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("nothing to train: no parameter requires a gradient")
        fast = [p for n, p in self.params if n.endswith("lora_B")]
        slow = [p for n, p in self.params if not n.endswith("lora_B")]
        groups = [{"params": slow, "lr_scale": 1.0}]
        if fast:
            groups.append({"params": fast, "lr_scale": cfg.lora_plus_ratio})
        self.opt = torch.optim.AdamW(groups, lr=cfg.learning_rate, weight_decay=cfg.weight_decay, betas=(0.9, 0.999))
        self.step = 0                       # optimizer steps taken
        self.history: List[dict] = []
        self.save_fn, self.load_fn = save_fn, load_fn
        os.makedirs(out_dir, exist_ok=True)

    # -- checkpoints ---------------------------------------------------------------------------------------
    def save(self, tag: str) -> str:
        d = os.path.join(self.out_dir, tag)
        os.makedirs(d, exist_ok=True)
        if self.save_fn:
            self.save_fn(d)
        if self.cfg.save_optimizer_state:
            st = {}
            for n, p in self.params:
                s = self.opt.state.get(p)
                if s:
                    st["adam_m_" + n], st["adam_v_" + n] = s["exp_avg"].float().cpu(), s["exp_avg_sq"].float().cpu()
            ST.save_file(st, os.path.join(d, "optimizer.safetensors"))
        with open(os.path.join(d, "trainer_state.json"), "w", encoding="utf-8") as f:
            json.dump({"adam_step": self.step, "config": asdict(self.cfg), "history": self.history[-50:]}, f)
        return d

    def resume(self, d: str) -> None:
        if self.load_fn:
            self.load_fn(d)
        with open(os.path.join(d, "trainer_state.json"), encoding="utf-8") as f:
            state = json.load(f)
        self.step = int(state["adam_step"])
        path = os.path.join(d, "optimizer.safetensors")
        if os.path.exists(path):
            st = ST.load_file(path)
            for n, p in self.params:
                if "adam_m_" + n in st:
                    self.opt.state[p] = {"step": torch.tensor(float(self.step)),
                                         "exp_avg": st["adam_m_" + n].to(p.device, p.dtype).clone(),
                                         "exp_avg_sq": st["adam_v_" + n].to(p.device, p.dtype).clone()}

    # -- the loop ------------------------------------------------------------------------------------------
    def _average_gradients(self) -> None:
        if self.dist is None or self.dist[1] == 1:
            return
        import torch.distributed as D

        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float()
                          for _, p in self.params])
        D.all_reduce(flat)
        flat /= self.dist[1]
        off = 0
        for _, p in self.params:
            n = p.numel()
            p.grad = flat[off:off + n].view_as(p).to(p.dtype)
            off += n

    def fit(self, micro_batches: Iterable, step_fn: Callable, total_steps: int,
            on_step: Optional[Callable[[dict], None]] = None) -> List[dict]:
        """``micro_batches`` yields what ``step_fn`` consumes; ``gradient_accumulation_steps`` of them make one
        optimizer step.  ``total_steps`` (optimizer steps of the whole run) shapes the schedule."""
        cfg = self.cfg
        self.model.train()
        accum, loss_sum, metrics_sum, t0 = 0, 0.0, {}, time.time()
        for batch in micro_batches:
            loss, metrics = step_fn(batch)
            (loss / cfg.gradient_accumulation_steps).backward()
            loss_sum += float(loss.detach())
            for k, v in (metrics or {}).items():
                metrics_sum[k] = metrics_sum.get(k, 0.0) + float(v)
            accum += 1
            if accum < cfg.gradient_accumulation_steps:
                continue
            self._average_gradients()
            norm = float(torch.nn.utils.clip_grad_norm_([p for _, p in self.params],
                                                        cfg.max_grad_norm if cfg.max_grad_norm > 0 else float("inf")))
            lr = lr_at(self.step, total_steps, cfg)
            for g in self.opt.param_groups:
                g["lr"] = lr * g.get("lr_scale", 1.0)
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)
            self.step += 1
            rec = {"step": self.step, "loss": loss_sum / accum, "grad_norm": norm, "lr": lr,
                   "step_ms": (time.time() - t0) * 1e3, **{k: v / accum for k, v in metrics_sum.items()}}
            self.history.append(rec)
            if on_step:
                on_step(rec)
            accum, loss_sum, metrics_sum, t0 = 0, 0.0, {}, time.time()
            if cfg.checkpoint_every and self.step % cfg.checkpoint_every == 0 and (self.dist is None or self.dist[0] == 0):
                self.save(f"checkpoint-{self.step}")
            if cfg.max_steps and self.step >= cfg.max_steps:
                break
        self.model.eval()
        return self.history


@torch.no_grad()
def sample_completions(net, prompt_ids: List[int], n: int, max_new_tokens: int, temperature: float = 1.0,
                       eos_id: Optional[int] = None, generator: Optional[torch.Generator] = None,
                       device="cpu") -> List[List[int]]:
    """``n`` sampled continuations of one prompt from the network being trained (GRPO roll-outs).  The whole prefix
    is re-run each step: roll-outs during training are short, and this keeps the sampler free of cache state."""
    ids = torch.tensor([prompt_ids] * n, dtype=torch.long, device=device)
    done = torch.zeros(n, dtype=torch.bool, device=device)
    for _ in range(max_new_tokens):
        logits = net.logits(net(ids)[:, -1])
        if temperature <= 0:
            nxt = logits.argmax(-1)
        else:
            probs = torch.softmax(logits / temperature, -1)
            nxt = torch.multinomial(probs.cpu(), 1, generator=generator)[:, 0].to(device)
        if eos_id is not None:
            nxt = torch.where(done, torch.full_like(nxt, eos_id), nxt)
            done = done | (nxt == eos_id)
        ids = torch.cat([ids, nxt[:, None]], 1)
        if eos_id is not None and bool(done.all()):
            break
    out = []
    for row in ids[:, len(prompt_ids):].tolist():
        if eos_id is not None and eos_id in row:
            row = row[: row.index(eos_id) + 1]
        out.append(row)
    return out
