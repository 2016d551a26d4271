"""Low-rank adapters for training: wrapped linears, 4-bit (NF4) frozen bases, target presets, adapter files.

Counterpart of the reference's LoRA layer and adapter checkpoints (zig/lib/ml/src/graph/lora.zig; defaults and
presets in zig/pkg/inference/docs/finetuning/FINETUNING.md "LoRA Defaults": rank 16 / alpha 32, scale alpha / rank,
presets all-linear / attention-only / mlp-only; QLoRA with NF4 bases).  Adapters are written in the PEFT layout that
:mod:`antfly_b200.formats.lora` merges at load time, so a trained adapter is served by dropping it into the model
directory.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from ..formats import safetensors_io as ST

PRESETS = {
    "all-linear": ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj",
                   "query", "key", "value", "attention.output.dense", "intermediate.dense", "output.dense"),
    "attention-only": ("q_proj", "k_proj", "v_proj", "o_proj", "query", "key", "value", "attention.output.dense"),
    "mlp-only": ("gate_proj", "up_proj", "down_proj", "intermediate.dense", "output.dense"),
}

# The 16 levels of the 4-bit NormalFloat code: quantiles of a standard normal, scaled to [-1, 1], with an exact zero.
NF4_LEVELS = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0])


def nf4_quantize(w: torch.Tensor, block: int = 64):
    """[out, in] -> (codes uint8 [out * in / 2] two per byte, absmax fp32 per block of ``block`` values)."""
    flat = w.detach().float().reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    blocks = flat.view(-1, block)
    absmax = blocks.abs().amax(1).clamp_min(1e-12)
    idx = (blocks / absmax[:, None]).unsqueeze(-1).sub(NF4_LEVELS.to(flat.device)).abs().argmin(-1).to(torch.uint8)
    idx = idx.reshape(-1)
    return (idx[0::2] | (idx[1::2] << 4)).contiguous(), absmax


def nf4_dequantize(codes: torch.Tensor, absmax: torch.Tensor, shape, block: int = 64) -> torch.Tensor:
    idx = torch.stack([codes & 0xF, codes >> 4], 1).reshape(-1).long()
    vals = NF4_LEVELS.to(codes.device)[idx].view(-1, block) * absmax[:, None]
    n = 1
    for s in shape:
        n *= s
    return vals.reshape(-1)[:n].view(*shape)


class LoraLinear(nn.Module):
    """``y = x W^T + b + scale * (dropout(x) A^T) B^T`` with W frozen (kept as given, or as NF4 codes that are
    expanded per call) and A [r, in] / B [out, r] trainable.  B starts at zero, so training starts at the base model."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], rank: int, alpha: float,
                 dropout: float = 0.0, nf4: bool = False, rslora: bool = False, generator=None):
        super().__init__()
        out_f, in_f = weight.shape
        self.in_features, self.out_features, self.rank = in_f, out_f, rank
        self.scale = alpha / math.sqrt(rank) if rslora else alpha / rank
        self.nf4 = nf4
        if nf4:
            codes, absmax = nf4_quantize(weight)
            self.register_buffer("codes", codes)
            self.register_buffer("absmax", absmax)
            self.compute_dtype = weight.dtype if weight.dtype != torch.float32 else torch.float32
        else:
            self.register_buffer("weight", weight.detach())
        self.register_buffer("bias", bias.detach() if bias is not None else None)
        a = torch.empty(rank, in_f, dtype=torch.float32)
        nn.init.kaiming_uniform_(a, a=math.sqrt(5), generator=generator)
        self.lora_A = nn.Parameter(a)
        self.lora_B = nn.Parameter(torch.zeros(out_f, rank, dtype=torch.float32))
        self.drop = nn.Dropout(dropout) if dropout > 0 else None

    def base_weight(self) -> torch.Tensor:
        if self.nf4:
            return nf4_dequantize(self.codes, self.absmax, (self.out_features, self.in_features)).to(self.compute_dtype)
        return self.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.base_weight()
        y = torch.nn.functional.linear(x.to(w.dtype), w, self.bias)
        xa = self.drop(x) if self.drop is not None else x
        delta = (xa.float() @ self.lora_A.t()) @ self.lora_B.t()
        return y + (self.scale * delta).to(y.dtype)


def target_names(preset: Optional[str], target_modules: Optional[Sequence[str]]) -> Sequence[str]:
    if target_modules:
        return tuple(target_modules)
    key = (preset or "all-linear").replace("_", "-")
    if key == "moe-experts":
        raise ValueError("target_preset moe-experts is not supported: expert weights are not adapted")
    if key not in PRESETS:
        raise ValueError(f"unknown target_preset {preset!r}; expected one of {sorted(PRESETS)}")
    return PRESETS[key]


def inject(model: nn.Module, rank: int = 16, alpha: float = 32.0, preset: Optional[str] = "all-linear",
           target_modules: Optional[Sequence[str]] = None, dropout: float = 0.0, nf4: bool = False,
           rslora: bool = False, seed: int = 0) -> List[str]:
    """Replace every ``nn.Linear`` whose qualified name ends with a target by a :class:`LoraLinear`; freeze everything
    else.  Returns the adapted module names."""
    targets = target_names(preset, target_modules)
    gen = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        p.requires_grad_(False)
    adapted = []
    for name, mod in list(model.named_modules()):
        if not isinstance(mod, nn.Linear) or not any(name == t or name.endswith("." + t) for t in targets):
            continue
        parent = model
        parts = name.split(".")
        for part in parts[:-1]:
            parent = getattr(parent, part)
        setattr(parent, parts[-1], LoraLinear(mod.weight.data, mod.bias.data if mod.bias is not None else None, rank,
                                              alpha, dropout, nf4, rslora, gen))
        adapted.append(name)
    if not adapted:
        raise ValueError(f"no linear layer matches the targets {list(targets)}")
    return adapted


def adapter_state(model: nn.Module) -> Dict[str, torch.Tensor]:
    """PEFT names: ``base_model.model.<module>.lora_A.weight`` / ``lora_B.weight``."""
    out = {}
    for name, mod in model.named_modules():
        if isinstance(mod, LoraLinear):
            out[f"base_model.model.{name}.lora_A.weight"] = mod.lora_A.detach().float().cpu()
            out[f"base_model.model.{name}.lora_B.weight"] = mod.lora_B.detach().float().cpu()
    return out


def save_adapter(model: nn.Module, path: str, rank: int, alpha: float, targets: Iterable[str], rslora: bool = False,
                 base_model: str = "", extra: Optional[dict] = None) -> None:
    os.makedirs(path, exist_ok=True)
    ST.save_file(adapter_state(model), os.path.join(path, "adapter_model.safetensors"))
    cfg = {"peft_type": "LORA", "r": int(rank), "lora_alpha": float(alpha), "use_rslora": bool(rslora),
           "target_modules": sorted(set(t.rsplit(".", 1)[-1] for t in targets)), "bias": "none",
           "fan_in_fan_out": False, "base_model_name_or_path": base_model}
    cfg.update(extra or {})
    with open(os.path.join(path, "adapter_config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)


def load_adapter(model: nn.Module, path: str) -> int:
    """Copy a saved adapter's factors into the model's :class:`LoraLinear` modules; returns how many were set."""
    sd = ST.load_file(os.path.join(path, "adapter_model.safetensors"))
    n = 0
    for name, mod in model.named_modules():
        if isinstance(mod, LoraLinear):
            a, b = sd.get(f"base_model.model.{name}.lora_A.weight"), sd.get(f"base_model.model.{name}.lora_B.weight")
            if a is None or b is None:
                raise KeyError(f"{path}: no factors for {name}")
            with torch.no_grad():
                mod.lora_A.copy_(a)
                mod.lora_B.copy_(b)
            n += 1
    return n
