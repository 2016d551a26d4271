"""Low-rank adapters (PEFT layout) merged into a checkpoint at load time.

An adapter directory holds ``adapter_config.json`` (``r``, ``lora_alpha``, optionally ``use_rslora``, ``target_modules``,
``modules_to_save``) and ``adapter_model.safetensors`` with, per adapted linear ``<module>``,
``base_model.model.<module>.lora_A.weight`` [r, in] and ``...lora_B.weight`` [out, r].  Serving never keeps the two
factors apart: ``W <- W + scale * B @ A`` with ``scale = lora_alpha / r`` (``lora_alpha / sqrt(r)`` for rank-stabilised
adapters) is applied to the state dict before the weights are packed for the kernels, so an adapted model costs
exactly what its base costs.

The reference does this for the retrieval adapter of its Jina v5 embedder
(zig/pkg/inference/src/architectures/session_factory.zig:3620-3710, ``adapters/retrieval/`` below the model
directory; merge in zig/pkg/inference/src/ops/gpu_hosted_store.zig:105-160) and its ``pull`` fetches adapter artifacts
wherever a repository has them (zig/pkg/inference/src/registry/download.zig:586-610).  Here any checkpoint takes
an adapter: one lying in the model directory itself, or a named one under ``adapters/<name>/``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Tuple

import torch

from . import safetensors_io as ST

DEFAULT_ADAPTER = "retrieval"


def find_adapter(model_dir: str, name: Optional[str] = None) -> Optional[str]:
    """Directory of the adapter to apply: ``adapters/<name>`` when a name is given (error when absent), else an
    adapter in the model directory itself, else ``adapters/retrieval`` when there is one."""
    def complete(d: str) -> bool:
        have_c = os.path.exists(os.path.join(d, "adapter_config.json"))
        have_w = os.path.exists(os.path.join(d, "adapter_model.safetensors"))
        if have_c != have_w:
            raise ValueError(f"{d}: an adapter needs both adapter_config.json and adapter_model.safetensors")
        return have_c

    if name:
        d = os.path.join(model_dir, "adapters", name)
        if not complete(d):
            raise FileNotFoundError(f"{model_dir}: no adapter named {name!r}")
        return d
    for d in (model_dir, os.path.join(model_dir, "adapters", DEFAULT_ADAPTER)):
        if complete(d):
            return d
    return None


def adapter_scale(config: dict) -> float:
    r = int(config.get("r") or 0)
    if r <= 0:
        raise ValueError("adapter_config.json: rank r must be positive")
    alpha = float(config.get("lora_alpha") if config.get("lora_alpha") is not None else r)
    return alpha / math.sqrt(r) if config.get("use_rslora") else alpha / r


def _module_of(key: str) -> Tuple[Optional[str], Optional[str]]:
    """``base_model.model.<module>.lora_A[.<adapter>].weight`` -> (module, "A" | "B")."""
    for tag, which in ((".lora_A", "A"), (".lora_B", "B")):
        i = key.find(tag)
        if i >= 0 and key.endswith(".weight"):
            mod = key[:i]
            for prefix in ("base_model.model.", "base_model."):
                if mod.startswith(prefix):
                    mod = mod[len(prefix):]
                    break
            return mod, which
    return None, None


def _resolve(sd: Dict[str, torch.Tensor], module: str) -> Optional[str]:
    """The state-dict key of ``<module>.weight``, allowing for a prefix one side has and the other lacks
    (``model.`` / ``bert.`` / ...)."""
    want = module + ".weight"
    if want in sd:
        return want
    hits = [k for k in sd if k.endswith("." + want) or want.endswith("." + k)]
    return hits[0] if len(hits) == 1 else None


def merge_lora(sd: Dict[str, torch.Tensor], adapter_sd: Dict[str, torch.Tensor], config: dict) -> List[str]:
    """Adds ``scale * B @ A`` to every adapted weight of ``sd`` (in place, in fp32, cast back to the weight's dtype) and
    replaces ``modules_to_save`` tensors by the adapter's copies.  Returns the names of the merged weights; an adapted
    module that the checkpoint does not have is an error."""
    scale = adapter_scale(config)
    pairs: Dict[str, Dict[str, torch.Tensor]] = {}
    saved: Dict[str, torch.Tensor] = {}
    for key, t in adapter_sd.items():
        mod, which = _module_of(key)
        if mod is not None:
            pairs.setdefault(mod, {})[which] = t
        elif ".modules_to_save." in key:                     # a fully trained copy of a module (e.g. a new head)
            plain = key.replace("base_model.model.", "", 1)
            head, tail = plain.split(".modules_to_save.", 1)
            saved[head + "." + tail.split(".", 1)[1]] = t
    merged = []
    for mod, ab in sorted(pairs.items()):
        if "A" not in ab or "B" not in ab:
            raise ValueError(f"adapter: {mod} has only one of lora_A / lora_B")
        key = _resolve(sd, mod)
        if key is None:
            raise KeyError(f"adapter targets {mod}, which the checkpoint does not have")
        w = sd[key]
        a, b = ab["A"].float(), ab["B"].float()
        if config.get("fan_in_fan_out"):
            delta = (b @ a).t()
        else:
            delta = b @ a
        if delta.shape != w.shape:
            raise ValueError(f"adapter: {mod} is {tuple(w.shape)}, its factors give {tuple(delta.shape)}")
        sd[key] = (w.float() + scale * delta).to(w.dtype)
        merged.append(key)
    for name, t in saved.items():
        key = name if name in sd else _resolve(sd, name.rsplit(".", 1)[0]) if name.endswith(".weight") else None
        if key is not None:
            sd[key] = t.to(sd[key].dtype)
            merged.append(key)
    return merged


def apply_adapter(sd: Dict[str, torch.Tensor], model_dir: str, name: Optional[str] = None) -> Optional[dict]:
    """Merge the model directory's adapter (see :func:`find_adapter`) into ``sd``.  Returns
    ``{"path", "rank", "scale", "merged"}`` or None when there is no adapter."""
    d = find_adapter(model_dir, name)
    if d is None:
        return None
    with open(os.path.join(d, "adapter_config.json"), encoding="utf-8") as f:
        config = json.load(f)
    merged = merge_lora(sd, ST.load_file(os.path.join(d, "adapter_model.safetensors")), config)
    return {"path": d, "rank": int(config["r"]), "scale": adapter_scale(config), "merged": len(merged)}
