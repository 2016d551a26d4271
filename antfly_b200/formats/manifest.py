"""Model-directory resolution and manifest detection.

Lookup order and task directory names follow the reference (zig/pkg/inference/src/server/server.zig:995-1040,
src/main.zig:29-31): an absolute path, ``models_dir/<name>``, then ``models_dir/<task>/<name>``; the default models
directory is ``$ANTFLY_INFERENCE_MODELS_DIR`` or ``~/.antfly/inference/models``.  Files recognised in a model
directory are the ones of zig/pkg/inference/src/models/manifest.zig:123-200.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

TASK_DIRS = ("embedders", "rerankers", "generators", "chunkers", "recognizers", "rewriters", "classifiers",
             "readers", "transcribers")


def default_models_dir() -> str:
    return os.environ.get("ANTFLY_INFERENCE_MODELS_DIR") or os.path.expanduser("~/.antfly/inference/models")


def resolve_model_path(name: str, models_dir: Optional[str] = None, task: Optional[str] = None) -> Optional[str]:
    if os.path.isabs(name) and os.path.isdir(name):
        return name
    root = models_dir or default_models_dir()
    cands = [os.path.join(root, name)]
    for t in ([task] if task else []) + [t for t in TASK_DIRS if t != task]:
        cands.append(os.path.join(root, t, name))
    for c in cands:
        if os.path.isdir(c):
            return c
    # registry form: "[hf:]owner/name[:variant]" names the directory a pull wrote, models_dir/owner/name
    bare = name[3:] if name.startswith("hf:") else name
    bare = bare.split(":", 1)[0]
    if bare != name and "/" in bare:
        return resolve_model_path(bare, models_dir, task)
    return None


@dataclass
class Manifest:
    path: str
    weights: Optional[str] = None          # "safetensors" | "gguf" | "onnx"
    weight_files: List[str] = field(default_factory=list)
    config: Dict = field(default_factory=dict)
    has_tokenizer_json: bool = False
    has_sentencepiece: bool = False
    chat_template: Optional[str] = None
    tasks: List[str] = field(default_factory=list)
    capabilities: List[str] = field(default_factory=list)

    @property
    def model_type(self) -> str:
        """embedder / reranker / generator, from the manifest tasks, else from config.json."""
        for t in self.tasks:
            if t in ("embedder", "reranker", "generator", "chunker"):
                return t
        arch = " ".join(self.config.get("architectures") or [])
        if "ForSequenceClassification" in arch:
            return "reranker"
        if "CausalLM" in arch or self.config.get("model_type") in ("llama", "mistral", "qwen2", "qwen3", "gemma", "phi3", "mixtral", "qwen2_moe", "qwen3_moe", "gpt2",
                                                                     "gpt_neox", "opt", "gptj", "phi"):
            return "generator"
        return "embedder"


def read_manifest(model_dir: str) -> Manifest:
    m = Manifest(model_dir)
    files = sorted(os.listdir(model_dir))
    st = [f for f in files if f.endswith(".safetensors")]
    gg = [f for f in files if f.endswith(".gguf")]
    ox = [f for f in files if f.endswith(".onnx")]
    if st:
        m.weights, m.weight_files = "safetensors", st
    elif gg:
        m.weights, m.weight_files = "gguf", gg
    elif ox:
        m.weights, m.weight_files = "onnx", ox
    for name, attr in (("config.json", "config"),):
        p = os.path.join(model_dir, name)
        if os.path.exists(p):
            with open(p, encoding="utf-8") as f:
                setattr(m, attr, json.load(f))
    m.has_tokenizer_json = "tokenizer.json" in files
    m.has_sentencepiece = "tokenizer.model" in files
    ct = os.path.join(model_dir, "chat_template.jinja")
    if os.path.exists(ct):
        with open(ct, encoding="utf-8") as f:
            m.chat_template = f.read()
    else:
        tc = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(tc):
            with open(tc, encoding="utf-8") as f:
                m.chat_template = json.load(f).get("chat_template")
    mm = os.path.join(model_dir, "model_manifest.json")
    if os.path.exists(mm):
        with open(mm, encoding="utf-8") as f:
            d = json.load(f)
        m.tasks = list(d.get("tasks", [d["task"]] if "task" in d else []))
        m.capabilities = list(d.get("capabilities", []))
    return m
