"""Server configuration: one schema filled from a YAML / JSON file, environment variables and CLI flags.

Fields and defaults follow the reference's inference ``Config`` object (specs/openapi/inference/api.yaml:2634-2805):
``api_url``, ``models_dir``, ``keep_alive``, ``max_loaded_models``, ``pool_size``, ``backend_priority``,
``max_concurrent_requests``, ``max_queue_size``, ``request_timeout``, ``preload``, ``max_memory_mb``,
``model_strategies``, ``allow_downloads``, ``log``.  Durations use the Go notation the reference documents
("5m", "1h30m", "30s", "250ms", "0").  Precedence: defaults < file < environment < explicit overrides.  Environment
names are ``ANTFLY_INFERENCE_<FIELD>`` (the older ``TERMITE_<FIELD>`` is read too), lists comma-separated.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field, fields
from typing import Dict, List, Mapping, Optional

_UNITS = {"ns": 1e-9, "us": 1e-6, "µs": 1e-6, "ms": 1e-3, "s": 1.0, "m": 60.0, "h": 3600.0}
_DUR = re.compile(r"(\d+(?:\.\d+)?)(ns|us|µs|ms|s|m|h)")


def parse_duration(text) -> float:
    """Go-style duration -> seconds ("0" or 0 -> 0.0; a bare number counts as seconds)."""
    if isinstance(text, (int, float)):
        return float(text)
    s = str(text).strip()
    if s in ("", "0"):
        return 0.0
    try:
        return float(s)
    except ValueError:
        pass
    pos, total = 0, 0.0
    for m in _DUR.finditer(s):
        if m.start() != pos:
            raise ValueError(f"bad duration {text!r}")
        total += float(m.group(1)) * _UNITS[m.group(2)]
        pos = m.end()
    if pos != len(s):
        raise ValueError(f"bad duration {text!r}")
    return total


@dataclass
class LogConfig:
    level: str = "info"
    style: str = "text"            # text | json


@dataclass
class Config:
    api_url: str = "http://localhost:8080"
    api_key: Optional[str] = None
    models_dir: Optional[str] = None
    keep_alive: str = "5m"
    max_loaded_models: int = 0
    pool_size: int = 1
    backend_priority: List[str] = field(default_factory=lambda: ["cuda", "native"])
    max_concurrent_requests: int = 0
    max_queue_size: int = 0
    request_timeout: str = "0"
    preload: List[str] = field(default_factory=list)
    max_memory_mb: int = 0
    model_strategies: Dict[str, str] = field(default_factory=dict)
    allow_downloads: bool = False
    content_security: Dict[str, object] = field(default_factory=dict)
    data_dir: Optional[str] = None      # tables are kept here across restarts (none: in memory only)
    log: LogConfig = field(default_factory=LogConfig)

    # -- derived -------------------------------------------------------------------------------------------
    @property
    def keep_alive_s(self) -> float:
        return parse_duration(self.keep_alive)

    @property
    def request_timeout_s(self) -> float:
        return parse_duration(self.request_timeout)

    @property
    def host_port(self):
        m = re.match(r"^(?:\w+://)?(\[[^\]]+\]|[^:/\[\]]+)(?::(\d+))?", self.api_url)
        if not m:
            raise ValueError(f"bad api_url {self.api_url!r}")
        return m.group(1).strip("[]"), int(m.group(2) or 8080)

    def device(self) -> str:
        """First usable entry of backend_priority: ``cuda`` (or ``<backend>:cuda``) needs a GPU, ``native`` /
        ``<backend>:cpu`` is the CPU path; backends this build does not have (onnx, xla, metal, mlx) are skipped."""
        import torch

        for entry in self.backend_priority:
            backend, _, dev = entry.partition(":")
            if backend not in ("cuda", "native"):
                continue
            if backend == "cuda" or dev == "cuda":
                if torch.cuda.is_available():
                    return "cuda"
                continue
            return "cpu"
        return "cuda" if torch.cuda.is_available() else "cpu"

    def strategy(self, model: str) -> str:
        """eager | lazy | bounded for a model (per-model override, else from keep_alive)."""
        s = self.model_strategies.get(model)
        if s:
            if s not in ("eager", "lazy", "bounded"):
                raise ValueError(f"unknown loading strategy {s!r} for {model}")
            return s
        return "eager" if self.keep_alive_s == 0 else "lazy"

    def validate(self) -> "Config":
        parse_duration(self.keep_alive), parse_duration(self.request_timeout), self.host_port
        for k in ("max_loaded_models", "pool_size", "max_concurrent_requests", "max_queue_size", "max_memory_mb"):
            if int(getattr(self, k)) < 0:
                raise ValueError(f"{k} must be >= 0")
        if self.pool_size < 1:
            raise ValueError("pool_size must be >= 1")
        for m in self.model_strategies:
            self.strategy(m)
        from .api.content import ContentSecurity

        ContentSecurity.from_dict(self.content_security, self.allow_downloads)      # raises on bad values
        return self

    def to_dict(self) -> dict:
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["log"] = {"level": self.log.level, "style": self.log.style}
        return d


def _coerce(name: str, value, current):
    if isinstance(current, bool):
        return value if isinstance(value, bool) else str(value).strip().lower() in ("1", "true", "yes", "on")
    if isinstance(current, int) and not isinstance(current, bool):
        return int(value)
    if isinstance(current, list):
        return [s.strip() for s in value.split(",") if s.strip()] if isinstance(value, str) else list(value)
    if isinstance(current, dict):
        if isinstance(value, str):
            return dict(kv.split("=", 1) for kv in value.split(",") if "=" in kv)
        return dict(value)
    if isinstance(current, LogConfig):
        if isinstance(value, Mapping):
            return LogConfig(**{k: v for k, v in value.items() if k in ("level", "style")})
        return LogConfig(level=str(value))
    return value if value is None else str(value)


def load_config(path: Optional[str] = None, env: Optional[Mapping[str, str]] = None, **overrides) -> Config:
    cfg = Config()
    known = {f.name for f in fields(Config)}

    def apply(src: Mapping, where: str, strict: bool) -> None:
        for k, v in src.items():
            if k not in known:
                if strict:
                    raise ValueError(f"{where}: unknown configuration key {k!r}")
                continue
            if v is not None:
                setattr(cfg, k, _coerce(k, v, getattr(cfg, k)))

    if path:
        with open(path) as f:
            text = f.read()
        if path.endswith(".json"):
            data = json.loads(text)
        else:
            import yaml

            data = yaml.safe_load(text) or {}
        if not isinstance(data, Mapping):
            raise ValueError(f"{path}: expected a mapping at the top level")
        apply(data, path, strict=True)
    env = os.environ if env is None else env
    from_env = {}
    for name in known:
        for prefix in ("TERMITE_", "ANTFLY_INFERENCE_"):
            if prefix + name.upper() in env:
                from_env[name] = env[prefix + name.upper()]
    apply(from_env, "environment", strict=False)
    apply({k: v for k, v in overrides.items()}, "overrides", strict=True)
    return cfg.validate()
