"""Structured logging: one line per event, as ``key=value`` text or as JSON, chosen by the server configuration
(``log: {level, style}``).  Fields the reference's loggers carry on every request line -- endpoint, status, duration,
work units, model -- are passed as keyword arguments (zig/lib/structlog text / json formatters, termite's zap
request logs)."""
from __future__ import annotations

import json
import logging
import sys
import time
from typing import Optional

_RESERVED = set(logging.LogRecord("", 0, "", 0, "", None, None).__dict__) | {"message", "asctime"}


class _Formatter(logging.Formatter):
    def __init__(self, style: str):
        super().__init__()
        self.json = style == "json"

    def format(self, record: logging.LogRecord) -> str:
        fields = {k: v for k, v in record.__dict__.items() if k not in _RESERVED}
        ts = time.strftime("%Y-%m-%dT%H:%M:%S", time.gmtime(record.created)) + ".%03dZ" % (record.msecs,)
        if self.json:
            body = {"ts": ts, "level": record.levelname.lower(), "logger": record.name, "msg": record.getMessage()}
            body.update(fields)
            if record.exc_info:
                body["error"] = self.formatException(record.exc_info)
            return json.dumps(body, default=str)
        kv = " ".join(f"{k}={json.dumps(v, default=str) if isinstance(v, str) and ' ' in v else v}"
                      for k, v in fields.items())
        line = f"{ts} {record.levelname.lower():5s} {record.name}: {record.getMessage()}" + (f" {kv}" if kv else "")
        if record.exc_info:
            line += "\n" + self.formatException(record.exc_info)
        return line


def setup(level: str = "info", style: str = "text", stream=None) -> logging.Logger:
    """Configure the ``antfly_b200`` logger tree (idempotent) and return its root."""
    lg = logging.getLogger("antfly_b200")
    lg.setLevel(getattr(logging, str(level).upper(), logging.INFO))
    for h in list(lg.handlers):
        lg.removeHandler(h)
    h = logging.StreamHandler(stream or sys.stderr)
    h.setFormatter(_Formatter(style))
    lg.addHandler(h)
    lg.propagate = False
    return lg


def get(name: Optional[str] = None) -> logging.Logger:
    return logging.getLogger("antfly_b200" + (f".{name}" if name else ""))


def event(logger: logging.Logger, level: int, msg: str, **fields) -> None:
    logger.log(level, msg, extra=fields)
