"""Time-limited result cache for idempotent requests (embeddings of a text, scores of a query / document pair).

The reference's server keeps per-task result caches with a two-minute lifetime keyed by a hash of model and input
(go/pkg/termite/embedding_cache.go, reranking cache, ner_cache.go): repeated texts -- the same document re-embedded
by several index builders, the same query retried -- skip the model.  Entries are per input item, so a batch that
mixes seen and unseen texts only computes the unseen ones.
"""
from __future__ import annotations

import hashlib
import threading
import time
from collections import OrderedDict
from typing import Callable, Hashable, Optional


class ResultCache:
    def __init__(self, ttl_s: float = 120.0, max_entries: int = 65536, clock: Callable[[], float] = time.monotonic):
        self.ttl, self.max_entries, self._clock = ttl_s, max_entries, clock
        self._d: "OrderedDict[Hashable, tuple]" = OrderedDict()
        self._lock = threading.Lock()
        self.hits = self.misses = 0

    @staticmethod
    def key(*parts) -> str:
        h = hashlib.sha256()
        for p in parts:
            b = p if isinstance(p, bytes) else repr(p).encode("utf-8")
            h.update(len(b).to_bytes(8, "little"))
            h.update(b)
        return h.hexdigest()

    def get(self, key: Hashable):
        now = self._clock()
        with self._lock:
            item = self._d.get(key)
            if item is not None and now - item[0] <= self.ttl:
                self._d.move_to_end(key)
                self.hits += 1
                return item[1]
            if item is not None:
                del self._d[key]
            self.misses += 1
            return None

    def put(self, key: Hashable, value) -> None:
        if self.ttl <= 0 or self.max_entries <= 0:
            return
        now = self._clock()
        with self._lock:
            self._d[key] = (now, value)
            self._d.move_to_end(key)
            while len(self._d) > self.max_entries:
                self._d.popitem(last=False)
            # opportunistic expiry from the old end
            while self._d:
                k, (t, _v) = next(iter(self._d.items()))
                if now - t <= self.ttl:
                    break
                del self._d[k]

    def __len__(self) -> int:
        with self._lock:
            return len(self._d)
