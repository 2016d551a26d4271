"""Rank-failure detection on the host.

Every rank writes a heartbeat (a wall-clock timestamp) into the process group's key/value store between steps;
before launching a step a rank checks its peers' heartbeats and refuses to launch kernels that would wait on a
rank that stopped beating (the device-side waits are bounded anyway and would report a timeout status instead of
hanging).  On a detected failure the survivors tear the group down and can re-form a smaller one
(8 -> 4 -> 2 -> 1).  Failures are only ever injected on the host: a rank that raises, exits or never joins.
"""
from __future__ import annotations

import time
from typing import List


class HeartbeatMonitor:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, dead_after_s: float = 10.0,
                 prefix: str = "afb/hb/"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.dead_after_s, self.prefix = interval_s, dead_after_s, prefix
        self._last = 0.0

    def beat(self, force: bool = True) -> None:
        now = time.time()
        if force or now - self._last >= self.interval_s:
            self.store.set(f"{self.prefix}{self.rank}", repr(now))
            self._last = now

    def last_seen(self, rank: int) -> float:
        try:
            if not self.store.check([f"{self.prefix}{rank}"]):
                return 0.0
            return float(self.store.get(f"{self.prefix}{rank}").decode())
        except Exception:
            return 0.0

    def dead_ranks(self) -> List[int]:
        now = time.time()
        return [r for r in range(self.world) if r != self.rank and now - self.last_seen(r) > self.dead_after_s]

    def survivors(self) -> List[int]:
        dead = set(self.dead_ranks())
        return [r for r in range(self.world) if r not in dead]


def largest_power_of_two_group(ranks: List[int]) -> List[int]:
    """Survivors that form the next smaller tensor-parallel group (8 -> 4 -> 2 -> 1)."""
    n = 1
    while n * 2 <= len(ranks):
        n *= 2
    return sorted(ranks)[:n]
