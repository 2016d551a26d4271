"""Rank-failure detection and elastic recovery, all on the host.

Detection.  Every rank writes a heartbeat (a wall-clock timestamp) into a key/value store between steps; before
launching a step a rank checks its peers' heartbeats and refuses to launch kernels that would wait on a rank that
stopped beating (the device-side waits are bounded anyway and would report a timeout status instead of hanging).
A collective that raises (a short process-group timeout) is treated the same way.

Recovery.  The survivors agree on the next smaller tensor-parallel group (8 -> 4 -> 2 -> 1: the largest power of
two that the survivors can fill, lowest ranks first), tear the old process group down, form the new one under a new
epoch of the same store, re-shard the weights from the checkpoint for the new world size, and resume every
unfinished request by prefilling its prompt plus the tokens it had already produced.  Greedy decoding therefore
continues exactly where a fresh run of the smaller group, given the same prefix, would be.  Ranks that are alive
but not needed leave with ``members`` not containing them.

The store has to outlive any single rank of the group: ``ElasticGroup`` takes an existing store (a ``TCPStore``
hosted by the launcher or by a process that is not a rank).  Failures are only ever injected on the host: a rank
that raises, exits between steps or never joins.  The reference has no counterpart (single process; its
collectives are host copies, zig/pkg/inference/src/graph/collective_ops.zig:43-130).
"""
from __future__ import annotations

import datetime
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence


class HeartbeatMonitor:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, dead_after_s: float = 10.0,
                 prefix: str = "afb/hb/", members: Optional[Sequence[int]] = None):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.dead_after_s, self.prefix = interval_s, dead_after_s, prefix
        self.members = list(members) if members is not None else list(range(world))
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
        return [r for r in self.members if r != self.rank and now - self.last_seen(r) > self.dead_after_s]

    def survivors(self) -> List[int]:
        dead = set(self.dead_ranks())
        return [r for r in self.members if r not in dead]


def largest_power_of_two_group(ranks: List[int]) -> List[int]:
    """Survivors that form the next smaller tensor-parallel group (8 -> 4 -> 2 -> 1)."""
    n = 1
    while n * 2 <= len(ranks):
        n *= 2
    return sorted(ranks)[:n]


class GroupLost(RuntimeError):
    """This rank is alive but is not a member of the re-formed group."""


@dataclass
class ElasticGroup:
    """A tensor-parallel process group that can shrink.  ``uid`` is this process's permanent id (its rank in the
    first group); ``members`` are the uids of the current group in rank order."""
    store: object
    uid: int
    members: List[int]
    backend: str = "gloo"
    timeout_s: float = 20.0
    dead_after_s: float = 3.0
    epoch: int = 0
    monitor: HeartbeatMonitor = field(init=False)

    def __post_init__(self):
        self.monitor = HeartbeatMonitor(self.store, self.uid, len(self.members), dead_after_s=self.dead_after_s,
                                        members=self.members)
        # The heartbeat comes from a thread of its own: a step (or a weight reload) may take longer than the
        # death limit, and a rank that is merely busy must not look dead.  The thread dies with the process; a
        # process that is alive but stuck is caught by the process group's collective timeout instead.
        import threading

        self._stop = threading.Event()

        def beat_forever():
            while not self._stop.wait(max(0.05, self.dead_after_s / 5.0)):
                try:
                    self.store.set(f"{self.monitor.prefix}{self.uid}", repr(time.time()))
                except Exception:
                    return

        self._beater = threading.Thread(target=beat_forever, name="afb-heartbeat", daemon=True)
        self._beater.start()

    def close(self) -> None:
        self._stop.set()

    # -- current view --------------------------------------------------------------------------------------------
    @property
    def rank(self) -> int:
        return self.members.index(self.uid)

    @property
    def world(self) -> int:
        return len(self.members)

    def form(self) -> None:
        """(Re-)creates the process group of the current members under this epoch's key prefix."""
        import torch.distributed as dist

        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass
        self.monitor = HeartbeatMonitor(self.store, self.uid, self.world, dead_after_s=self.dead_after_s,
                                        members=self.members)
        self.monitor.beat()
        if self.world == 1:
            return
        sub = dist.PrefixStore(f"afb/epoch{self.epoch}/", self.store)
        dist.init_process_group(self.backend, store=sub, rank=self.rank, world_size=self.world,
                                timeout=datetime.timedelta(seconds=self.timeout_s))

    # -- failure handling ----------------------------------------------------------------------------------------
    def check(self) -> List[int]:
        """Heartbeat, then the uids of members that stopped beating (empty = healthy)."""
        self.monitor.beat()
        return self.monitor.dead_ranks()

    def regroup(self, settle_s: float = 0.0) -> List[int]:
        """Agrees with the other survivors on the next group and forms it.  The proposal of the first survivor to
        write wins (compare-and-set on the epoch's key), so every survivor adopts the same member list even if
        their views of who is dead differ for a moment.  Raises GroupLost on a survivor that is left out."""
        if settle_s > 0:
            time.sleep(settle_s)
        self.monitor.beat()
        proposal = largest_power_of_two_group(self.monitor.survivors())
        key = f"afb/regroup/{self.epoch + 1}"
        mine = ",".join(str(r) for r in proposal)
        won = self.store.compare_set(key, "", mine).decode()
        members = [int(x) for x in won.split(",")]
        self.epoch += 1
        if self.uid not in members:
            import torch.distributed as dist

            if dist.is_initialized():
                try:
                    dist.destroy_process_group()
                except Exception:
                    pass
            self.members = members
            raise GroupLost(f"rank {self.uid} is not part of the re-formed group {members}")
        self.members = members
        self.form()
        return members


def elastic_generate(group: ElasticGroup, build_engine: Callable[[int, int], object], prompts: Sequence[Sequence[int]],
                     params, before_step: Optional[Callable[[int, ElasticGroup], None]] = None,
                     max_regroups: int = 3) -> Dict[str, object]:
    """Greedy generation that survives the loss of ranks between steps.

    ``build_engine(tp_rank, tp_size)`` loads this rank's weight shard for that world size (from the checkpoint) and
    returns an ``LLMEngine`` whose model communicates over the CURRENT default process group.  ``before_step`` is a
    test hook called with the global step number (failure injection: a rank exits there, nothing in flight).
    Returns {"tokens": per-prompt token lists, "regroups": n, "world": final world size, "members": final uids}.
    """
    import copy

    import torch.distributed as dist

    done: List[List[int]] = [[] for _ in prompts]
    regroups, step_no = 0, 0
    engine = build_engine(group.rank, group.world)
    while True:
        todo = [i for i in range(len(prompts)) if len(done[i]) < params.max_tokens]
        if not todo:
            break
        # (re-)admit what is unfinished: prompt + the tokens already produced, fewer tokens left to make
        rids = {}
        for i in todo:
            sp = copy.copy(params)
            sp.max_tokens = params.max_tokens - len(done[i])
            rids[i] = engine.add_request(list(prompts[i]) + done[i], sp)
        taken = {i: 0 for i in todo}
        failed = False
        while any(not engine.reqs[r].finished for r in rids.values()):
            if before_step is not None:
                before_step(step_no, group)
            dead = group.check() if group.world > 1 else []
            if dead:
                failed = True
            else:
                try:
                    engine.step()
                except (RuntimeError, dist.DistBackendError) as e:  # a collective timed out or a peer vanished
                    if group.world == 1:
                        raise
                    failed = True
            if failed:
                break
            step_no += 1
            for i, r in rids.items():   # tokens count as accepted once a step completed on this rank
                out = engine.reqs[r].out
                done[i].extend(out[taken[i]:])
                taken[i] = len(out)
        if not failed:
            continue
        if regroups >= max_regroups:
            raise RuntimeError("too many regroups")
        regroups += 1
        # Survivors may have completed different numbers of steps (one saw the failure a step later): agree on the
        # shortest accepted prefix per prompt before resuming, through the long-lived store.
        group.regroup(settle_s=group.dead_after_s)
        done = _agree_on_prefix(group, done)
        engine = build_engine(group.rank, group.world)
    return {"tokens": done, "regroups": regroups, "world": group.world, "members": list(group.members)}


def _agree_on_prefix(group: ElasticGroup, done: List[List[int]]) -> List[List[int]]:
    """Every member publishes how many tokens it accepted per prompt; all truncate to the minimum."""
    key = f"afb/resume/{group.epoch}/"
    group.store.set(key + str(group.uid), ",".join(str(len(d)) for d in done))
    lens = [len(d) for d in done]
    for m in group.members:
        group.store.wait([key + str(m)], datetime.timedelta(seconds=group.timeout_s))
        theirs = [int(x) for x in group.store.get(key + str(m)).decode().split(",")]
        lens = [min(a, b) for a, b in zip(lens, theirs)]
    return [d[:n] for d, n in zip(done, lens)]
