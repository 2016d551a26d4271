"""Model check of the flag-free cross-GPU hand-off used by the fused tensor-parallel step.

The protocol (csrc/kernels/gemm_mxfp8.cu mode 4 + csrc/kernels/norms.cu, csrc/kernels/sampling.cu): every rank
stores its contribution into slot [rank] of EVERY rank's buffer; a consumer polls its own slots until none holds the
sentinel, uses the values, and puts the sentinel back.  Two buffers alternate between the collectives of a step and
a single buffer serves the arg-max merge at the end of the step.  Nothing but program order inside a rank and
the data itself synchronises the ranks.

This test runs the protocol as an interleaving simulation: ranks are coroutines whose every slot access is one
scheduling point, and a seeded random scheduler picks who moves next (including long stalls of single ranks).  Each
consumed value is checked to be exactly the contribution of the expected (step, collective, source): a value
overwritten before it was read, or a stale one read twice, fails the test.  It also shows the negative: with a
single buffer for consecutive collectives the same simulation does find a violation.
"""
import random

import pytest

SENTINEL = None


def _rank_program(rank, world, bufs, argmax_buf, steps, collectives, buffers_in_rotation, log):
    """Generator: yields at every shared-memory access."""
    for s in range(steps):
        for k in range(collectives):
            b = (s * collectives + k) % buffers_in_rotation
            # producer half (GEMM epilogue): one store per destination rank, in any order
            for dst in range(world):
                yield
                bufs[dst][b][rank] = (s, k, rank)
            # consumer half (norm kernel): poll own slots until all landed ...
            got = {}
            while len(got) < world:
                for src in range(world):
                    if src in got:
                        continue
                    yield
                    v = bufs[rank][b][src]
                    if v is not SENTINEL:
                        got[src] = v
            for src in range(world):
                if got[src] != (s, k, src):
                    log.append((rank, s, k, src, got[src]))
            # ... then restore the sentinel
            for src in range(world):
                yield
                bufs[rank][b][src] = SENTINEL
        # arg-max merge: one buffer, same discipline
        for dst in range(world):
            yield
            argmax_buf[dst][rank] = ("tok", s, rank)
        got = {}
        while len(got) < world:
            for src in range(world):
                if src in got:
                    continue
                yield
                v = argmax_buf[rank][src]
                if v is not SENTINEL:
                    got[src] = v
        for src in range(world):
            if got[src] != ("tok", s, src):
                log.append((rank, s, "argmax", src, got[src]))
            yield
            argmax_buf[rank][src] = SENTINEL


def _simulate(world, seed, steps=3, collectives=4, buffers_in_rotation=2, max_moves=2_000_000):
    rng = random.Random(seed)
    bufs = [[[SENTINEL] * world for _ in range(buffers_in_rotation)] for _ in range(world)]
    argmax_buf = [[SENTINEL] * world for _ in range(world)]
    log = []
    progs = [_rank_program(r, world, bufs, argmax_buf, steps, collectives, buffers_in_rotation, log)
             for r in range(world)]
    alive = list(range(world))
    favourite, burst = None, 0
    moves = 0
    while alive and moves < max_moves:
        moves += 1
        if burst > 0 and favourite in alive:
            r, burst = favourite, burst - 1     # let one rank run far ahead (or leave the others far behind)
        else:
            r = rng.choice(alive)
            if rng.random() < 0.02:
                favourite, burst = r, rng.randint(50, 2000)
        try:
            next(progs[r])
        except StopIteration:
            alive.remove(r)
    assert not alive, "the simulation did not finish: a wait can never be satisfied (deadlock)"
    return log


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_two_alternating_buffers_are_enough(world):
    for seed in range(40):
        assert _simulate(world, seed) == []


def test_one_buffer_for_consecutive_collectives_is_not_enough():
    """The same schedule space does break a single shared buffer: a fast rank's next contribution lands before a
    slow rank has restored the sentinel, is wiped by that restore, and somebody then waits for ever (or a stale
    value is read).  Shows the simulation can see the hazard it is meant to rule out."""
    def broken(seed):
        try:
            return bool(_simulate(4, seed, buffers_in_rotation=1, max_moves=200_000))
        except AssertionError:
            return True

    assert any(broken(seed) for seed in range(40))


# ---------------------------------------------------------------------------------------------------------------
# Counter hand-off of the data-parallel embedding gather (csrc/kernels/pool.cu afb_pool_gather +
# afb_peer_counter_wait) and of the sharded top-k merge (csrc/kernels/index_ops.cu push / wait halves): producers
# store rows into slot [rank] of EVERY rank's buffer of the step's parity and bump that rank's arrival counter;
# the consumer polls its own counter (bounded) for the cumulative target, then reads.  Counters only grow.
# ---------------------------------------------------------------------------------------------------------------
from antfly_b200.parallel.dp_embed import GatherSchedule  # noqa: E402  (the schedule arithmetic under test)

TIMEOUT = "timeout"


def _counter_rank(rank, world, bufs, counters, steps, rows, n_parities, poll_budget, log, status, absent):
    sched = GatherSchedule(world)
    for s in range(steps):
        par, target = sched.next(rows)
        par %= n_parities
        if n_parities == 1:
            target = (s + 1) * world * rows
        if rank in absent:
            return  # a rank that never launches its step: pushes nothing, waits for nothing
        # producer CTAs: one row each, store then bump (release).  A rank whose status word already carries a
        # cross-GPU timeout pushes nothing more: its later rows must not complete a slower peer's OLDER target.
        for dst in range(world if not status[rank] else 0):
            for row in range(rows):
                yield
                bufs[dst][par][rank][row] = (s, rank, row)
                yield
                counters[dst][par] += 1
        polls = 0
        while counters[rank][par] - target < 0:   # consumer: bounded poll of the OWN counter
            yield
            polls += 1
            if status[rank] or polls > poll_budget:
                status[rank] = TIMEOUT            # sticky: later waits give up on their first poll
                break
        if status[rank]:
            continue                              # results of a timed-out step are not trusted by the host
        for src in range(world):                  # the reads of whatever the caller enqueues after the wait
            for row in range(rows):
                yield
                v = bufs[rank][par][src][row]
                if v != (s, src, row):
                    log.append((rank, s, src, row, v))


def _simulate_counters(world, seed, steps=5, rows=3, n_parities=2, poll_budget=10 ** 9, absent=(), max_moves=4_000_000):
    rng = random.Random(seed)
    bufs = [[[[None] * rows for _ in range(world)] for _ in range(n_parities)] for _ in range(world)]
    counters = [[0] * n_parities for _ in range(world)]
    log, status = [], [None] * world
    progs = [_counter_rank(r, world, bufs, counters, steps, rows, n_parities, poll_budget, log, status, set(absent))
             for r in range(world)]
    alive = list(range(world))
    favourite, burst, moves = None, 0, 0
    while alive and moves < max_moves:
        moves += 1
        if burst > 0 and favourite in alive:
            r, burst = favourite, burst - 1
        else:
            r = rng.choice(alive)
            if rng.random() < 0.02:
                favourite, burst = r, rng.randint(50, 3000)
        try:
            next(progs[r])
        except StopIteration:
            alive.remove(r)
    assert not alive, "the simulation did not finish (deadlock)"
    return log, status


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_counter_handoff_with_two_parities_never_reads_stale_or_overwritten_rows(world):
    for seed in range(25):
        log, status = _simulate_counters(world, seed)
        assert log == [] and status == [None] * world


def test_counter_handoff_with_one_buffer_is_not_enough():
    """A fast rank's rows of step s+1 land in the single buffer while a slow rank still reads step s."""
    assert any(_simulate_counters(4, seed, n_parities=1)[0] for seed in range(40))


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_a_rank_that_never_arrives_ends_in_timeout_status_not_deadlock(world):
    """The missing rank's rows never come: every other rank's first wait runs out of its budget, records the
    timeout, and all its later waits give up at once -- the programs terminate and nothing is consumed."""
    for seed in range(10):
        log, status = _simulate_counters(world, seed, poll_budget=500, absent=(world - 1,))
        assert log == []
        assert status[:world - 1] == [TIMEOUT] * (world - 1)


def test_gather_schedule_targets_are_cumulative_per_parity_and_wrap_like_int32():
    s = GatherSchedule(4)
    assert [s.next(10) for _ in range(4)] == [(0, 40), (1, 40), (0, 80), (1, 80)]
    s.pushed = [2 ** 31 - 8, 0]
    par, target = s.next(4)              # 2^31 + 8 wraps to a negative int32; the device compare is on the difference
    assert par == 0 and target == -(2 ** 31) + 8
