"""Host-side runtime (C++): KV block allocator and step scheduler.  No GPU needed."""
import numpy as np
import pytest

from antfly_b200.runtime.kv_cache import BlockAllocator, KvOutOfBlocks
from antfly_b200.runtime.scheduler import QueueFull, SchedulerPolicy, StepScheduler


def test_block_table_append_truncate_detach():
    a = BlockAllocator(num_blocks=8, page=16)
    a.attach(1)
    slots = a.append(1, 20)
    assert len(slots) == 20 and a.length(1) == 20
    bt = a.block_table(1)
    assert len(bt) == 2 and list(slots[:16]) == [bt[0] * 16 + i for i in range(16)]
    assert a.free_blocks == 6
    a.truncate(1, 16)  # rollback: second block freed
    assert a.free_blocks == 7 and a.length(1) == 16
    a.truncate(1, 3)
    assert a.free_blocks == 7 and len(a.block_table(1)) == 1
    a.detach(1)
    assert a.free_blocks == 8
    st = a.stats()
    assert st["acquired"] == st["released"] == 2


def test_append_is_all_or_nothing_when_pool_is_exhausted():
    a = BlockAllocator(num_blocks=2, page=16)
    a.attach(1)
    a.append(1, 30)
    a.attach(2)
    with pytest.raises(KvOutOfBlocks):
        a.append(2, 17)
    assert a.length(2) == 0 and a.free_blocks == 0
    with pytest.raises(KvOutOfBlocks):
        a.append(1, 3)
    assert a.length(1) == 30
    a.append(1, 2)
    assert a.stats()["oom"] == 2


def test_shared_prefix_refcounts_and_copy_on_write():
    a = BlockAllocator(num_blocks=8, page=16)
    a.attach(1)
    a.append(1, 40)  # blocks: 2 full + 1 partial (8 tokens)
    parent = a.block_table(1)
    a.attach_shared(2, 1, 40)
    child = a.block_table(2)
    assert list(child[:2]) == list(parent[:2]) and child[2] != parent[2]
    assert a.refcount(int(parent[0])) == 2 and a.refcount(int(parent[2])) == 1
    src, dst = a.take_cow()
    assert list(src) == [parent[2]] and list(dst) == [child[2]]
    a.attach_shared(3, 1, 32)  # exact block boundary: nothing to copy
    assert len(a.take_cow()[0]) == 0 and a.refcount(int(parent[1])) == 3
    a.detach(1)
    assert a.refcount(int(parent[0])) == 2  # still held by the children
    a.detach(2); a.detach(3)
    assert a.free_blocks == 8


def test_sliding_window_trim_releases_only_whole_old_tiles():
    a = BlockAllocator(num_blocks=64, page=16)
    a.attach(1)
    a.append(1, 300)
    assert a.trim_window(1, 100) == (300 - 100) // 64 * 64 // 16
    assert a.length(1) == 300
    a.append(1, 100)
    assert a.trim_window(1, 100) == 4


def test_truncate_cannot_cut_into_blocks_the_window_released():
    """After the sliding window released old blocks, a rollback may only go back to a token whose block still
    exists (anything else would append into a block that is gone); a full reset is allowed."""
    a = BlockAllocator(num_blocks=64, page=16)
    a.attach(1)
    a.append(1, 300)
    assert a.trim_window(1, 100) == 12                   # blocks of tokens 0..191 released
    with pytest.raises(KeyError):
        a.truncate(1, 150)
    a.truncate(1, 250)                                   # speculative-decoding style rollback: fine
    slots = a.append(1, 5)
    assert a.length(1) == 255 and (slots >= 0).all()
    a.truncate(1, 0)
    slots = a.append(1, 20)
    assert a.length(1) == 20 and (slots >= 0).all() and a.free_blocks == 62


def test_append_batch_matches_single_appends():
    a = BlockAllocator(num_blocks=32, page=16)
    for s in (1, 2, 3):
        a.attach(s)
        a.append(s, 15 + s)
    tables = np.zeros((3, 4), dtype=np.int32)
    slots, lens = a.append_batch(np.array([1, 2, 3]), np.array([1, 1, 1], dtype=np.int32), 4, tables)
    assert list(lens) == [17, 18, 19]
    for i, s in enumerate((1, 2, 3)):
        bt = a.block_table(s)
        assert list(tables[i, : len(bt)]) == list(bt)
        pos = lens[i] - 1
        assert slots[i] == bt[pos // 16] * 16 + pos % 16


def _drain(s, items, finish_after=None):
    toks, fin = [], []
    for it in items:
        toks.append(1 if it.mode == "decode" else 1)
        fin.append(False)
    s.complete_step(items, toks, fin)


def test_scheduler_decode_first_budgets_and_leader_rule():
    s = StepScheduler(SchedulerPolicy(max_step_items=4, max_step_query_tokens=64, prefill_chunk=32, min_chunk=8))
    s.admit(1, 100, 10)  # leader: prompt bigger than a chunk
    items = s.claim_step()
    assert [(i.request_id, i.mode, i.q_len, i.kv_before) for i in items] == [(1, "prefill", 32, 0)]
    _drain(s, items)
    s.admit(2, 5, 10)
    items = s.claim_step()
    # request 1 continues (32 more), request 2's whole prompt fits the remaining 32-token budget
    assert [(i.request_id, i.q_len) for i in items] == [(1, 32), (2, 5)]
    _drain(s, items)
    items = s.claim_step()
    # request 2 is decoding now and goes first; request 1 continues its prefill behind it
    assert items[0].request_id == 2 and items[0].mode == "decode" and items[0].kv_before == 5
    assert items[1].request_id == 1 and items[1].kv_before == 64
    _drain(s, items)
    st = s.stats()
    assert st["step_batches_total"] == 3 and st["step_singleton_batches_total"] == 1


def test_scheduler_streak_fairness_and_fail_rollback():
    s = StepScheduler(SchedulerPolicy(max_step_items=1, max_step_query_tokens=512, prefill_chunk=256, decode_streak=2))
    s.admit(1, 4, 100)
    _drain(s, s.claim_step())  # prefill of 1 completes -> decoding
    s.admit(2, 4, 100)
    modes = []
    for _ in range(4):
        items = s.claim_step()
        modes.append((items[0].request_id, items[0].mode))
        _drain(s, items)
    # only one item fits per step: two decode-only steps, then the waiting prefill gets its turn
    assert modes[:3] == [(1, "decode"), (1, "decode"), (2, "prefill")]
    items = s.claim_step()
    snap = s.snapshot()
    assert snap["in_flight"] == 1
    with pytest.raises(RuntimeError):
        s.claim_step()
    s.fail_step()
    assert s.snapshot()["in_flight"] == 0 and s.stats()["failed_steps_total"] == 1
    again = s.claim_step()
    assert [(i.request_id, i.q_len, i.kv_before) for i in again] == [(i.request_id, i.q_len, i.kv_before) for i in items]


def test_scheduler_queue_full_finish_and_kv_budget():
    s = StepScheduler(SchedulerPolicy(max_step_items=8, max_step_query_tokens=512, max_queue=2, max_kv_blocks=3,
                                      page=16))
    s.admit(1, 40, 2)
    s.admit(2, 40, 2)
    with pytest.raises(QueueFull):
        s.admit(3, 10, 2)
    items = s.claim_step()
    # leader needs 3 blocks (exempt); the second request's 3 blocks exceed the budget and are skipped
    assert [i.request_id for i in items] == [1]
    assert s.stats()["step_kv_block_skips_total"] == 1
    s.complete_step(items, [1], [False])
    items = s.claim_step()
    s.complete_step(items, [1] * len(items), [False] * len(items))  # request 1 reaches max_new_tokens = 2
    assert s.snapshot()["decode"] + s.snapshot()["waiting"] + s.snapshot()["prefill"] == 1
    s.admit(3, 10, 2)  # room again
    assert s.cancel(3)
