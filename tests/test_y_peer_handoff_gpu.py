"""Counter hand-offs of the data-parallel embedding gather and of the sharded top-k merge, on ONE GPU.

Positive cases emulate the ranks one after another on the same device: every "rank's" push kernel stores into all
ranks' buffers (all of them local here) and bumps their counters; the consumers are launched after all pushes, so
no kernel ever waits for a kernel that is launched later.  Negative cases make a wait run out on purpose (a
counter that nothing bumps) and check that the kernel returns, the status word carries the peer-timeout code and
later waits give up at once; nothing faults or hangs."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

needs_gpu = pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
c_int = ctypes.c_int


def _ptrs(addrs):
    return (ctypes.c_void_p * len(addrs))(*addrs)


@needs_gpu
def test_pool_gather_pushes_rows_and_counter_wait_sees_them():
    from antfly_b200 import _native as N
    from antfly_b200.ops import dense as Dn
    from antfly_b200.ops.dense import POOL_MODES
    from antfly_b200.parallel.dp_embed import GatherSchedule

    dev = torch.device("cuda")
    world, B, H = 3, 5, 256
    n = world * B * H
    # one "symmetric buffer" per emulated rank: [2 parities][world * B, H] floats + 2 counters
    bufs = [torch.zeros(2 * n + 64, dtype=torch.float32, device=dev) for _ in range(world)]
    scheds = [GatherSchedule(world) for _ in range(world)]
    torch.manual_seed(0)
    for step in range(3):
        lens = torch.randint(1, 9, (world, B))
        hs, expect, targets = [], [], []
        for r in range(world):
            L = lens[r].to(dev).int()
            starts = (torch.cumsum(L, 0) - L).int()
            h = torch.randn(int(L.sum()), H, device=dev).bfloat16()
            hs.append((h, starts, L))
            # fp32 reference of the same op (the CPU path of the wrapper)
            expect.append(Dn.pool(h.cpu(), starts.cpu(), L.cpu(), mode="mean", normalize=True).to(dev))
        for r in range(world):
            par, target = scheds[r].next(B)
            targets.append((par, target))
            h, starts, L = hs[r]
            out = torch.empty((B, H), dtype=torch.float32, device=dev)
            peer_out = _ptrs([b.data_ptr() + 4 * n * par for b in bufs])
            peer_ready = _ptrs([b.data_ptr() + 4 * (2 * n + par) for b in bufs])
            rc = N.cuda().afb_pool_gather(N.ptr(h), N.ptr(starts), N.ptr(L), None, N.ptr(out), c_int(B), c_int(H),
                                          c_int(POOL_MODES["mean"]), c_int(1), peer_out, peer_ready, c_int(world),
                                          c_int(r * B), N.stream_ptr())
            N.check(rc, "afb_pool_gather")
            torch.testing.assert_close(out, expect[r], atol=2e-5, rtol=1e-4)
        want = torch.cat(expect, 0)
        for r in range(world):
            par, target = targets[r]
            ready = bufs[r][2 * n + par: 2 * n + par + 1]
            N.check(N.cuda().afb_peer_counter_wait(N.ptr(ready), c_int(target), N.stream_ptr()), "wait")
            got = bufs[r][par * n: par * n + n].view(world * B, H)
            torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
            assert int(ready.view(torch.int32).item()) == target
    assert N.status() == 0


@needs_gpu
def test_select_push_and_merge_equal_a_plain_merge_and_carry_the_overflow_flag():
    from antfly_b200 import _native as N
    from antfly_b200.ops import index_ops as IX

    dev = torch.device("cuda")
    world, nq, k, cap = 4, 7, 5, 64
    slot, per_par = nq * k, world * (2 * nq * k + nq)
    bufs = [torch.zeros(2 * per_par + 64, dtype=torch.int32, device=dev) for _ in range(world)]
    torch.manual_seed(1)
    for step, overflow_rank in enumerate([None, 2, None]):
        par = step & 1
        target = (step // 2 + 1) * world * nq
        locals_ = []
        for r in range(world):
            vals = torch.rand(nq, cap, device=dev)
            ids = (torch.arange(nq * cap, device=dev).view(nq, cap) + 100000 * r).int()
            counts = torch.full((nq,), cap, dtype=torch.int32, device=dev)
            if overflow_rank == r:
                counts[3] = cap + 9      # the producer reports more candidates than its buffer holds
            sticky = torch.zeros(1, dtype=torch.int32, device=dev)
            P = ctypes.c_void_p * world
            push = (P(*[b.data_ptr() + 4 * (par * per_par + r * slot) for b in bufs]),
                    P(*[b.data_ptr() + 4 * (par * per_par + world * slot + r * slot) for b in bufs]),
                    P(*[b.data_ptr() + 4 * (par * per_par + 2 * world * slot + r * nq) for b in bufs]),
                    P(*[b.data_ptr() + 4 * (2 * per_par + par) for b in bufs]))
            tv, ti, _, _ = IX.topk_select([(vals, ids, counts, cap)], nq, k, cap, overflow=sticky, push=push)
            locals_.append((tv, ti))
        ref_v, ref_i, _, _ = IX.topk_select([(v, i, None, k) for v, i in locals_], nq, k, world * k)
        for r in range(world):
            b = bufs[r]
            srcs, flags = [], []
            for s in range(world):
                o = par * per_par + s * slot
                srcs.append((b[o: o + slot].view(torch.float32).view(nq, k),
                             b[par * per_par + world * slot + s * slot: par * per_par + world * slot + (s + 1) * slot].view(nq, k),
                             None, k))
                f0 = par * per_par + 2 * world * slot + s * nq
                flags.append(b[f0: f0 + nq])
            ready = b[2 * per_par + par: 2 * per_par + par + 1]
            tv, ti, _, ovf = IX.topk_select(srcs, nq, k, world * k, want_threshold=False, wait=(ready, target),
                                            src_flags=flags)
            torch.testing.assert_close(tv, ref_v)
            assert torch.equal(ti, ref_i)
            assert int(ovf) == (1 if overflow_rank is not None else 0)
    assert N.status() == 0


@needs_gpu
def test_gather_and_merge_waits_expire_with_status_then_later_waits_and_pushes_stop():
    from antfly_b200 import _native as N
    from antfly_b200.ops import index_ops as IX

    dev = torch.device("cuda")
    assert N.status() == 0
    never = torch.zeros(4, dtype=torch.int32, device=dev)   # a counter that nothing bumps
    t0 = time.perf_counter()
    N.check(N.cuda().afb_peer_counter_wait(N.ptr(never), c_int(1), N.stream_ptr()), "wait")
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    t0 = time.perf_counter()
    N.check(N.cuda().afb_peer_counter_wait(N.ptr(never), c_int(1), N.stream_ptr()), "wait")
    torch.cuda.synchronize()
    second = time.perf_counter() - t0
    assert 1.0 < first < 10.0, first     # ran to the cross-GPU wait limit (about two seconds), not forever
    assert second < 0.5, second          # the recorded timeout makes the next wait give up at once
    assert N.status() & 16
    assert N.status() == 0               # reading cleared it
    # the merge half of the select: same wait inside the kernel, result still produced from what is there
    nq, k = 3, 4
    vals = torch.rand(nq, k, device=dev).sort(-1).values
    ids = torch.arange(nq * k, device=dev).view(nq, k).int()
    t0 = time.perf_counter()
    tv, ti, _, _ = IX.topk_select([(vals, ids, None, k)], nq, k, k, wait=(never, 1))
    torch.cuda.synchronize()
    assert 1.0 < time.perf_counter() - t0 < 10.0
    torch.testing.assert_close(tv, vals)
    # while the timeout is recorded the push half stores nothing and bumps no counter
    sink = torch.zeros(nq * k * 2 + nq + 1, dtype=torch.int32, device=dev)
    P = ctypes.c_void_p * 1
    push = (P(sink.data_ptr()), P(sink.data_ptr() + 4 * nq * k), P(sink.data_ptr() + 8 * nq * k),
            P(sink.data_ptr() + 4 * (2 * nq * k + nq)))
    IX.topk_select([(vals, ids, None, k)], nq, k, k, push=push)
    torch.cuda.synchronize()
    assert int(sink.abs().sum()) == 0
    assert N.status() & 16
    assert N.status() == 0
    IX.topk_select([(vals, ids, None, k)], nq, k, k, push=push)   # healthy again: rows land, counter counts CTAs
    torch.cuda.synchronize()
    assert int(sink[-1]) == nq
    assert N.status() == 0


@needs_gpu
def test_poison_from_another_thread_reaches_the_named_device():
    """A watchdog runs on a timer thread whose current device is 0 whatever the main thread selected; the poison
    must be written to the device that is named.  With one GPU this checks the call path from a non-main thread."""
    import threading

    from antfly_b200 import _native as N

    dev_index = torch.cuda.current_device()
    out = {}
    t = threading.Thread(target=lambda: out.setdefault("rc", N.poison_waits(dev_index)))
    t.start()
    t.join()
    assert out["rc"] == 0
    never = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    N.check(N.cuda().afb_peer_counter_wait(N.ptr(never), c_int(1), N.stream_ptr()), "wait")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5      # poisoned: gave up on its first poll
    assert N.status() & 16
    assert N.status() == 0
