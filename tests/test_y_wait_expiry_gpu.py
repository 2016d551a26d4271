"""Failure detection on the device without faulting it: a cross-GPU wait that nothing will ever satisfy runs out,
reports through the status word, and poisons later waits so queued kernels drain; the host can poison waits too."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_cross_gpu_wait_expires_with_status_and_later_waits_give_up_at_once():
    """Failure detection on the device: a one-shot slot that no rank ever fills makes the consumer's bounded wait
    run out; the kernel returns normally, the status word carries the peer-timeout code, and while that code is
    set every further wait gives up on its first poll (a queued graph drains instead of serving one limit per
    kernel).  Reading the status clears it."""
    import ctypes
    import time

    from antfly_b200 import _native as N
    from antfly_b200.ops import quant as Q

    dev = torch.device("cuda")
    T, H, world = 4, 1024, 2
    slots = torch.full((world, T, H), -32768, dtype=torch.int16, device=dev)  # bf16 -0.0 everywhere: nothing landed
    residual = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)
    gamma = torch.ones(H, dtype=torch.bfloat16, device=dev)
    sum_out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    c_int, c_long, c_float = ctypes.c_int, ctypes.c_long, ctypes.c_float

    def run():
        mx = Q.new_mx(T, H, 2, dev)
        rc = N.cuda().afb_norm_tp(
            None, N.ptr(slots), c_int(world), c_long(T * H), c_int(2), N.ptr(residual), None, N.ptr(gamma), None,
            N.ptr(sum_out), None, None, c_int(T), c_int(H), c_float(1e-5), c_int(1), c_int(0), N.ptr(mx.q0),
            N.ptr(mx.q1), N.ptr(mx.sf0), N.ptr(mx.sf1), None, c_int(0), c_int(0), None, None, None, None, None, None,
            c_int(0), c_int(0), N.stream_ptr())
        N.check(rc, "afb_norm_tp")
        torch.cuda.synchronize()

    assert N.status() == 0
    t0 = time.perf_counter()
    run()
    first = time.perf_counter() - t0
    t0 = time.perf_counter()
    run()
    second = time.perf_counter() - t0
    st = N.status()
    assert st & 16, st                   # peer-flag timeout recorded
    assert 1.0 < first < 10.0, first     # the wait ran to its limit (about two seconds), not forever
    assert second < 0.5, second          # poisoned: the next wait gave up at once
    assert N.status() == 0               # reading cleared it
    # the host can poison the waits too (what a watchdog or a SIGTERM handler does before the process leaves)
    assert N.poison_waits() == 0
    t0 = time.perf_counter()
    run()
    assert time.perf_counter() - t0 < 0.5
    assert N.status() & 16
    assert N.status() == 0
