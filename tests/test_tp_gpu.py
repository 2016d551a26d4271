"""Fused tensor-parallel path on real GPUs (needs at least two): child ranks under torchrun compare the peer-memory
fused step with the NCCL baseline.  Skipped on a single-GPU machine."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_tp_check(n: int, port: int):
    script = os.path.join(os.path.dirname(__file__), "helpers", "tp_fused_check.py")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), script], capture_output=True,
                       text=True, timeout=300, env=env)
    out = r.stdout + r.stderr
    assert out.count("TP_FUSED_CHECK OK") == n, out[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_fused_tp_single_rank_pushes_to_itself():
    """The fused kernels with a world of one: every push lands in the rank's own symmetric buffer."""
    _run_tp_check(1, 29576)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_tp_matches_nccl_baseline():
    n = 2
    script = os.path.join(os.path.dirname(__file__), "helpers", "tp_fused_check.py")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29577", script], capture_output=True,
                       text=True, timeout=300, env=env)
    out = r.stdout + r.stderr
    assert out.count("TP_FUSED_CHECK OK") == n, out[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_dp_embedding_gather_and_sharded_search_merge():
    n = 2
    script = os.path.join(os.path.dirname(__file__), "helpers", "dp_sharded_check.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29578", script], capture_output=True,
                       text=True, timeout=300, env=dict(os.environ, NCCL_DEBUG="WARN"))
    out = r.stdout + r.stderr
    assert out.count("DP_SHARDED_CHECK OK") == n, out[-3000:]


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
