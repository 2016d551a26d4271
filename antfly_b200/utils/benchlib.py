"""Measurement plumbing shared by the benchmark workloads (bench.py and the workloads that live inside the package):
clock sampling during the timed region, process-group bootstrap with exit guards, max-over-ranks, orderly exit."""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import sys
import time


def clock_sampler():
    """Starts nvidia-smi sampling SM clocks and throttle reasons every 50 ms for the GPUs of this job.  Only local
    rank 0 samples (for all of the job's GPUs); started before the warm-up steps because the tool takes longer to
    produce its first line than a short timed region lasts.  Returns None on the other ranks."""
    if int(os.environ.get("LOCAL_RANK", "0")) != 0:
        return None
    q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    n = int(os.environ.get("WORLD_SIZE", "1"))
    try:
        return subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "50",
                                 "-i", ",".join(str(i) for i in range(n))], stdout=subprocess.PIPE, text=True)
    except Exception:
        return None


def clock_summary(proc, t_begin=None, t_end=None):
    """Median SM clock and the throttle reasons seen between t_begin and t_end (datetime, local time); if the
    window caught no sample, all samples since the sampler started (warm-up and timed steps) are used."""
    import datetime

    if proc is None:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["not sampled on this rank"], "samples": 0}
    proc.terminate()
    try:
        out, _ = proc.communicate(timeout=5)
    except Exception:
        proc.kill()
        out = ""
    rows = []
    for line in out.strip().splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 10:
            continue
        try:
            ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
            rows.append((ts, float(f[2]), float(f[3]), f[6:10]))
        except ValueError:
            continue
    window = [r for r in rows if t_begin is not None and t_end is not None and t_begin <= r[0] <= t_end]
    scope = "timed region"
    if not window:
        window, scope = rows, "warm-up and timed steps"
    sm, mx, reasons = [r[1] for r in window], [r[2] for r in window], set()
    for r in window:
        for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3]):
            if v.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons), "samples": len(sm), "scope": scope}


def log(msg):
    if os.environ.get("ANTFLY_B200_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')} t={time.perf_counter():.1f}] {msg}", file=sys.stderr,
              flush=True)


def dist_setup(n_gpus):
    import torch
    import torch.distributed as dist

    import antfly_b200  # noqa: F401  (multicast-off defaults before NCCL / the symmetric allocator start)
    from antfly_b200.parallel.launch import install_exit_guards

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # A run that stops making progress dumps every thread's Python stack, drains THIS rank's GPU (poison the
    # bounded kernel waits, wait out one wait limit) and exits, instead of sitting in a collective until some outer
    # limit kills it without warning; SIGTERM takes the same path.  The default leaves ample room for a cold
    # start (first import on a fresh machine, an 8B model build, prefill).
    limit = int(os.environ.get("ANTFLY_B200_BENCH_WATCHDOG_S", "600" if world > 1 else "0"))
    if world > 1 or limit > 0:
        install_exit_guards(local, watchdog_s=limit)
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def finish(world):
    """Multi-rank exit: GPU idle, every rank here, process group destroyed, then leave (see finish_ranks)."""
    if world <= 1:
        return
    from antfly_b200.parallel.launch import finish_ranks

    finish_ranks()


def barrier(world):
    import torch

    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


