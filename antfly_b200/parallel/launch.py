"""Starting and, above all, STOPPING multi-rank jobs without leaving kernels behind.

``run_ranks`` starts ``torch.distributed.run`` in a process group of its own and enforces a time limit politely:
on expiry it sends SIGTERM to the whole group, gives the ranks time to drain their GPUs, and only then SIGKILLs
what is left.  ``install_exit_guards`` is the rank-side half: SIGTERM and an optional watchdog both poison the
bounded kernel waits of THIS rank's GPU, wait longer than one cross-GPU wait limit and then leave.  A rank killed
outright while its kernels poll a peer's memory is what this avoids; a job's inner limits must therefore also add
up to less than whatever outer limit would kill it without warning.
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import threading
import time
from typing import Dict, Optional, Sequence, Tuple

#: seconds between SIGTERM and SIGKILL: longer than the ranks' own drain (``_native.DRAIN_SECONDS``)
TERM_GRACE_S = 12.0


def rank_env(extra: Optional[Dict[str, str]] = None) -> Dict[str, str]:
    """Environment of a multi-rank child: NVLink multicast off in NCCL and in the symmetric-memory allocator (a
    rank that goes away while bound to a multicast object can fault its peers' GPUs), rendezvous on loopback."""
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    env.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    if extra:
        env.update(extra)
    return env


def run_ranks(n: int, script_and_args: Sequence[str], port: int, timeout_s: float,
              env: Optional[Dict[str, str]] = None) -> Tuple[int, str]:
    """Runs ``script_and_args`` on n ranks of this machine.  Returns (exit code, combined output); exit code -15 /
    -9 when the limit ended the job.  Never raises on timeout."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), *script_and_args]
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=rank_env(env),
                         start_new_session=True)
    try:
        out, _ = p.communicate(timeout=timeout_s)
        return p.returncode, out
    except subprocess.TimeoutExpired:
        pass
    out = ""
    try:
        os.killpg(p.pid, signal.SIGTERM)       # the launcher forwards it; ranks run their drain handlers
    except ProcessLookupError:
        pass
    try:
        out, _ = p.communicate(timeout=TERM_GRACE_S)
    except subprocess.TimeoutExpired:
        try:
            os.killpg(p.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass
        out, _ = p.communicate()
    return p.returncode if p.returncode is not None else -9, (out or "") + "\n[run_ranks] time limit reached"


def install_exit_guards(local_device: int, watchdog_s: float = 0.0, exit_code: int = 3) -> None:
    """Rank-side: SIGTERM, and a watchdog after `watchdog_s` seconds (0 = none), drain this rank's GPU before the
    process goes away.  The watchdog also dumps every thread's Python stack first."""
    import faulthandler

    def leave(code: int) -> None:
        try:
            from .. import _native as N

            N.drain_for_exit(local_device)
        finally:
            os._exit(code)

    def on_term(*_):
        leave(4)

    def on_watchdog():
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        leave(exit_code)

    try:
        signal.signal(signal.SIGTERM, on_term)
    except ValueError:  # not the main thread
        pass
    if watchdog_s > 0:
        t = threading.Timer(watchdog_s, on_watchdog)
        t.daemon = True
        t.start()


def finish_ranks(group=None, grace_s: float = 20.0) -> None:
    """Orderly multi-rank exit: GPU idle, every rank here, process group destroyed (NCCL lets go of its peer
    mappings), then leave.  A teardown that blocks is cut short by a timer -- the GPU is idle by then."""
    import gc

    import torch
    import torch.distributed as dist

    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier(group)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    t = threading.Timer(grace_s, lambda: os._exit(0))
    t.daemon = True
    t.start()
    gc.collect()
    try:
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)
