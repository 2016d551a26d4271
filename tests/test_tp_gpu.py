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
