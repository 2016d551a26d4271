"""Fused tensor-parallel path on real GPUs (needs at least two): child ranks under torchrun compare the peer-memory
fused step with the NCCL baseline.  Skipped on a single-GPU machine."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


from antfly_b200.parallel.launch import run_ranks

# Time limits: each child job gets 240 s and is ended politely (SIGTERM, the ranks drain their GPUs, SIGKILL only
# after a grace period); the three jobs of this file together stay far below any outer limit of a test run.
_LIMIT_S = 240


def _run_check(n: int, port: int, script_name: str, marker: str):
    script = os.path.join(os.path.dirname(__file__), "helpers", script_name)
    rc, out = run_ranks(n, [script], port, _LIMIT_S, env={"NCCL_DEBUG": "WARN"})
    assert out.count(marker) == n, out[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_fused_tp_single_rank_pushes_to_itself():
    """The fused kernels with a world of one: every push lands in the rank's own symmetric buffer."""
    _run_check(1, 29576, "tp_fused_check.py", "TP_FUSED_CHECK OK")


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_tp_matches_nccl_baseline():
    _run_check(2, 29577, "tp_fused_check.py", "TP_FUSED_CHECK OK")


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_dp_embedding_gather_and_sharded_search_merge():
    _run_check(2, 29578, "dp_sharded_check.py", "DP_SHARDED_CHECK OK")
