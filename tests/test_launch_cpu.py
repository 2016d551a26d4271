"""Polite termination of multi-rank jobs: a job that overruns its limit gets SIGTERM first, its ranks run their
exit guards (on a GPU box: poison the bounded kernel waits and drain), and only stragglers are killed."""
import os
import sys
import textwrap
import time

from antfly_b200.parallel.launch import rank_env, run_ranks


def test_rank_env_switches_nvlink_multicast_off_by_default():
    env = rank_env({"X": "1"})
    assert env["NCCL_NVLS_ENABLE"] == "0" and env["TORCH_SYMM_MEM_DISABLE_MULTICAST"] == "1" and env["X"] == "1"
    import antfly_b200  # noqa: F401

    assert os.environ.get("NCCL_NVLS_ENABLE") == "0"


def test_overrunning_job_is_terminated_politely(tmp_path):
    script = tmp_path / "sleeper.py"
    script.write_text(textwrap.dedent('''
        import os, signal, sys, time
        def on_term(*_):
            print(f"rank {os.environ['RANK']}: drained", flush=True)
            os._exit(4)
        signal.signal(signal.SIGTERM, on_term)
        print(f"rank {os.environ['RANK']}: started", flush=True)
        time.sleep(600)
    '''))
    t0 = time.time()
    rc, out = run_ranks(2, [str(script)], 29621, timeout_s=12.0, env={"PYTHONPATH": os.pathsep.join(sys.path)})
    took = time.time() - t0
    assert out.count("started") == 2, out
    assert out.count("drained") == 2, out      # both ranks ran their SIGTERM path before going away
    assert "time limit reached" in out
    assert took < 40, took
    assert rc != 0


def test_job_that_finishes_in_time_returns_its_output(tmp_path):
    script = tmp_path / "quick.py"
    script.write_text("import os; print('hello from', os.environ['RANK'])\n")
    rc, out = run_ranks(2, [str(script)], 29622, timeout_s=120.0)
    assert rc == 0 and out.count("hello from") == 2
