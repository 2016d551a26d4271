"""Host runtime under sanitizers: the C++ sources are rebuilt with AddressSanitizer + UndefinedBehaviorSanitizer
(and, for the threaded paths, ThreadSanitizer) together with a seeded stress driver, and the run must be clean."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRCS = sorted(str(p) for p in (ROOT / "csrc" / "host").glob("*.cpp"))
MAIN = str(ROOT / "csrc" / "host" / "selftest" / "sanitize_main.cpp")


def _build_and_run(tmp_path, flags, mode, env_extra):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / f"sanitize_{mode}")
    cmd = [cxx, "-std=c++17", "-O1", "-g", "-pthread", "-fno-omit-frame-pointer", *flags, *SRCS, MAIN, "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 and "cannot find" in r.stderr:
        pytest.skip("sanitizer runtime not installed: " + r.stderr.splitlines()[-1])
    assert r.returncode == 0, r.stderr[-3000:]
    for seed in ("1", "2"):
        run = subprocess.run([exe, mode, seed], capture_output=True, text=True, timeout=600,
                             env={**os.environ, **env_extra})
        assert run.returncode == 0, (run.stdout + run.stderr)[-4000:]
        assert "failures=0" in run.stdout and "Sanitizer" not in run.stderr and "runtime error" not in run.stderr, \
            run.stderr[-4000:]


def test_host_runtime_under_asan_and_ubsan(tmp_path):
    _build_and_run(tmp_path, ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "asan",
                   {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1"})


def test_threaded_paths_under_tsan(tmp_path):
    _build_and_run(tmp_path, ["-fsanitize=thread"], "tsan", {"TSAN_OPTIONS": "halt_on_error=1"})
