"""In-tree build of the native libraries.

Two shared objects are produced next to this file, under ``antfly_b200/_lib``:

* ``libafb_cuda.so``  -- every ``csrc/kernels/*.cu`` compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); plain ``extern "C"`` entry points, loaded with ctypes.
* ``libafb_host.so``  -- every ``csrc/host/*.cpp`` compiled by g++ (KV block allocator, scheduler,
  file-format readers, quantisation codecs, CPU oracle).

No torch headers are involved, so a full rebuild takes seconds per file and files compile in parallel.
Objects are rebuilt only when their source (or any header under ``csrc/common``) is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "_lib"
OBJ_DIR = LIB_DIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-march=x86-64-v3", "-fopenmp-simd"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return cand


def _newest_header_mtime() -> float:
    m = 0.0
    for p in list((CSRC / "common").glob("*")) + list((CSRC / "host").glob("*.h")) + list(
        (CSRC / "kernels").glob("*.cuh")
    ) + list((CSRC / "include").glob("*.h")):
        m = max(m, p.stat().st_mtime)
    return m


def _needs(obj: Path, src: Path, hdr_mtime: float) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return t < src.stat().st_mtime or t < hdr_mtime


def _run(cmd: list[str]) -> str:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> dict:
    """Compile everything that is out of date.  Returns {'cuda': path, 'host': path}."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header_mtime()
    nvcc = _nvcc()
    cu_srcs = sorted((CSRC / "kernels").glob("*.cu"))
    cpp_srcs = sorted((CSRC / "host").glob("*.cpp"))
    jobs = []
    for src in cu_srcs:
        obj = OBJ_DIR / (src.stem + ".cu.o")
        if force or _needs(obj, src, hdr):
            flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
            jobs.append([nvcc, *flags, "-c", str(src), "-o", str(obj)])
    for src in cpp_srcs:
        obj = OBJ_DIR / (src.stem + ".cpp.o")
        if force or _needs(obj, src, hdr):
            jobs.append(["g++", *CXX_FLAGS, "-c", str(src), "-o", str(obj)])
    logs = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            for out in ex.map(_run, jobs):
                logs.append(out)
                if verbose and out.strip():
                    print(out, file=sys.stderr)
    cuda_lib = LIB_DIR / "libafb_cuda.so"
    host_lib = LIB_DIR / "libafb_host.so"
    cu_objs = [str(OBJ_DIR / (s.stem + ".cu.o")) for s in cu_srcs]
    cpp_objs = [str(OBJ_DIR / (s.stem + ".cpp.o")) for s in cpp_srcs]
    if cu_objs and (jobs or not cuda_lib.exists()):
        _run([nvcc, "--shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(cuda_lib), *cu_objs,
              "-lcudart"])
    if cpp_objs and (jobs or not host_lib.exists()):
        _run(["g++", "-shared", "-pthread", "-o", str(host_lib), *cpp_objs])
    return {"cuda": cuda_lib, "host": host_lib, "logs": logs}


if __name__ == "__main__":
    res = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print("built:", res["cuda"], res["host"])
