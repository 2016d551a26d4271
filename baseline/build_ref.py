"""Installs the one part of the reference that builds offline: its CUDA kernel translation unit.

The reference project is a Zig + Go monorepo (no Python package, neither toolchain on this machine), so the
``pip install`` of it fails and its own host code cannot run here.  What does build is
``zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu``: self-contained (no #include), every entry
point ``extern "C"``.  This script copies that file UNCHANGED into ``baseline/_ref/`` (git-ignored) and compiles it
with nvcc for sm_100a into a cubin that ``baseline/ref_cuda.py`` loads through the CUDA driver API -- the same way
the reference loads its embedded PTX (``ops/cuda/kernels.zig:1980-2007``).  No file of this repository's own
kernels, models or engine is involved.

    python baseline/build_ref.py [--reference /root/reference]

On a machine without the reference checkout (the GPU box) an existing ``baseline/_ref`` is used as is.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REL = "zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu"
CU = os.path.join(REF_DIR, "inference_cuda_kernels.cu")
CUBIN = os.path.join(REF_DIR, "inference_cuda_kernels.sm_100a.cubin")
META = os.path.join(REF_DIR, "build.json")


def sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def build(reference_root: str = "/root/reference", force: bool = False) -> dict:
    os.makedirs(REF_DIR, exist_ok=True)
    src = os.path.join(reference_root, REL)
    if os.path.exists(src):
        if force or not os.path.exists(CU) or sha256(CU) != sha256(src):
            shutil.copyfile(src, CU)
    if not os.path.exists(CU):
        raise FileNotFoundError(f"{CU} is missing and no reference checkout at {reference_root}")
    meta = {"source": REL, "sha256": sha256(CU)}
    if force or not os.path.exists(CUBIN) or os.path.getmtime(CUBIN) < os.path.getmtime(CU):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        cmd = [nvcc, "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-o", CUBIN, CU]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on the reference kernels:\n" + r.stdout + r.stderr)
        meta["nvcc"] = " ".join(cmd[1:-2])
    meta["cubin_bytes"] = os.path.getsize(CUBIN)
    with open(META, "w") as f:
        json.dump(meta, f, indent=1)
    return meta


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(json.dumps(build(a.reference, a.force)))
