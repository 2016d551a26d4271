"""The reference arm's launcher reproduces the reference's launch geometry, and the reference kernel file it
drives is byte-identical to the reference's and compiles for sm_100a.

Formulas checked against zig/pkg/inference/src/ops/cuda/kernels.zig: launch1d (:1913, block 256, grid
ceil(n / 256)), launchBlocks (:1919), launch2d (:1925), the tiled linear launchers (:402-470, grid
(ceil(out / 4), ceil(rows / 2)), 256 threads), attention (:1068-1131), and the dispatch rules of
cuda_compute.zig:573 (tiles when rows >= 2, in >= 256, out >= 4)."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "baseline", name + ".py"))
    m = importlib.util.module_from_spec(spec)
    sys.modules[name] = m
    spec.loader.exec_module(m)
    return m


def test_launch_geometry_matches_the_reference_helpers():
    R = _load("ref_cuda")
    assert R.grid_1d(1) == ((1, 1, 1), 256) and R.grid_1d(256) == ((1, 1, 1), 256) and R.grid_1d(257) == ((2, 1, 1), 256)
    assert R.grid_blocks(16384, 256) == ((16384, 1, 1), 256)
    # BERT-base request of 32 x 512 tokens
    rows = 32 * 512
    assert R.grid_tiled_linear(rows, 768) == ((192, 8192, 1), 256)
    assert R.grid_tiled_linear(rows, 3072) == ((768, 8192, 1), 256)
    assert R.grid_tiled_linear(3, 5) == ((2, 2, 1), 256)
    assert R.linear_uses_tiles(rows, 768, 768) and R.linear_uses_tiles(2, 256, 4)
    assert not R.linear_uses_tiles(1, 768, 768) and not R.linear_uses_tiles(32, 255, 8) and not R.linear_uses_tiles(32, 768, 1)
    assert R.attention_uses_block_kernel(512, 64) and R.attention_uses_block_kernel(512, 128)
    assert not R.attention_uses_block_kernel(513, 64) and not R.attention_uses_block_kernel(128, 256)


def test_a_256_document_batch_must_be_fed_in_pipeline_sized_requests():
    """256 x 512 padded tokens in one call would need grid.y = 65,536 for the tiled linear -- one more than a
    launch accepts -- so the arm feeds the reference's own request size (batch_size 32)."""
    R = _load("ref_cuda")
    whole, _ = R.grid_tiled_linear(256 * 512, 768)
    assert whole[1] == 65536 and not R.grid_fits(whole)
    chunks = R.request_chunks(256)
    assert len(chunks) == 8 and chunks[0] == (0, 32) and chunks[-1] == (224, 256)
    for lo, hi in chunks:
        g, _ = R.grid_tiled_linear((hi - lo) * 512, 3072)
        assert R.grid_fits(g)
    # 32-bit index arithmetic of the kernels stays in range for a request
    assert 32 * 512 * 3072 < 2 ** 32 and 32 * 512 * 12 * 64 < 2 ** 32


def test_reference_kernel_file_is_unmodified_and_builds_for_sm_100a():
    B = _load("build_ref")
    ref = "/root/reference/" + B.REL
    if not os.path.exists(ref) and not os.path.exists(B.CU):
        pytest.skip("no reference checkout and no installed copy")
    meta = B.build()
    assert os.path.getsize(B.CUBIN) > 100_000
    if os.path.exists(ref):
        assert meta["sha256"] == B.sha256(ref)
    src = open(B.CU).read()
    for name in _load("ref_cuda").RefModule.NAMES:
        assert f"void {name}(" in src
