"""The tcgen05 / tensor-memory flash attention kernel (csrc/kernels/attention_tc.cu) against the fp32 reference op:
packed encoder attention and causal paged prefill, head widths 64 and 128, lengths 1..512, windows, GQA.

Each case runs in a child process (tests/helpers/attention_tc_check.py) and reports through one JSON line, so a
first run of this kernel on a device is isolated from the test session's own CUDA context.  Tolerance: the one the
other attention tests use (2e-2 absolute + 2e-2 relative on bf16 outputs)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
needs_gpu = pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
HELPER = os.path.join(os.path.dirname(__file__), "helpers", "attention_tc_check.py")


def _run(spec):
    r = subprocess.run([sys.executable, HELPER, json.dumps(spec)], capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, (r.stdout + r.stderr)[-2000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["status"] == 0, res
    assert res["finite"] and res["bad"] == 0, res
    return res


VARLEN = [
    dict(D=64, Hq=12, Hkv=12, lens=[1, 32, 100, 128, 129, 300, 512], causal=False, window=0),     # BERT-base heads
    dict(D=64, Hq=4, Hkv=4, lens=[77, 255, 256, 257], causal=True, window=0),
    dict(D=64, Hq=4, Hkv=4, lens=[40, 400], causal=False, window=64),                             # two-sided local
    dict(D=128, Hq=8, Hkv=2, lens=[5, 64, 65, 200, 511], causal=True, window=0),                  # GQA
    dict(D=128, Hq=4, Hkv=4, lens=[130, 333], causal=True, window=100),
    dict(D=128, Hq=2, Hkv=2, lens=[512, 512], causal=False, window=0),
]


@needs_gpu
@pytest.mark.parametrize("case", VARLEN, ids=lambda c: f"D{c['D']}-h{c['Hq']}/{c['Hkv']}-{'c' if c['causal'] else 'b'}-w{c['window']}")
def test_tensor_core_varlen_attention_matches_fp32_reference(case):
    _run(dict(case, kind="varlen", seed=1))


PAGED = [
    dict(D=128, Hq=8, Hkv=2, q_lens=[128, 17, 300], ctx_lens=[0, 500, 64], window=0, page=16),    # chunked prefill
    dict(D=128, Hq=4, Hkv=4, q_lens=[5, 5], ctx_lens=[1000, 31], window=0, page=16),             # speculative verify
    dict(D=128, Hq=4, Hkv=1, q_lens=[200], ctx_lens=[300], window=128, page=32),
    dict(D=64, Hq=4, Hkv=2, q_lens=[256, 40], ctx_lens=[100, 0], window=0, page=16),
    dict(D=64, Hq=2, Hkv=2, q_lens=[64], ctx_lens=[700], window=0, page=64),
]


@needs_gpu
@pytest.mark.parametrize("case", PAGED, ids=lambda c: f"D{c['D']}-h{c['Hq']}/{c['Hkv']}-p{c['page']}-w{c['window']}")
def test_tensor_core_paged_prefill_attention_matches_fp32_reference(case):
    _run(dict(case, kind="paged", seed=2))
