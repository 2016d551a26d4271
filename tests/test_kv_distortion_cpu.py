"""KV-codec score distortion report: sample stream, ordering of the codecs and the residual-scale sweep."""
import json

import numpy as np
import torch

from antfly_b200.ops import kv_quant as KQ
from antfly_b200.utils import kv_distortion as KD


def _splitmix(x):
    m = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def test_sample_stream_matches_scalar_definition():
    m = (1 << 64) - 1
    got = KD.sample_values(np.array([0, 5, 777]), 7, 0x1234ABCD)
    for r, s in enumerate((0, 5, 777)):
        for i in range(7):
            mixed = _splitmix(0x1234ABCD ^ ((s + 1) * 0x9E3779B97F4A7C15 & m) ^ ((i + 1) * 0xBF58476D1CE4E5B9 & m))
            want = np.float32(mixed >> 40) / np.float32(1 << 24) * 2.0 - 1.0
            assert got[r, i] == np.float32(want)
    assert got.min() >= -1.0 and got.max() < 1.0


def test_sketch_signs_match_host_residual_score():
    torch.manual_seed(0)
    H, D = 2, 64
    key = torch.rand(5, H, D) * 2 - 1
    q = torch.rand(H, D) * 2 - 1
    rows = KQ.encode_rows("turbo3", key)
    signs = KD.sketch_signs(rows, H, D)
    pq = torch.einsum("hd,hpd->hp", q, KQ.random_signs(H, D))
    unit = (signs * pq[None]).mean(-1)                                   # [T, H]
    base = (KQ.decode_rows("turbo3", rows, H, D) * q[None]).sum(-1)
    # the host attention over a single token returns that token's value; its score shows through two tokens' weights
    vals = torch.zeros(2, H, D)
    vals[0, :, 0] = 1.0
    v_rows = KQ.encode_rows("int8", vals, value=True)
    for t in (1, 3):
        k2 = torch.stack([rows[0], rows[t]])
        out = KQ.attention_host("turbo3", q, k2, v_rows, H, scale=1.0)
        w0 = out[:, 0]                                                    # softmax weight of token 0
        s = base + KQ.RESIDUAL_SCALE * unit
        want = torch.softmax(torch.stack([s[0], s[t]]), 0)[0]
        assert torch.allclose(w0, want, atol=2e-3)


def test_report_orders_codecs_and_finds_builtin_scale(capsys):
    rep = KD.measure(samples=256, heads=4, D=64)
    c = rep["codecs"]
    assert rep["dots"] == 256 * 4
    assert c["int8"]["rmse"] < c["fp8"]["rmse"] < c["int4"]["rmse"] < c["turbo3"]["rmse"]
    assert abs(c["polar4"]["rmse"] - c["int4"]["rmse"]) < 0.1
    assert c["turbo3"]["key_bytes_per_token"] < c["polar4"]["key_bytes_per_token"] < c["int4"]["key_bytes_per_token"]
    # the sketch correction helps, and the sweep's best multiplier is positive and near the built-in one
    assert rep["turbo3_residual_best"]["rmse"] < rep["turbo3_base"]["rmse"]
    assert rep["codecs"]["turbo3"]["rmse"] < rep["turbo3_base"]["rmse"]
    assert 0.0 < rep["turbo3_residual_best"]["scale"] <= 0.5
    assert len(rep["scale_sweep"]) == 33
    KD.main(["--samples", "64", "--num-kv-heads", "2", "--head-dim", "64"])
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert "scale_sweep" not in line and line["head_dim"] == 64
