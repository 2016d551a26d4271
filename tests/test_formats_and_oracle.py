"""Formats (safetensors, GGUF + codecs), tokenizer rules, manifest lookup, CPU oracle.  No GPU needed."""
import ctypes
import json
import os

import numpy as np
import pytest
import torch

from antfly_b200 import _native as N
from antfly_b200.formats import gguf, manifest
from antfly_b200.formats import safetensors_io as st
from antfly_b200.models.bert import BertConfig, BertModel, pack_sequences
from antfly_b200.tokenizer import ByteTokenizer, WordPieceTokenizer


def test_safetensors_roundtrip_and_upstream_compat(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(4, 4).to(torch.bfloat16),
         "e": torch.empty(0, 3)}
    p = str(tmp_path / "m.safetensors")
    st.save_file(t, p, {"format": "pt"})
    back = st.load_file(p)
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) for k in t)
    try:
        from safetensors.torch import load_file, save_file
    except ImportError:
        return
    up = load_file(p)
    assert all(torch.equal(up[k], t[k]) for k in t)
    p2 = str(tmp_path / "u.safetensors")
    save_file({k: v for k, v in t.items()}, p2)
    ours = st.load_file(p2)
    assert all(torch.equal(ours[k], t[k]) for k in t)


def test_bert_weights_roundtrip_through_hf_names(tmp_path):
    cfg = BertConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, vocab_size=300)
    m = BertModel.random_init(cfg, device="cpu", seed=3)
    p = str(tmp_path / "model.safetensors")
    st.save_file(m.state_dict_hf(), p)
    m2 = BertModel.from_state_dict(cfg, st.load_model_dir(str(tmp_path)), device="cpu")
    b = pack_sequences([[5, 6, 7, 8], [9, 10]])
    torch.testing.assert_close(m.embed(b), m2.embed(b))


@pytest.mark.parametrize("ty,tol", [(0, 0.0), (1, 2e-3), (8, 2e-2), (2, 0.2)])
def test_gguf_write_read_dequantize(tmp_path, ty, tol):
    w = torch.randn(8, 64)
    p = str(tmp_path / "m.gguf")
    gguf.write_gguf(p, {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 64,
                        "tokenizer.ggml.tokens": ["a", "b"], "llama.rope.freq_base": 500000.0},
                    {"blk.0.attn_q.weight": (ty, w), "token_embd.weight": (0, torch.ones(2, 64))})
    f = gguf.GGUFFile(p)
    assert f.version == 3 and f.metadata["llama.block_count"] == 2 and f.metadata["tokenizer.ggml.tokens"] == ["a", "b"]
    info = f.tensors["blk.0.attn_q.weight"]
    assert info.shape == (8, 64) and gguf.hf_name(info.name) == "model.layers.0.self_attn.q_proj.weight"
    back = f.tensor("blk.0.attn_q.weight")
    assert float((back - w).abs().max()) <= tol * float(w.abs().max()) + 1e-7
    assert gguf.llama_config_from_gguf(f.metadata)["rope_theta"] == 500000.0


def test_q4k_and_mxfp4_decode_against_a_python_restatement():
    lib = N.host()
    rng = np.random.default_rng(0)
    # Q4_K: one super-block
    blk = rng.integers(0, 256, 144, dtype=np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.02).tobytes(), dtype=np.uint8)
    out = np.empty(256, dtype=np.float32)
    assert lib.afb_gguf_dequantize(12, blk.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                   ctypes.c_long(256)) == 0
    d, dmin = float(np.float16(0.01)), float(np.float16(0.02))
    sc, qs = blk[4:16], blk[16:]
    def sm(j):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
    ref = np.empty(256, dtype=np.float32)
    for c in range(4):
        s1, m1 = sm(2 * c); s2, m2 = sm(2 * c + 1)
        q = qs[32 * c:32 * c + 32]
        ref[64 * c:64 * c + 32] = d * s1 * (q & 0xF) - dmin * m1
        ref[64 * c + 32:64 * c + 64] = d * s2 * (q >> 4) - dmin * m2
    np.testing.assert_allclose(out, ref, rtol=1e-6, atol=1e-7)
    # MXFP4: scale 2^1, nibbles 0..15 in the low half
    blk = np.zeros(17, dtype=np.uint8)
    blk[0] = 128
    blk[1:17] = np.arange(16, dtype=np.uint8)
    out = np.empty(32, dtype=np.float32)
    lib.afb_gguf_dequantize(39, blk.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(32))
    np.testing.assert_allclose(out[:16], 2.0 * np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6]))
    assert np.all(out[16:] == 0)


def test_fp8_kv_codec_matches_torch_and_int4_roundtrip():
    lib = N.host()
    lib.afb_f32_to_e4m3.restype = ctypes.c_uint8
    lib.afb_f32_to_e4m3.argtypes = [ctypes.c_float]
    lib.afb_e4m3_to_f32.restype = ctypes.c_float
    lib.afb_e4m3_to_f32.argtypes = [ctypes.c_uint8]
    vals = torch.cat([torch.randn(2000) * 3, torch.tensor([0.0, 448.0, 1000.0, -1000.0, 2 ** -9, 2 ** -10, 0.0019])])
    ours = torch.tensor([lib.afb_f32_to_e4m3(float(v)) for v in vals], dtype=torch.uint8)
    ref = vals.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert float((ours == ref).float().mean()) > 0.999
    lut = np.empty(256, dtype=np.float32)
    lib.afb_e4m3_lut(lut.ctypes.data_as(ctypes.c_void_p))
    tl = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    ok = ~np.isnan(tl)
    np.testing.assert_array_equal(lut[ok], tl[ok])
    x = np.random.default_rng(1).standard_normal(64).astype(np.float32)
    enc = np.empty(36, dtype=np.uint8); dec = np.empty(64, dtype=np.float32)
    lib.afb_kv_encode_int4(x.ctypes.data_as(ctypes.c_void_p), enc.ctypes.data_as(ctypes.c_void_p), 64)
    lib.afb_kv_decode_int4(enc.ctypes.data_as(ctypes.c_void_p), dec.ctypes.data_as(ctypes.c_void_p), 64)
    assert np.abs(dec - x).max() <= np.abs(x).max() / 7 * 0.51 + 1e-3


def test_pair_encoding_gives_the_query_priority_and_types():
    tk = ByteTokenizer(512)
    ids, types = tk.encode_pair("qqqq", "d" * 100, max_length=20)
    assert len(ids) == 20 and ids[0] == tk.special.cls_id and ids[5] == tk.special.sep_id and ids[-1] == tk.special.sep_id
    assert types == [0] * 6 + [1] * 14
    ids, types = tk.encode_pair("q" * 100, "dddd", max_length=20)
    assert len(ids) == 20 and types == [0] * 19 + [1]  # the query took the whole budget; only the last [SEP] is type 1
    wp = WordPieceTokenizer({"[PAD]": 0, "[UNK]": 1, "[CLS]": 2, "[SEP]": 3, "hello": 4, "wor": 5, "##ld": 6, ",": 7})
    assert wp.encode("Hello, world") == [4, 7, 5, 6] and wp.decode([2, 4, 7, 5, 6, 3]) == "hello , world"
    assert wp.encode_for_model("hello zzz", 8) == [2, 4, 1, 3]


def test_manifest_resolution(tmp_path):
    d = tmp_path / "embedders" / "org" / "m"
    d.mkdir(parents=True)
    (d / "config.json").write_text(json.dumps({"model_type": "bert", "architectures": ["BertModel"]}))
    (d / "model.safetensors").write_bytes(b"")
    (d / "model_manifest.json").write_text(json.dumps({"tasks": ["embedder"], "capabilities": ["sparse"]}))
    p = manifest.resolve_model_path("org/m", str(tmp_path), "embedders")
    assert p == str(d)
    m = manifest.read_manifest(p)
    assert m.weights == "safetensors" and m.model_type == "embedder" and m.capabilities == ["sparse"]
    assert manifest.resolve_model_path("nope", str(tmp_path)) is None


def test_cpu_oracle_matches_torch_reference_path():
    from antfly_b200.ops import cpu_oracle

    cfg = BertConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, vocab_size=300)
    m = BertModel.random_init(cfg, device="cpu", seed=1, dtype=torch.float32)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(5, 300, (3, 16), generator=g, dtype=torch.int32)
    mask = torch.ones(3, 16, dtype=torch.int32)
    mask[1, 10:] = 0
    out = cpu_oracle.bert_embed(m, ids, None, mask)
    seqs = [ids[b][mask[b] > 0].tolist() for b in range(3)]
    ref = m.embed(pack_sequences(seqs))
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=2e-2)  # the torch path rounds activations to bf16
    x = torch.nn.functional.normalize(torch.randn(500, 64, generator=g), dim=-1)
    idx, dist = cpu_oracle.topk(out, x, 5, "cosine")
    d = 1 - torch.nn.functional.normalize(out, dim=-1) @ x.t()
    rv, ri = torch.topk(d, 5, largest=False)
    assert torch.equal(idx.long(), ri) and torch.allclose(dist, rv, atol=1e-5)
