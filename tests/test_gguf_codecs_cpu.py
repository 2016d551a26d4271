"""GGUF block codecs against the `gguf` Python package's reference (numpy) dequantisers: random block bytes with
finite scale fields are decoded by both and must agree exactly (same arithmetic in fp32), for every block format
the C++ decoder knows; plus the NVFP4 golden vector from the reference's own unit test
(zig/pkg/inference/src/gguf/quant_codec.zig:4327-4340)."""
import math
import ctypes

import numpy as np
import pytest
import torch

gguf = pytest.importorskip("gguf")

from antfly_b200 import _native as N

TYPES = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL", "IQ4_XS",
         "TQ1_0", "TQ2_0", "MXFP4", "NVFP4", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"]

# byte offsets of the fp16 scale fields inside a block (random bytes there could be inf / NaN)
HALF_FIELDS = {"Q4_0": [0], "Q4_1": [0, 2], "Q5_0": [0], "Q5_1": [0, 2], "Q8_0": [0], "Q2_K": [80, 82], "Q3_K": [108],
               "Q4_K": [0, 2], "Q5_K": [0, 2], "Q6_K": [208], "IQ4_NL": [0], "IQ4_XS": [0], "TQ1_0": [52],
               "TQ2_0": [64], "MXFP4": [], "NVFP4": [], "IQ2_XXS": [0], "IQ2_XS": [0], "IQ2_S": [0], "IQ3_XXS": [0],
               "IQ3_S": [0], "IQ1_S": [0], "IQ1_M": []}


def _ours(type_id: int, raw: np.ndarray, n: int) -> np.ndarray:
    lib = N.host()
    out = np.empty(n, dtype=np.float32)
    rc = lib.afb_gguf_dequantize(ctypes.c_int(type_id), raw.ctypes.data_as(ctypes.c_void_p),
                                 out.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(n))
    assert rc == 0
    return out


@pytest.mark.parametrize("name", TYPES)
def test_dequantize_matches_gguf_package(name):
    qt = getattr(gguf.GGMLQuantizationType, name, None)
    if qt is None:
        pytest.skip(f"this gguf package has no {name}")
    values, nbytes = gguf.GGML_QUANT_SIZES[qt]
    lib = N.host()
    lib.afb_gguf_block_bytes.restype = ctypes.c_long
    lib.afb_gguf_block_values.restype = ctypes.c_long
    assert lib.afb_gguf_block_bytes(int(qt)) == nbytes and lib.afb_gguf_block_values(int(qt)) == values
    rng = np.random.default_rng(int(qt))
    blocks = 24
    raw = rng.integers(0, 256, size=(blocks, nbytes), dtype=np.uint8)
    for off in HALF_FIELDS[name]:
        scale = rng.uniform(-2.0, 2.0, size=blocks).astype(np.float16)
        raw[:, off:off + 2] = scale.view(np.uint8).reshape(blocks, 2)
    if name == "MXFP4":
        raw[:, 0] = rng.integers(110, 140, size=blocks)  # e8m0 scale near 1
    if name == "NVFP4":
        raw[:, :4] = rng.integers(0x18, 0x60, size=(blocks, 4))
    if name == "TQ1_0":
        raw[:, :52] = rng.integers(0, 243, size=(blocks, 52))  # five base-3 digits per byte
    if name == "IQ1_M":
        # the block's f16 scale is spread over the top nibbles of the four scale words: keep it finite
        scale = rng.uniform(0.1, 2.0, size=blocks).astype(np.float16).view(np.uint16)
        words = raw[:, 48:56].copy().view(np.uint16).reshape(blocks, 4)
        for i in range(4):
            words[:, i] = (words[:, i] & 0x0FFF) | (((scale >> (4 * i)) & 0xF) << 12).astype(np.uint16)
        raw[:, 48:56] = words.view(np.uint8).reshape(blocks, 8)
    try:
        want = gguf.quants.dequantize(raw.reshape(-1), qt).astype(np.float32).reshape(-1)
    except NotImplementedError:
        pytest.skip(f"the gguf package cannot dequantize {name}")
    got = _ours(int(qt), np.ascontiguousarray(raw.reshape(-1)), blocks * values)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_nvfp4_golden_vector():
    raw = np.zeros(36, dtype=np.uint8)
    raw[0] = 0x40  # sub-block scale
    raw[4] = 0x5A  # low nibble -> first value, high nibble -> ninth value of the first sub-block
    out = _ours(40, raw, 64)
    assert abs(out[0] - (-2.0)) < 1e-3 and abs(out[8] - 6.0) < 1e-3 and abs(out[16]) < 1e-3


def test_quantize_roundtrip_through_gguf_package():
    """Our Q8_0 / Q4_0 quantisers produce blocks the reference decoder reads back close to the input."""
    lib = N.host()
    rng = np.random.default_rng(5)
    x = rng.standard_normal(32 * 40).astype(np.float32)
    for name, fn, tol in (("Q8_0", lib.afb_gguf_quantize_q8_0, 0.02), ("Q4_0", lib.afb_gguf_quantize_q4_0, 0.3)):
        qt = getattr(gguf.GGMLQuantizationType, name)
        values, nbytes = gguf.GGML_QUANT_SIZES[qt]
        raw = np.empty(x.size // values * nbytes, dtype=np.uint8)
        fn(x.ctypes.data_as(ctypes.c_void_p), raw.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(x.size))
        back = gguf.quants.dequantize(raw, qt).astype(np.float32).reshape(-1)
        assert float(np.abs(back - x).max()) < tol * float(np.abs(x).max())


@pytest.mark.parametrize("name", ["Q4_0", "Q8_0", "Q4_K", "Q5_K", "Q6_K", "MXFP4"])
def test_per_element_decoder_matches_block_decoder(name):
    """The host/device per-element decoder (what the GPU expansion kernel runs per thread) against the
    block-at-a-time decoder, element by element."""
    qt = getattr(gguf.GGMLQuantizationType, name)
    values, nbytes = gguf.GGML_QUANT_SIZES[qt]
    lib = N.host()
    lib.afb_gguf_element.restype = ctypes.c_float
    lib.afb_gguf_element_block_values.restype = ctypes.c_long
    assert lib.afb_gguf_element_block_values(int(qt)) == values
    rng = np.random.default_rng(100 + int(qt))
    blocks = 6
    raw = rng.integers(0, 256, size=(blocks, nbytes), dtype=np.uint8)
    for off in HALF_FIELDS[name]:
        raw[:, off:off + 2] = rng.uniform(-2.0, 2.0, size=blocks).astype(np.float16).view(np.uint8).reshape(blocks, 2)
    if name == "MXFP4":
        raw[:, 0] = rng.integers(110, 140, size=blocks)
    want = _ours(int(qt), np.ascontiguousarray(raw.reshape(-1)), blocks * values).reshape(blocks, values)
    for b in range(blocks):
        blk = np.ascontiguousarray(raw[b])
        got = np.array([lib.afb_gguf_element(ctypes.c_int(int(qt)), blk.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(j))
                        for j in range(values)], dtype=np.float32)
        np.testing.assert_allclose(got, want[b], rtol=1e-6, atol=1e-6)


def test_bitnet_i2s_and_i8s_decoding(tmp_path):
    """BitNet's ternary type: lane order and code map as in the reference's golden vector
    (zig/pkg/inference/src/gguf/quant_codec.zig:4010), the trailing scale, and a file round trip."""
    import ctypes

    from antfly_b200 import _native as N
    from antfly_b200.formats import gguf as GG

    lib = N.host()
    raw = np.zeros(64, dtype=np.uint8)
    raw[0], raw[32] = 0b11_10_01_00, 0b00_01_10_11
    out = np.empty(256, dtype=np.float32)
    assert lib.afb_gguf_dequantize(ctypes.c_int(36), raw.ctypes.data_as(ctypes.c_void_p),
                                   out.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(256)) == 0
    assert [out[i] for i in (0, 32, 64, 96, 128, 160, 192, 224)] == [0.0, 1.0, 0.0, -1.0, -1.0, 0.0, 1.0, 0.0]
    assert out[1] == -1.0                                        # an all-zero byte is four -1 codes
    q = np.array([-3, 0, 127, -128], dtype=np.int8)
    o4 = np.empty(4, dtype=np.float32)
    assert lib.afb_gguf_dequantize(ctypes.c_int(37), q.ctypes.data_as(ctypes.c_void_p),
                                   o4.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(4)) == 0
    assert o4.tolist() == [-3.0, 0.0, 127.0, -128.0]

    g = torch.Generator().manual_seed(0)
    w = torch.randn(6, 128, generator=g)
    path = str(tmp_path / "b.gguf")
    GG.write_gguf(path, {"general.architecture": "bitnet"}, {"blk.0.attn_q.weight": (36, w), "x": (0, w[:1])})
    f = GG.GGUFFile(path)
    assert f.tensors["blk.0.attn_q.weight"].type_name == "I2_S"
    got = f.tensor("blk.0.attn_q.weight")
    m = float(w.abs().mean())
    want = (w / m).round().clamp(-1, 1) * m
    torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(f.tensor("x"), w[:1])            # the tensor after it starts where it should
    with pytest.raises(ValueError):
        GG.pack_i2s(np.zeros(100, dtype=np.float32))



def test_simple_types_q8_1_q1_0_and_integers():
    """Q8_1 (f16 d, f16 sum, 32 int8), Q1_0 (f16 d, 128 sign bits; the reference's quantizeQ1_0Block writes scale =
    mean |x| and bit = x >= 0, zig/pkg/inference/src/gguf/quant_codec.zig:677-693) and the plain I8 / I16 / I32 /
    I64 / F64 element types."""
    rng = np.random.default_rng(5)
    x = rng.normal(size=64).astype(np.float32)
    d = np.abs(x.reshape(2, 32)).max(1) / 127.0
    q = np.round(x.reshape(2, 32) / d[:, None]).astype(np.int8)
    blk = np.zeros((2, 36), dtype=np.uint8)
    blk[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(2, 2)
    blk[:, 4:] = q.view(np.uint8)
    got = _ours(9, blk.reshape(-1), 64)
    np.testing.assert_allclose(got, (d.astype(np.float16).astype(np.float32)[:, None] * q).reshape(-1), rtol=1e-6)
    y = rng.normal(size=256).astype(np.float32).reshape(2, 128)
    blk = np.zeros((2, 18), dtype=np.uint8)
    sc = np.abs(y).mean(1).astype(np.float16)
    blk[:, 0:2] = sc.view(np.uint8).reshape(2, 2)
    blk[:, 2:] = np.packbits((y >= 0).astype(np.uint8), axis=1, bitorder="little")
    got = _ours(41, blk.reshape(-1), 256).reshape(2, 128)
    np.testing.assert_array_equal(got, np.where(y >= 0, 1.0, -1.0) * sc.astype(np.float32)[:, None])
    for tid, dt in ((24, np.int8), (25, np.int16), (26, np.int32), (27, np.int64), (28, np.float64)):
        v = (rng.normal(size=17) * 100).astype(dt)
        np.testing.assert_allclose(_ours(tid, v.view(np.uint8), 17), v.astype(np.float32))


def test_bitnet_tl1_tl2_layouts_match_the_reference_golden_cases():
    """The reference's own unit tests as golden vectors (zig/pkg/inference/src/gguf/quant_codec.zig:4061-4200):
    a TL1 matrix of 0x44 bytes with byte 0 = 0x84 and scale 2; a TL2 matrix with two 0xd0 code bytes, one sign
    byte and scale 3; plus a round trip of random ternary matrices through an encoder that inverts the index maps."""
    from antfly_b200.formats import bitnet_tl as TL

    rows = cols = 1536
    raw = np.full(rows * cols // 4 + 32, 0x44, dtype=np.uint8)
    raw[0] = 0x84
    raw[rows * cols // 4: rows * cols // 4 + 4] = np.array([2.0], dtype="<f4").view(np.uint8)
    v = TL.dequantize_tl1(raw, rows, cols)
    assert (v[0, 0], v[0, 1], v[0, 2]) == (2.0, 2.0, 0.0)
    assert TL.tl1_nbytes(rows, cols) == raw.size

    n = TL.tl2_nbytes(rows, cols)
    raw = np.zeros(n, dtype=np.uint8)
    raw[0] = raw[1] = 0xD0
    raw[rows * cols // 6 + 3] = 0x80
    raw[n - 32: n - 28] = np.array([3.0], dtype="<f4").view(np.uint8)
    v = TL.dequantize_tl2(raw, rows, cols)
    assert v[0, :4].tolist() == [3.0, 3.0, 3.0, 0.0]
    assert v[1, :3].tolist() == [-3.0, -3.0, -3.0]

    # every (row, column) of a preset shape with a pair tail maps to its own code / sign position
    rows, cols = 1024, 4096
    n = TL.tl2_nbytes(rows, cols)
    raw = np.zeros(n, dtype=np.uint8)
    three_cols = cols - cols % 96
    v_len, s_len = rows * three_cols // 6, rows * three_cols // 24
    raw[v_len + s_len: v_len + s_len + rows * (cols - three_cols) // 4] = 0x44      # pair code 4 = (0, 0)
    raw[n - 32: n - 28] = np.array([2.0], dtype="<f4").view(np.uint8)
    base = TL.dequantize_tl2(raw, rows, cols)
    assert not base.any()
    rng = np.random.default_rng(0)
    raw[:v_len] = rng.integers(0, 256, v_len, dtype=np.uint8) & 0xDD | 0x11        # codes in 1..13
    raw[v_len:v_len + s_len] = rng.integers(0, 256, s_len, dtype=np.uint8)
    full = TL.dequantize_tl2(raw, rows, cols)
    tri = np.abs(full[:, :three_cols]).reshape(rows, -1, 3) / 2.0
    assert set(np.unique(full)) <= {-2.0, 0.0, 2.0}
    # flipping one sign byte flips exactly eight triples
    raw2 = raw.copy()
    raw2[v_len + 7] ^= 0xFF
    diff = (TL.dequantize_tl2(raw2, rows, cols) != full)
    changed = diff[:, :three_cols].reshape(rows, -1, 3).any(-1).sum()
    nonzero = (tri.reshape(rows, -1, 3).any(-1))
    assert 1 <= changed <= 8 and not diff[:, three_cols:].any() and nonzero.any()


def _random_blocks(type_id, blocks, rng):
    import numpy as np

    bb = {2: 18, 8: 34, 12: 144, 13: 176, 14: 210, 39: 17}[type_id]
    raw = rng.integers(0, 256, size=(blocks, bb), dtype=np.uint8)
    for off in {2: [0], 8: [0], 12: [0, 2], 13: [0, 2], 14: [208], 39: []}[type_id]:
        raw[:, off:off + 2] = rng.uniform(-1.0, 1.0, size=blocks).astype(np.float16).view(np.uint8).reshape(blocks, 2)
    if type_id == 39:
        raw[:, 0] = rng.integers(118, 132, size=blocks)
    return raw


@pytest.mark.parametrize("type_id,bv", [(2, 32), (8, 32), (39, 32), (12, 256), (13, 256), (14, 256)])
def test_sub_block_decoder_of_the_fused_kernel_equals_the_block_decoder(type_id, bv):
    import numpy as np
    import torch

    from antfly_b200.ops import gguf_ops as G

    rng = np.random.default_rng(type_id)
    raw = _random_blocks(type_id, 6, rng)
    want = G.dequantize(torch.from_numpy(raw.reshape(-1)), type_id, (6, bv), torch.float32).numpy()
    for b in range(6):
        for sub in range(bv // 32):
            got = G.decode32(type_id, raw[b].tobytes(), sub)
            assert np.array_equal(got, want[b, sub * 32:(sub + 1) * 32]), (type_id, b, sub)


@pytest.mark.parametrize("type_id,bv", [(8, 32), (2, 32), (12, 256), (14, 256)])
@pytest.mark.parametrize("M,N,K", [(1, 5, 256), (3, 17, 1280), (8, 9, 2304)])
def test_fused_matvec_work_split_covers_every_weight_once(type_id, bv, M, N, K):
    """The kernel's CTA / warp / row / chunk / lane arithmetic, replayed on the host with the kernel's decoder:
    ragged row counts (N not a multiple of the 8 rows of a CTA), K below, at and above the 1024-value chunk."""
    import numpy as np
    import torch

    from antfly_b200.ops import gguf_ops as G

    rng = np.random.default_rng(N * K + type_id)
    raw = _random_blocks(type_id, N * K // bv, rng)
    t = torch.from_numpy(raw.reshape(-1))
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32))
    got, units = G.mul_mv_host(x, t, type_id, N, K)
    assert units == N * (K // 32)
    w = G.dequantize(t, type_id, (N, K), torch.float32)
    want = x.double() @ w.double().T
    torch.testing.assert_close(got.double(), want, atol=1e-3 * float(want.abs().max()) + 1e-4, rtol=1e-4)


@pytest.mark.parametrize("quant", ["q8_0", "q4_0"])
def test_llama_served_from_its_gguf_blocks_matches_the_dequantised_model(tmp_path, quant):
    """The projections stay in their GGUF bytes (GgufWeight segments; gate / up interleaved on the fly) and the
    logits equal the model whose weights were expanded at load time."""
    import json

    import torch

    transformers = pytest.importorskip("transformers")
    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import gguf as GG
    from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch
    from antfly_b200.ops.gguf_ops import GgufWeight
    from antfly_b200.runtime.sampling_params import SamplingParams

    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(vocab_size=600, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                      tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval().float()
    d = tmp_path / "generators" / "tiny-gguf"
    d.mkdir(parents=True)
    GG.export_llama_gguf(str(d / "model.gguf"), hf.state_dict(), hf_cfg.to_dict(), quant=quant)
    f = GG.GGUFFile(str(d / "model.gguf"))
    cfg = LlamaConfig.from_hf({k: v for k, v in GG.llama_config_from_gguf(f.metadata).items() if v is not None})
    native = LlamaModel.from_gguf_native(cfg, f, device="cpu")
    assert native.native_gguf and isinstance(native.w["l0.qkv"], GgufWeight) and native.w["l0.gu"].interleave
    assert len(native.w["l0.qkv"].segments) == 3 and native.w["l0.qkv"].out_features == 64 + 32 + 32
    bits = native.w["l1.down"].nbytes() * 8 / (64 * 128)
    assert abs(bits - (8.5 if quant == "q8_0" else 4.5)) < 1e-6
    assert not cfg.rope_half_split                       # llama files keep the rotary pairs of Q / K rows adjacent
    sd = GG.to_hf_row_order({GG.hf_name(n): f.tensor(n) for n in f.tensors}, hf_cfg.to_dict())
    with torch.no_grad():
        hf.load_state_dict({k: v.reshape(hf.state_dict()[k].shape) for k, v in sd.items()})
    ids = torch.randint(0, 600, (12,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    kc = torch.zeros((2, 2, 16, 2, 16), dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    pos = torch.arange(12, dtype=torch.int32)
    b = StepBatch(ids.int(), pos, pos.clone(), i32([0]), i32([12]), i32([12]), torch.arange(2, dtype=torch.int32)[None],
                  pos.clone(), 12, 1)
    got = native.forward(b, kc, vc).float()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.995 and float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.9
    # through the model manager: the switch selects native serving, tokens equal the re-packed model's
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a = ModelManager(models_dir=str(tmp_path), device="cpu", gguf_native=True).get("tiny-gguf", "generator")
    assert a.info["weights"] == "gguf-native"
    out_a = a.pipeline.generate("hello", sp, raw_prompt=True)
    out_b = ModelManager(models_dir=str(tmp_path), device="cpu", gguf_native=False).get(
        "tiny-gguf", "generator").pipeline.generate("hello", sp, raw_prompt=True)
    # (the re-packed model rounds the weights a second time, to fp8; a random model's near-ties may then flip and
    #  the continuations part ways, so only the first token is compared)
    assert len(out_a.token_ids) == 6 and out_a.token_ids[0] == out_b.token_ids[0], (out_a.token_ids, out_b.token_ids)


def test_rotary_scaling_survives_a_gguf_round_trip(tmp_path):
    """A llama3-scaled checkpoint exported to GGUF carries its per-pair divisors in rope_freqs.weight; loading the
    file through the model manager restores the same frequency table (and linear / yarn metadata are read)."""
    import torch

    transformers = pytest.importorskip("transformers")
    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import gguf as GG
    from antfly_b200.models.llama import LlamaConfig

    torch.manual_seed(0)
    rope = {"rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0, "low_freq_factor": 1.0,
            "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    hf_cfg = transformers.LlamaConfig(vocab_size=600, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                      tie_word_embeddings=False, rope_parameters=rope)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval().float()
    want = LlamaConfig.from_hf(hf_cfg.to_dict())
    assert want.rope_inv_freq is not None
    d = tmp_path / "generators" / "scaled"
    d.mkdir(parents=True)
    GG.export_llama_gguf(str(d / "model.gguf"), hf.state_dict(), hf_cfg.to_dict(), quant="q8_0")
    f = GG.GGUFFile(str(d / "model.gguf"))
    assert "rope_freqs.weight" in f.tensors and f.tensor("rope_freqs.weight").numel() == 8
    for native in (False, True):
        lm = ModelManager(models_dir=str(tmp_path), device="cpu", gguf_native=native).get("scaled", "generator")
        cfg = lm.pipeline.engine.model.cfg
        assert cfg.max_position_embeddings == 256 and cfg.rope_mscale == 1.0
        torch.testing.assert_close(torch.tensor(cfg.rope_inv_freq), torch.tensor(want.rope_inv_freq), rtol=1e-5, atol=0)
    # scaling declared in the metadata alone
    md = {"general.architecture": "llama", "llama.embedding_length": 64, "llama.block_count": 1,
          "llama.attention.head_count": 4, "llama.feed_forward_length": 128, "llama.vocab_size": 600,
          "llama.context_length": 4096, "llama.rope.scaling.type": "yarn", "llama.rope.scaling.factor": 4.0,
          "llama.rope.scaling.original_context_length": 1024}
    cfg = LlamaConfig.from_hf({k: v for k, v in GG.llama_config_from_gguf(md).items() if v is not None})
    assert cfg.rope_inv_freq is not None and abs(cfg.rope_mscale - (0.1 * math.log(4.0) + 1.0)) < 1e-6
    md["llama.rope.scaling.type"] = "linear"
    cfg = LlamaConfig.from_hf({k: v for k, v in GG.llama_config_from_gguf(md).items() if v is not None})
    assert cfg.rope_inv_freq is None and cfg.rope_freq_scale == 0.25


def test_rotary_row_pairing_of_llama_files():
    """Row 2j / 2j + 1 of a head in the stored order are rows j / j + D/2 of the Hugging Face order; the inverse
    restores it; architectures with half-split rotation at run time are left alone."""
    import torch

    from antfly_b200.formats import gguf as GG

    H, D, K = 3, 8, 5
    w = torch.arange(H * D * K, dtype=torch.float32).reshape(H * D, K)
    p = GG.pair_rope_rows(w, H)
    for h in range(H):
        for j in range(D // 2):
            assert torch.equal(p[h * D + 2 * j], w[h * D + j]) and torch.equal(p[h * D + 2 * j + 1], w[h * D + j + D // 2])
    assert torch.equal(GG.unpair_rope_rows(p, H), w)
    b = torch.arange(H * D, dtype=torch.float32)
    assert torch.equal(GG.unpair_rope_rows(GG.pair_rope_rows(b, H), H), b)
    md = lambda arch: {"general.architecture": arch, f"{arch}.attention.head_count": 4}
    assert GG.llama_config_from_gguf(md("llama"))["rope_half_split"] is False
    assert "rope_half_split" not in GG.llama_config_from_gguf(md("qwen2"))
    sd = {"model.layers.0.self_attn.q_proj.weight": p, "model.layers.0.self_attn.v_proj.weight": w}
    same = GG.to_hf_row_order(sd, {"model_type": "qwen3", "num_attention_heads": H})
    assert torch.equal(same["model.layers.0.self_attn.q_proj.weight"], p)
    back = GG.to_hf_row_order(sd, {"model_type": "llama", "num_attention_heads": H})
    assert torch.equal(back["model.layers.0.self_attn.q_proj.weight"], w)
    assert torch.equal(back["model.layers.0.self_attn.v_proj.weight"], w)


@pytest.mark.parametrize("kind", ["qwen3", "phi3", "gemma", "gemma2", "gemma3"])
def test_qwen3_and_phi3_gguf_names_round_trip_and_serve(tmp_path, kind):
    """Per-head Q / K norms (attn_q_norm / attn_k_norm) and Phi-3's fused attn_qkv / stacked ffn_up survive export and
    loading, Gemma's norm tensors travel as 1 + gamma; the model served from the file agrees with transformers."""
    import torch

    transformers = pytest.importorskip("transformers")
    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import gguf as GG
    from antfly_b200.models.llama import StepBatch

    torch.manual_seed(0)
    common = dict(vocab_size=600, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=128, tie_word_embeddings=False)
    if kind == "qwen3":
        hf_cfg = transformers.Qwen3Config(**common, head_dim=32)
        hf = transformers.Qwen3ForCausalLM(hf_cfg).eval().float()
        with torch.no_grad():
            for n, p in hf.named_parameters():
                if n.endswith(("q_norm.weight", "k_norm.weight")):
                    p.uniform_(0.5, 1.5)
    elif kind.startswith("gemma"):
        extra = {"head_dim": 16, "hidden_activation": "gelu_pytorch_tanh"}
        if kind == "gemma":
            hf_cfg = transformers.GemmaConfig(**{**common, **extra})
            hf = transformers.GemmaForCausalLM(hf_cfg)
        elif kind == "gemma2":
            hf_cfg = transformers.Gemma2Config(**{**common, **extra, "query_pre_attn_scalar": 24, "sliding_window": 8,
                                                  "num_hidden_layers": 3, "attn_logit_softcapping": 4.0,
                                                  "final_logit_softcapping": 3.0})
            hf_cfg.tie_word_embeddings = False
            hf = transformers.Gemma2ForCausalLM(hf_cfg)
        else:
            hf_cfg = transformers.Gemma3TextConfig(**{**common, **extra, "query_pre_attn_scalar": 24,
                                                      "sliding_window": 8, "num_hidden_layers": 3,
                                                      "layer_types": ["sliding_attention", "full_attention",
                                                                      "sliding_attention"],
                                                      "rope_parameters": {
                                                          "sliding_attention": {"rope_type": "default",
                                                                                "rope_theta": 10000.0},
                                                          "full_attention": {"rope_type": "linear", "factor": 4.0,
                                                                             "rope_theta": 1000000.0}}})
            hf_cfg.tie_word_embeddings = False
            hf = transformers.Gemma3ForCausalLM(hf_cfg)
        hf = hf.eval().float()
        with torch.no_grad():
            for n, p in hf.named_parameters():
                if "norm" in n:
                    p.uniform_(-0.3, 0.3)
    else:
        hf_cfg = transformers.Phi3Config(**common, pad_token_id=0)
        hf = transformers.Phi3ForCausalLM(hf_cfg).eval().float()
    d = tmp_path / "generators" / kind
    d.mkdir(parents=True)
    GG.export_llama_gguf(str(d / "model.gguf"), hf.state_dict(), hf_cfg.to_dict(), quant="q8_0")
    f = GG.GGUFFile(str(d / "model.gguf"))
    if kind == "qwen3":
        assert "blk.0.attn_q_norm.weight" in f.tensors and "blk.1.attn_k_norm.weight" in f.tensors
        assert f.metadata["qwen3.attention.key_length"] == 32
    elif kind.startswith("gemma"):
        if kind != "gemma":
            assert "blk.0.post_attention_norm.weight" in f.tensors and "blk.2.post_ffw_norm.weight" in f.tensors
        stored = f.tensor("blk.0.attn_norm.weight")
        torch.testing.assert_close(stored, hf.state_dict()["model.layers.0.input_layernorm.weight"] + 1.0,
                                   atol=1e-6, rtol=0)
    else:
        assert "blk.0.attn_qkv.weight" in f.tensors and "blk.0.ffn_up.weight" in f.tensors
        assert GG.hf_name("blk.0.ffn_up.weight", "phi3") == "model.layers.0.mlp.gate_up_proj.weight"
        assert GG.hf_name("blk.0.ffn_up.weight", "llama") == "model.layers.0.mlp.up_proj.weight"
    ids = torch.randint(0, 600, (12,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    pos = torch.arange(12, dtype=torch.int32)
    for native in ((False, True) if kind == "qwen3" else (False,)):
        lm = ModelManager(models_dir=str(tmp_path), device="cpu", gguf_native=native).get(kind, "generator")
        model = lm.pipeline.engine.model
        assert lm.info.get("weights") == ("gguf-native" if native else lm.info.get("weights"))
        D = model.cfg.head_dim
        kc = torch.zeros((model.cfg.num_hidden_layers, 2, 16, 2, D), dtype=torch.bfloat16)
        b = StepBatch(ids.int(), pos, pos.clone(), i32([0]), i32([12]), i32([12]),
                      torch.arange(2, dtype=torch.int32)[None], pos.clone(), 12, 1)
        got = model.forward(b, kc, torch.zeros_like(kc)).float()
        cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
        assert float(cos.min()) > 0.99, (kind, native, cos)


@pytest.mark.parametrize("kind", ["mixtral", "qwen2_moe", "qwen3_moe"])
def test_mixture_of_experts_gguf_round_trip(tmp_path, kind):
    """Expert weights travel as one stacked tensor per projection (ffn_gate_exps / ffn_up_exps / ffn_down_exps), the
    router as ffn_gate_inp, a shared expert as *_shexp; Mixtral goes under the llama architecture with expert counts
    in the metadata.  The model loaded from the file agrees with transformers."""
    import torch

    transformers = pytest.importorskip("transformers")
    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import gguf as GG
    from antfly_b200.models.llama import StepBatch

    torch.manual_seed(0)
    common = dict(vocab_size=600, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=128, tie_word_embeddings=False)
    if kind == "mixtral":
        hf_cfg = transformers.MixtralConfig(**common, num_local_experts=4, num_experts_per_tok=2)
        hf = transformers.MixtralForCausalLM(hf_cfg)
    elif kind == "qwen2_moe":
        hf_cfg = transformers.Qwen2MoeConfig(**common, moe_intermediate_size=96, shared_expert_intermediate_size=160,
                                             num_experts=4, num_experts_per_tok=2, decoder_sparse_step=1,
                                             mlp_only_layers=[])
        hf = transformers.Qwen2MoeForCausalLM(hf_cfg)
    else:
        hf_cfg = transformers.Qwen3MoeConfig(**common, head_dim=32, moe_intermediate_size=96, num_experts=4,
                                             num_experts_per_tok=2, decoder_sparse_step=1, mlp_only_layers=[],
                                             norm_topk_prob=True)
        hf = transformers.Qwen3MoeForCausalLM(hf_cfg)
    hf = hf.eval().float()
    d = tmp_path / "generators" / kind
    d.mkdir(parents=True)
    GG.export_llama_gguf(str(d / "model.gguf"), hf.state_dict(), hf_cfg.to_dict(), quant="q8_0")
    f = GG.GGUFFile(str(d / "model.gguf"))
    arch = {"mixtral": "llama", "qwen2_moe": "qwen2moe", "qwen3_moe": "qwen3moe"}[kind]
    assert f.metadata["general.architecture"] == arch and f.metadata[f"{arch}.expert_count"] == 4
    F = 128 if kind == "mixtral" else 96
    assert tuple(f.tensors["blk.0.ffn_gate_exps.weight"].shape) == (4, F, 64)
    assert tuple(f.tensors["blk.1.ffn_down_exps.weight"].shape) == (4, 64, F)
    assert tuple(f.tensors["blk.0.ffn_gate_inp.weight"].shape) == (4, 64) and f.tensors["blk.0.ffn_gate_inp.weight"].type == 0
    assert ("blk.0.ffn_up_shexp.weight" in f.tensors) == (kind == "qwen2_moe")
    cfg_d = GG.llama_config_from_gguf(f.metadata)
    assert cfg_d["model_type"] == kind and cfg_d["num_experts"] == 4 and cfg_d["norm_topk_prob"] == (kind != "qwen2_moe")
    lm = ModelManager(models_dir=str(tmp_path), device="cpu").get(kind, "generator")
    model = lm.pipeline.engine.model
    assert model.cfg.num_experts == 4 and model.cfg.rope_half_split == (kind != "mixtral")
    ids = torch.randint(0, 600, (12,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    pos = torch.arange(12, dtype=torch.int32)
    kc = torch.zeros((2, 2, 16, 2, model.cfg.head_dim), dtype=torch.bfloat16)
    b = StepBatch(ids.int(), pos, pos.clone(), i32([0]), i32([12]), i32([12]), torch.arange(2, dtype=torch.int32)[None],
                  pos.clone(), 12, 1)
    got = model.forward(b, kc, torch.zeros_like(kc)).float()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.98, (kind, cos)


_QUANT_BOUNDS = {"q4_0": 0.12, "q4_1": 0.09, "q5_0": 0.06, "q5_1": 0.045, "q8_0": 0.008, "q8_1": 0.008, "q2_k": 0.40,
                 "q3_k": 0.20, "q4_k": 0.09, "q5_k": 0.045, "q6_k": 0.025, "q8_k": 0.012}


@pytest.mark.parametrize("name", sorted(_QUANT_BOUNDS))
def test_block_quantisers_round_trip_within_their_precision(name):
    """Every exported block type: the bytes decode identically through this package's decoder and the gguf
    package's (where it has one), the error against the source is within the type's precision, a block of zeros
    and a block of one repeated value survive, and a second quantisation of the decoded values is a fixed point for
    the symmetric 8-bit types."""
    import ctypes

    from antfly_b200 import _native as N
    from antfly_b200.formats import gguf as GG

    ty = GG.QUANT_NAMES[name]
    rng = np.random.default_rng(ty)
    x = (rng.standard_normal(256 * 24) * 0.7).astype(np.float32)
    x[:256] = 0.0
    x[256:512] = 0.375
    raw = GG.quantize(x, ty)
    lib = N.host()
    lib.afb_gguf_block_bytes.restype = ctypes.c_long
    assert raw.size == x.size // int(lib.afb_gguf_block_values(ty)) * int(lib.afb_gguf_block_bytes(ty))
    back = np.empty_like(x)
    assert lib.afb_gguf_dequantize(ctypes.c_int(ty), raw.ctypes.data_as(ctypes.c_void_p),
                                   back.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(x.size)) == 0
    tname = name.upper()
    if tname not in ("Q8_1", "Q8_K"):
        ref = gguf.quants.dequantize(raw, getattr(gguf.GGMLQuantizationType, tname)).reshape(-1)
        np.testing.assert_array_equal(ref, back)
    body = slice(512, None)
    err = np.sqrt(((back[body] - x[body]) ** 2).mean()) / np.sqrt((x[body] ** 2).mean())
    assert err < _QUANT_BOUNDS[name], (name, err)
    assert np.all(back[:256] == 0.0)
    assert np.abs(back[256:512] - 0.375).max() < (0.2 if name in ("q2_k", "q3_k") else 0.02)
    with pytest.raises(ValueError):
        GG.quantize(x[:100], ty)
    with pytest.raises(NotImplementedError):
        GG.quantize(x, 16)


def test_k_quant_export_is_served_from_its_blocks(tmp_path):
    """export --quant q6_k / q4_k on a checkpoint whose rows are whole super-blocks; the native GGUF path serves the
    file from those bytes and agrees with transformers."""
    import torch

    transformers = pytest.importorskip("transformers")
    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import gguf as GG
    from antfly_b200.models.llama import StepBatch
    from antfly_b200.ops.gguf_ops import GgufWeight

    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(vocab_size=320, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                      tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval().float()
    ids = torch.randint(0, 320, (10,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    for quant, ty, floor in (("q6_k", 14, 0.995), ("q4_k", 12, 0.97)):
        d = tmp_path / "generators" / quant
        d.mkdir(parents=True)
        counts = GG.export_llama_gguf(str(d / "model.gguf"), hf.state_dict(), hf_cfg.to_dict(), quant=quant)
        assert counts[ty] == 8                                  # seven projections and the output matrix
        lm = ModelManager(models_dir=str(tmp_path), device="cpu", gguf_native=True).get(quant, "generator")
        model = lm.pipeline.engine.model
        assert isinstance(model.w["l0.qkv"], GgufWeight) and model.w["l0.qkv"].segments[0][1] == ty
        i32 = lambda x: torch.tensor(x, dtype=torch.int32)
        pos = torch.arange(10, dtype=torch.int32)
        kc = torch.zeros((1, 2, 16, 2, 64), dtype=torch.bfloat16)
        b = StepBatch(ids.int(), pos, pos.clone(), i32([0]), i32([10]), i32([10]), torch.arange(2, dtype=torch.int32)[None],
                      pos.clone(), 10, 1)
        got = model.forward(b, kc, torch.zeros_like(kc)).float()
        cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
        assert float(cos.min()) > floor, (quant, cos)
