"""BitNet b1.58 decoder against the Hugging Face model whose projections are swapped for a plain restatement of the
quantised linear (8-bit activations per token, ternary weights with one scale), from full-precision and from
packed 2-bit checkpoints."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch, bitnet_ternary


class QLinear(torch.nn.Linear):
    def forward(self, x):
        w = self.weight.float()
        m = w.abs().mean().clamp(min=1e-5)
        wq = (w / m).round().clamp(-1, 1) * m
        s = 127.0 / x.float().abs().amax(-1, keepdim=True).clamp(min=1e-5)
        xq = (x.float() * s).round().clamp(-128, 127) / s
        return torch.nn.functional.linear(xq, wq)


def _hf():
    torch.manual_seed(0)
    cfg = transformers.BitNetConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                    rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True,
                                    attention_dropout=0.0)
    hf = transformers.BitNetForCausalLM(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.uniform_(0.5, 1.5)
    for layer in hf.model.layers:
        for parent, names in ((layer.self_attn, ("q_proj", "k_proj", "v_proj", "o_proj")),
                              (layer.mlp, ("gate_proj", "up_proj", "down_proj"))):
            for n in names:
                old = getattr(parent, n)
                new = QLinear(old.in_features, old.out_features, bias=False)
                new.weight = old.weight
                setattr(parent, n, new)
    # the tied embedding / output matrix is kept in block-fp8 like every other model's
    from antfly_b200.ops import reference as R
    with torch.no_grad():
        q, e8 = R.quantize_block_fp8(hf.model.embed_tokens.weight.data)
        hf.model.embed_tokens.weight.data.copy_(R.dequantize_block_fp8(q, e8))
    return cfg, hf


def _run(model, cfg, ids, S, device="cpu"):
    page, nblk = 16, 3
    k_cache = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16,
                          device=device)
    v_cache = torch.zeros_like(k_cache)
    table = torch.arange(nblk, dtype=torch.int32, device=device)[None]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    pos = torch.arange(S, dtype=torch.int32, device=device)
    prefill = StepBatch(ids[:S].int(), pos, pos.clone(), i32([0]), i32([S]), i32([S]), table, pos.clone(), S, 1)
    a = model.forward(prefill, k_cache, v_cache).float()
    decode = StepBatch(ids[S:].int(), i32([S]), i32([S]), i32([0]), i32([1]), i32([S + 1]), table, i32([0]), 1, 1)
    return torch.cat([a, model.forward(decode, k_cache, v_cache).float()], 0)


@pytest.mark.parametrize("packed", [False, True])
def test_bitnet_matches_transformers(packed):
    hf_cfg, hf = _hf()
    d = hf_cfg.to_dict()
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    sd.pop("lm_head.weight", None)
    if packed:
        # the released layout: 2-bit codes, four output rows per byte, and the scale beside them
        d["quantization_config"] = {"quant_method": "bitnet", "linear_class": "autobitlinear",
                                    "quantization_mode": "offline"}
        for k in [k for k in sd if k.endswith("_proj.weight")]:
            t, m = bitnet_ternary(sd[k], None, False)
            codes = (t + 1).to(torch.uint8)
            R_ = codes.shape[0] // 4
            sd[k] = sum(codes[i * R_:(i + 1) * R_] << (2 * i) for i in range(4)).to(torch.uint8)
            sd[k.replace(".weight", ".weight_scale")] = torch.tensor([m])
    cfg = LlamaConfig.from_hf(d)
    assert cfg.bitnet and cfg.gate_act == "relu2" and cfg.tie_word_embeddings and not cfg.bitnet_scale_divides
    model = LlamaModel.from_state_dict(cfg, sd, device="cpu")
    S = 24
    ids = torch.randint(0, hf_cfg.vocab_size, (S + 1,), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = hf(ids[None]).logits[0].float()
    got = _run(model, cfg, ids, S)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.99, cos
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.8
    assert float((got - want).abs().max()) < 0.08 * max(float(want.abs().max()), 1.0)


def test_bitnet_ternary_unpacking_and_scale_conventions():
    t = torch.tensor([[1., -1.], [0., 1.], [-1., 0.], [1., 1.], [0., 0.], [-1., -1.], [1., 0.], [0., -1.]])
    codes = (t + 1).to(torch.uint8)
    packed = sum(codes[i * 2:(i + 1) * 2] << (2 * i) for i in range(4)).to(torch.uint8)
    got, sc = bitnet_ternary(packed, torch.tensor([0.25]), False)
    assert torch.equal(got, t) and sc == 0.25
    assert bitnet_ternary(packed, torch.tensor([0.25]), True)[1] == 4.0
    w = torch.tensor([[0.9, -0.05, 0.4], [-1.2, 0.6, 0.0]])
    tq, m = bitnet_ternary(w, None, False)
    assert abs(m - float(w.abs().mean())) < 1e-7 and set(tq.flatten().tolist()) <= {-1.0, 0.0, 1.0}
    assert tq.tolist() == [[1.0, -0.0, 1.0], [-1.0, 1.0, 0.0]]


def test_bitnet_gguf_names_config_and_decoded_weights(tmp_path):
    """A BitNet GGUF file: I2_S projections decode to ternary-times-scale matrices, which load with that scale
    (not a re-estimated one); the sub-norm tensors and the architecture key map to the model's names."""
    from antfly_b200.formats import gguf as GG

    assert GG.hf_name("blk.3.attn_sub_norm.weight") == "model.layers.3.self_attn.attn_sub_norm.weight"
    assert GG.hf_name("blk.0.ffn_sub_norm.weight") == "model.layers.0.mlp.ffn_sub_norm.weight"
    md = {"general.architecture": "bitnet-b1.58", "bitnet-b1.58.block_count": 2, "bitnet-b1.58.embedding_length": 128,
          "bitnet-b1.58.feed_forward_length": 256, "bitnet-b1.58.attention.head_count": 4,
          "bitnet-b1.58.attention.head_count_kv": 2, "bitnet-b1.58.vocab_size": 320}
    d = GG.llama_config_from_gguf(md)
    cfg = LlamaConfig.from_hf({k: v for k, v in d.items() if v is not None})
    assert cfg.bitnet and cfg.hidden_size == 128 and cfg.num_key_value_heads == 2 and cfg.tie_word_embeddings
    w = torch.randn(8, 128, generator=torch.Generator().manual_seed(2))
    path = str(tmp_path / "w.gguf")
    GG.write_gguf(path, md, {"blk.0.attn_q.weight": (36, w)})
    dec = GG.GGUFFile(path).tensor("blk.0.attn_q.weight")
    t, sc = bitnet_ternary(dec, None, False)
    m = float(w.abs().mean())
    assert abs(sc - m) < 1e-6 and torch.equal(t, (w / m).round().clamp(-1, 1))


def test_bitnet_gguf_export_round_trip(tmp_path):
    """Export the tiny BitNet to GGUF with ternary (I2_S) projections, read it back through the name / config
    mapping, and get the same logits as from the original weights."""
    from antfly_b200.formats import gguf as GG

    hf_cfg, hf = _hf()
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    sd.pop("lm_head.weight", None)
    d = hf_cfg.to_dict()
    path = str(tmp_path / "bitnet.gguf")
    counts = GG.export_llama_gguf(path, sd, d, quant="i2_s")
    assert counts[36] == 2 * 7                                   # seven projections per layer, two layers
    f = GG.GGUFFile(path)
    back = {GG.hf_name(n): f.tensor(n) for n in f.tensors}
    assert "model.layers.0.self_attn.attn_sub_norm.weight" in back
    cfg_d = {k: v for k, v in GG.llama_config_from_gguf(f.metadata).items() if v is not None}
    cfg = LlamaConfig.from_hf(cfg_d)
    assert cfg.bitnet and cfg.num_hidden_layers == 2 and cfg.gate_act == "relu2"
    ids = torch.randint(0, hf_cfg.vocab_size, (25,), generator=torch.Generator().manual_seed(5))
    want = _run(LlamaModel.from_state_dict(LlamaConfig.from_hf(d), dict(sd), device="cpu"), cfg, ids, 24)
    got = _run(LlamaModel.from_state_dict(cfg, back, device="cpu"), cfg, ids, 24)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.999, cos                         # embeddings / norms went through fp16
