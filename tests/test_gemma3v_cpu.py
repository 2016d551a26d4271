"""Gemma-3 image path against Hugging Face: vision tower + projector, and the decoder over a prompt with an image
(soft tokens, image tokens attending in both directions)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models.gemma3v import Gemma3VisionModel, SiglipVisionConfig, gemma3_pixels


def _hf(seed=0):
    torch.manual_seed(seed)
    cfg = transformers.Gemma3Config(
        text_config=dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=3,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, query_pre_attn_scalar=48,
                         sliding_window=6, max_position_embeddings=256, rms_norm_eps=1e-6,
                         layer_types=["sliding_attention", "full_attention", "sliding_attention"],
                         rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                          "full_attention": {"rope_type": "default", "rope_theta": 1000000.0}}),
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                           image_size=56, patch_size=14, num_channels=3),
        mm_tokens_per_image=4, image_token_index=300, boi_token_index=301, eoi_token_index=302)
    hf = transformers.Gemma3ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
            elif "norm" in n and "vision" not in n:
                p.uniform_(-0.3, 0.3)
            elif n.endswith("mm_input_projection_weight"):        # created as zeros
                p.normal_(0, 0.1)
    return cfg, hf


def test_vision_tower_and_projector_match_transformers():
    hf_cfg, hf = _hf()
    vc = SiglipVisionConfig.from_hf(hf_cfg.vision_config.to_dict())
    model = Gemma3VisionModel.from_state_dict(vc, hf.state_dict(), device="cpu", dtype=torch.float32,
                                              tokens_per_image=4)
    px = torch.randn(2, 3, 56, 56, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf.model.get_image_features(px)
    want = getattr(want, "pooler_output", want)
    got = model.soft_tokens(px).float()
    assert got.shape == tuple(want.shape) == (2, 4, 128)
    assert float(torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)) > 0.999
    torch.testing.assert_close(got, want.float(), atol=5e-2, rtol=5e-2)
    img = torch.randint(0, 256, (30, 80, 3), generator=torch.Generator().manual_seed(2), dtype=torch.uint8)
    p = gemma3_pixels(img, 56)
    assert p.shape == (3, 56, 56) and -1.0 <= float(p.min()) and float(p.max()) <= 1.0


def test_decoder_with_image_matches_transformers_and_engine():
    from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch
    from antfly_b200.models.qwen2vl import text_state_dict
    from antfly_b200.ops import reference as R
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    hf_cfg, hf = _hf(1)
    with torch.no_grad():
        for name, mod in hf.named_modules():
            if isinstance(mod, torch.nn.Linear) and "vision" not in name and "projector" not in name:
                q, e8 = R.quantize_block_fp8(mod.weight.data)
                mod.weight.data.copy_(R.dequantize_block_fp8(q, e8))
    IMG = 300
    ids = [2, 5, 6, 301] + [IMG] * 4 + [302, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16]
    S = len(ids) - 1
    px = torch.randn(1, 3, 56, 56, generator=torch.Generator().manual_seed(3))
    tt = torch.tensor([[int(t == IMG) for t in ids]])
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=px, token_type_ids=tt).logits[0].float()
        causal_only = hf(input_ids=torch.tensor([ids]), pixel_values=px, token_type_ids=torch.zeros_like(tt)).logits[0]
    assert float((want - causal_only).abs().max()) > 1e-3        # the two-way image attention changes the outputs

    sd = hf.state_dict()
    cfg = LlamaConfig.from_hf(hf_cfg.text_config.to_dict())
    assert cfg.post_norms and cfg.layer_windows == [6, 0, 6]
    model = LlamaModel.from_state_dict(cfg, text_state_dict(sd), device="cpu")
    vision = Gemma3VisionModel.from_state_dict(SiglipVisionConfig.from_hf(hf_cfg.vision_config.to_dict()), sd,
                                               device="cpu", dtype=torch.float32, tokens_per_image=4)
    soft = vision.soft_tokens(px)[0]
    page, nblk = 16, 3
    kc = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    table = torch.arange(nblk, dtype=torch.int32)[None]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    idx = torch.arange(S, dtype=torch.int32)
    rows = torch.tensor([4, 5, 6, 7])
    b = StepBatch(i32(ids[:S]), idx, idx.clone(), i32([0]), i32([S]), i32([S]), table, idx.clone(), S, 1,
                  embed_rows=rows, embed_vals=soft, bidir=(i32([4]), i32([4]), i32([8]), table, 4, rows))
    a = model.forward(b, kc, vc).float()
    d = StepBatch(i32(ids[S:]), i32([S]), i32([S]), i32([0]), i32([1]), i32([S + 1]), table, i32([0]), 1, 1)
    got = torch.cat([a, model.forward(d, kc, vc).float()], 0)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.99, cos
    assert float((got - want).abs().max()) < 0.08 * max(float(want.abs().max()), 1.0)

    # engine: the prompt is prefilled whole although the chunk size is smaller than it
    sp = SamplingParams(max_tokens=3, temperature=0.0)
    eng = LLMEngine(model, num_blocks=16, max_batch=2, use_cuda_graph=False, prefill_chunk=8, max_step_tokens=64)
    desc = {"rows": [4, 5, 6, 7], "vals": soft, "bidir": [(4, 8)]}
    out = eng.generate([ids[:S]], sp, soft=[desc])[0].token_ids
    assert out[0] == int(a[-1].argmax())
    assert eng.sched.stats()["step_prefill_items_total"] == 1       # one prefill item: no chunking


def test_gemma3_adapter_expands_placeholders():
    from antfly_b200.pipelines.vlm import Gemma3Adapter

    hf_cfg, hf = _hf(2)
    vision = Gemma3VisionModel.from_state_dict(SiglipVisionConfig.from_hf(hf_cfg.vision_config.to_dict()),
                                               hf.state_dict(), device="cpu", dtype=torch.float32, tokens_per_image=4)
    ad = Gemma3Adapter(vision, 300, 301, 302, newline_ids=[9, 9])
    img = torch.randint(0, 256, (40, 70, 3), generator=torch.Generator().manual_seed(0), dtype=torch.uint8)
    ids, soft = ad.expand([2, 301, 5, 301, 6], [img, img])
    assert ids == [2, 9, 9, 301, 300, 300, 300, 300, 302, 9, 9, 5, 9, 9, 301, 300, 300, 300, 300, 302, 9, 9, 6]
    assert soft["bidir"] == [(4, 8), (15, 19)] and soft["rows"] == [4, 5, 6, 7, 15, 16, 17, 18]
    assert soft["vals"].shape == (8, 128) and torch.equal(soft["vals"][:4].float(), soft["vals"][4:].float())
    assert ad.expand([2, 5], []) == ([2, 5], None)
    with pytest.raises(ValueError):
        ad.expand([2, 301], [])
    with pytest.raises(ValueError):
        ad.expand([2, 301], [img, img])
