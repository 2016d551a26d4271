"""Gemma-4 text decoder against transformers' Gemma4ForCausalLM: per-layer embeddings, KV-shared layers, the two
attention geometries with proportional RoPE, K = V full-attention layers, the MoE block, double-wide MLP, soft cap."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf(**over):
    torch.manual_seed(0)
    kw = dict(vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=6, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=8, vocab_size_per_layer_input=200,
              hidden_size_per_layer_input=8, num_kv_shared_layers=2, final_logit_softcapping=30.0,
              layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2, max_position_embeddings=128,
              tie_word_embeddings=True)
    kw.update(over)
    cfg = transformers.Gemma4TextConfig(**kw)
    m = transformers.Gemma4ForCausalLM(cfg).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n or "scale" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in m.named_buffers():
            if n.endswith("layer_scalar"):
                b.fill_(0.9)
    return cfg, m


CASES = {
    "ple_shared_kv": {},
    "k_eq_v_global_heads": dict(attention_k_eq_v=True, num_global_key_value_heads=1, num_kv_shared_layers=0),
    "moe_double_wide": dict(enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=48,
                            use_double_wide_mlp=True),
    "no_ple": dict(hidden_size_per_layer_input=0, num_kv_shared_layers=0, final_logit_softcapping=None),
}


@pytest.mark.parametrize("name", list(CASES))
def test_gemma4_text_logits_and_cached_decoding_match_transformers(name):
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel

    hf_cfg, hf = _hf(**CASES[name])
    cfg = Gemma4Config.from_hf(hf_cfg.to_dict())
    model = Gemma4TextModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    ids = torch.randint(1, 200, (1, 21), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids).logits[0]
    got, st = model.forward(ids[0])
    torch.testing.assert_close(got, want, atol=3e-4, rtol=3e-3)
    more = torch.randint(1, 200, (1, 4), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want2 = hf(torch.cat([ids, more], 1)).logits[0, 21:]
    got2 = []
    for t in range(4):
        lg, st = model.forward(more[0, t:t + 1], st)
        got2.append(lg[0])
    torch.testing.assert_close(torch.stack(got2), want2, atol=5e-4, rtol=5e-3)


def test_kv_shared_layers_keep_no_cache_of_their_own():
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel

    hf_cfg, hf = _hf()
    model = Gemma4TextModel.from_state_dict(Gemma4Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                            dtype=torch.float32)
    assert model.kv_source == {0: 0, 1: 1, 2: 2, 3: 3, 4: 3, 5: 2}
    _, st = model.forward(torch.tensor([3, 4, 5, 6]))
    assert sorted(st.kv) == [0, 1, 2, 3]


@pytest.mark.parametrize("clipped,standardize", [(False, False), (True, True)])
def test_gemma4_vision_tower_and_projector_match_transformers(clipped, standardize):
    from transformers.models.gemma4 import modeling_gemma4 as M

    from antfly_b200.models.gemma4v import Gemma4Projector, Gemma4VisionConfig, Gemma4VisionTower

    torch.manual_seed(0)
    vcfg = transformers.Gemma4VisionConfig(hidden_size=48, intermediate_size=96, num_hidden_layers=2,
                                           num_attention_heads=3, num_key_value_heads=3, head_dim=16, patch_size=4,
                                           pooling_kernel_size=2, position_embedding_size=32,
                                           use_clipped_linears=clipped, standardize=standardize)
    tcfg = transformers.Gemma4TextConfig(vocab_size=50, hidden_size=40, intermediate_size=64, num_hidden_layers=2,
                                         num_attention_heads=2, num_key_value_heads=1, head_dim=16, global_head_dim=16,
                                         hidden_size_per_layer_input=0, layer_types=["sliding_attention", "full_attention"])
    hf = M.Gemma4VisionModel(vcfg).eval().float()
    emb = M.Gemma4MultimodalEmbedder(vcfg, tcfg).eval().float()
    with torch.no_grad():
        hf.patch_embedder.position_embedding_table.normal_(0, 0.5)
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
        if clipped:
            for n, b in hf.named_buffers():
                if n.endswith(("input_max", "output_max")):
                    b.fill_(1.5)
                if n.endswith(("input_min", "output_min")):
                    b.fill_(-1.5)
        if standardize:
            hf.std_bias.normal_(0, 0.1)
            hf.std_scale.uniform_(0.5, 1.5)
    # two images: 4 x 4 patches and 4 x 2 patches (padded to 16)
    def grid(wd, ht):
        ys, xs = torch.meshgrid(torch.arange(ht), torch.arange(wd), indexing="ij")
        return torch.stack([xs.flatten(), ys.flatten()], -1)
    P = 16
    pos = torch.full((2, P, 2), -1)
    pos[0] = grid(4, 4)
    pos[1, :8] = grid(4, 2)
    pix = torch.rand(2, P, 3 * 16)
    pix[1, 8:] = 0
    with torch.no_grad():
        want = hf(pixel_values=pix, pixel_position_ids=pos).last_hidden_state
        want_proj = emb(want)
    cfg = Gemma4VisionConfig.from_hf(vcfg.to_dict())
    tower = Gemma4VisionTower.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    got = tower.forward(pix, pos)
    assert got.shape == want.shape == (4 + 2, 48)
    torch.testing.assert_close(got, want, atol=3e-4, rtol=3e-3)
    proj = Gemma4Projector(emb.embedding_projection.weight.detach().float(), vcfg.rms_norm_eps)
    torch.testing.assert_close(proj.forward(got), want_proj, atol=3e-4, rtol=3e-3)


@pytest.mark.parametrize("bidir", [None, "vision"])
def test_gemma4_image_prompt_matches_transformers(bidir):
    """Image placeholders take the projected soft tokens and the padding token's per-layer embedding; with
    ``use_bidirectional_attention = "vision"`` an image's tokens see each other in the sliding-window layers."""
    from transformers.models.gemma4 import modeling_gemma4 as M

    from antfly_b200.models.gemma4v import Gemma4Multimodal

    torch.manual_seed(0)
    v = transformers.Gemma4VisionConfig(hidden_size=48, intermediate_size=96, num_hidden_layers=2,
                                        num_attention_heads=3, num_key_value_heads=3, head_dim=16, patch_size=4,
                                        pooling_kernel_size=2, position_embedding_size=32)
    t = transformers.Gemma4TextConfig(vocab_size=120, hidden_size=40, intermediate_size=64, num_hidden_layers=3,
                                      num_attention_heads=2, num_key_value_heads=1, head_dim=16, global_head_dim=16,
                                      hidden_size_per_layer_input=8, vocab_size_per_layer_input=120, sliding_window=6,
                                      use_bidirectional_attention=bidir, pad_token_id=0,
                                      layer_types=["sliding_attention", "sliding_attention", "full_attention"])
    c = transformers.Gemma4Config(text_config=t, vision_config=v, audio_config=None, image_token_id=100)
    hf = M.Gemma4ForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        hf.model.vision_tower.patch_embedder.position_embedding_table.normal_(0, 0.5)
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)

    def grid(wd, ht):
        ys, xs = torch.meshgrid(torch.arange(ht), torch.arange(wd), indexing="ij")
        return torch.stack([xs.flatten(), ys.flatten()], -1)
    P = 16
    pos = torch.full((2, P, 2), -1)
    pos[0] = grid(4, 4)
    pos[1, :8] = grid(4, 2)
    pix = torch.rand(2, P, 3 * 16)
    pix[1, 8:] = 0
    ids = torch.tensor([[5, 6, 100, 100, 100, 100, 7, 8, 9, 100, 100, 10, 11, 12, 13, 14]])
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pix, image_position_ids=pos,
                  mm_token_type_ids=(ids == 100).long()).logits[0]
    model = Gemma4Multimodal.from_state_dict(c.to_dict(), hf.state_dict(), device="cpu", dtype=torch.float32)
    assert model.bidirectional_vision == (bidir == "vision")
    assert model.vision_groups(ids[0]).tolist() == [-1, -1, 0, 0, 0, 0, -1, -1, -1, 1, 1, -1, -1, -1, -1, -1]
    got, st = model.forward(ids[0], None, pix, pos)
    torch.testing.assert_close(got, want, atol=3e-4, rtol=3e-3)
    # text-only continuation after the image prompt
    nxt = torch.tensor([[20]])
    with torch.no_grad():
        full = torch.cat([ids, nxt], 1)
        want2 = hf(input_ids=full, pixel_values=pix, image_position_ids=pos,
                   mm_token_type_ids=(full == 100).long()).logits[0, -1]
    got2, _ = model.forward(nxt[0], st)
    torch.testing.assert_close(got2[0], want2, atol=5e-4, rtol=5e-3)


@pytest.mark.parametrize("hw", [(200, 333), (48, 48), (30, 900), (1000, 700)])
def test_gemma4_image_patches_match_the_transformers_processor(hw):
    import numpy as np
    from transformers.models.gemma4.image_processing_pil_gemma4 import Gemma4ImageProcessorPil

    from antfly_b200.models.gemma4v import gemma4_patches

    img = np.random.default_rng(hw[0]).integers(0, 256, size=(*hw, 3), dtype=np.uint8)
    for max_soft in (70, 280):
        want = Gemma4ImageProcessorPil(max_soft_tokens=max_soft).preprocess([img], return_tensors="pt")
        rows, pos, n = gemma4_patches(torch.from_numpy(img), 16, max_soft, 3)
        assert n == int(want["num_soft_tokens_per_image"][0])
        assert torch.equal(pos, want["image_position_ids"][0])
        # Pillow's bicubic and torch's antialiased bicubic differ by a few 8-bit steps on random noise
        diff = (rows - want["pixel_values"][0]).abs()
        assert rows.shape == want["pixel_values"][0].shape and float(diff.mean()) < 0.02, float(diff.mean())


def test_gemma4_loads_through_the_model_manager_and_answers_about_an_image(tmp_path):
    import json

    import numpy as np
    from transformers.models.gemma4 import modeling_gemma4 as M

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import safetensors_io as st
    from antfly_b200.models.gemma4v import gemma4_patches
    from antfly_b200.runtime.sampling_params import SamplingParams

    torch.manual_seed(0)
    v = transformers.Gemma4VisionConfig(hidden_size=48, intermediate_size=96, num_hidden_layers=1,
                                        num_attention_heads=3, num_key_value_heads=3, head_dim=16, patch_size=4,
                                        pooling_kernel_size=2, position_embedding_size=64)
    t = transformers.Gemma4TextConfig(vocab_size=600, hidden_size=40, intermediate_size=64, num_hidden_layers=2,
                                      num_attention_heads=2, num_key_value_heads=1, head_dim=16, global_head_dim=16,
                                      hidden_size_per_layer_input=8, vocab_size_per_layer_input=600, sliding_window=16,
                                      pad_token_id=0, layer_types=["sliding_attention", "full_attention"])
    c = transformers.Gemma4Config(text_config=t, vision_config=v, audio_config=None, image_token_id=590,
                                  boi_token_id=591, eoi_token_id=592)
    hf = M.Gemma4ForConditionalGeneration(c).eval().float()
    d = tmp_path / "generators" / "tiny-gemma4"
    d.mkdir(parents=True)
    st.save_file({k: v_.contiguous() for k, v_ in hf.state_dict().items()}, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(c.to_dict(), default=str))
    (d / "preprocessor_config.json").write_text(json.dumps({"max_soft_tokens": 70, "patch_size": 4}))
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")
    pipe = mgr.get("tiny-gemma4", "generator").pipeline
    img = torch.from_numpy(np.random.default_rng(0).integers(0, 256, size=(40, 64, 3), dtype=np.uint8))
    out = pipe.generate("what is this", SamplingParams(max_tokens=5, ignore_eos=True), raw_prompt=True, images=[img])
    # the same prompt through transformers: begin marker, soft-token placeholders, end marker, then the text
    rows, pos, n = gemma4_patches(img, 4, 70, 2)
    text_ids = pipe.tokenizer.encode_prompt("what is this", add_bos=True)
    at = 1 if text_ids[0] == pipe.tokenizer.special.bos_id else 0
    ids = text_ids[:at] + [591] + [590] * n + [592] + text_ids[at:]
    assert out.prompt_tokens == len(ids)
    seq = torch.tensor([ids])
    want = []
    for _ in range(5):
        with torch.no_grad():
            lg = hf(input_ids=seq, pixel_values=rows[None], image_position_ids=pos[None],
                    mm_token_type_ids=(seq == 590).long()).logits[0, -1]
        want.append(int(lg.argmax()))
        seq = torch.cat([seq, torch.tensor([[want[-1]]])], 1)
    assert out.token_ids == want
