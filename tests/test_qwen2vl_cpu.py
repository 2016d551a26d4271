"""Qwen2-VL vision tower, image patching and rotary position streams against the Hugging Face implementation."""
import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models import qwen2vl as QV


def _hf(seed=0):
    torch.manual_seed(seed)
    cfg = transformers.Qwen2VLConfig(
        text_config=dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-5,
                         rope_theta=10000.0, tie_word_embeddings=False, attention_dropout=0.0,
                         rope_scaling={"type": "mrope", "mrope_section": [4, 6, 6]}),
        vision_config=dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, mlp_ratio=2, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3),
        image_token_id=300, video_token_id=301, vision_start_token_id=302, vision_end_token_id=303)
    hf = transformers.Qwen2VLForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
            elif "norm" in n or "ln_q" in n:
                p.uniform_(0.5, 1.5)
    return cfg, hf


def test_vision_tower_matches_transformers():
    hf_cfg, hf = _hf()
    vc = QV.Qwen2VLVisionConfig.from_hf(hf_cfg.vision_config.to_dict())
    assert vc.depth == 2 and vc.embed_dim == 64 and vc.hidden_size == 128
    model = QV.Qwen2VLVisionModel.from_state_dict(vc, hf.state_dict(), device="cpu", dtype=torch.float32)
    grids = [(1, 4, 6), (1, 2, 2)]
    n = sum(t * h * w for t, h, w in grids)
    patches = torch.randn(n, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf.model.visual(patches, grid_thw=torch.tensor(grids)).pooler_output
    got = model.forward(patches, grids).float()
    assert got.shape == want.shape == (n // 4, 128)
    assert float(torch.nn.functional.cosine_similarity(got, want, dim=-1).min()) > 0.999
    torch.testing.assert_close(got, want, atol=5e-2, rtol=5e-2)


def test_image_patching_matches_image_processor():
    proc = transformers.Qwen2VLImageProcessor(min_pixels=56 * 56, max_pixels=28 * 28 * 64)
    rng = np.random.default_rng(0)
    vc = QV.Qwen2VLVisionConfig()
    for hw in ((84, 112), (100, 230), (40, 40), (700, 500)):
        img = rng.integers(0, 256, size=(*hw, 3), dtype=np.uint8)
        want = proc(images=[img], return_tensors="pt")
        got, grid = QV.image_to_patches(torch.from_numpy(img), vc, 56 * 56, 28 * 28 * 64)
        assert list(grid) == want["image_grid_thw"][0].tolist(), hw
        assert got.shape == want["pixel_values"].shape
        if hw == (84, 112):                       # already a multiple of 28: no resampling, exact agreement
            torch.testing.assert_close(got, want["pixel_values"].float(), atol=1e-5, rtol=1e-5)
        else:                                     # resampling filters differ slightly between libraries
            assert float((got - want["pixel_values"].float()).abs().mean()) < 0.05


def test_rope_index_and_rotation_match_transformers():
    hf_cfg, hf = _hf()
    IMG = 300
    grids = [(1, 4, 6), (1, 2, 4)]
    ids = [5, 6, 302] + [IMG] * 6 + [303, 7, 8, 9, 302] + [IMG] * 2 + [303, 10, 11]
    res = hf.model.get_rope_index(torch.tensor([ids]), torch.tensor([[int(t == IMG) for t in ids]]),
                                  image_grid_thw=torch.tensor(grids),
                                  attention_mask=torch.ones(1, len(ids), dtype=torch.long))
    want_pos, want_delta = res[0][:, 0], int(res[1].flatten()[0])
    pos, delta = QV.rope_index(ids, grids, IMG)
    assert torch.equal(pos, want_pos) and delta == want_delta
    assert QV.rope_index([1, 2, 3], [], IMG)[1] == 0
    with pytest.raises(ValueError):
        QV.rope_index([IMG] * 3, [(1, 4, 6)], IMG)
    # rotation against the library's multimodal rotary function
    from transformers.models.qwen2_vl import modeling_qwen2_vl as M

    rot = M.Qwen2VLRotaryEmbedding(hf_cfg.text_config)
    x = torch.randn(len(ids), 4, 32, generator=torch.Generator().manual_seed(3))
    cos, sin = rot(x, pos[:, None, :])
    q = x.transpose(0, 1)[None]
    want_q, _ = M.apply_multimodal_rotary_pos_emb(q, q, cos, sin, [4, 6, 6])
    got = QV.mrope_rotate(x, pos, 10000.0, [4, 6, 6])
    torch.testing.assert_close(got, want_q[0].transpose(0, 1), atol=1e-5, rtol=1e-5)
