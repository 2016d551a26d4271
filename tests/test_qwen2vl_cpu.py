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


def _round_text_linears(hf):
    from antfly_b200.ops import reference as R

    with torch.no_grad():
        for name, mod in hf.named_modules():
            if isinstance(mod, torch.nn.Linear) and "visual" not in name:
                q, e8 = R.quantize_block_fp8(mod.weight.data)
                mod.weight.data.copy_(R.dequantize_block_fp8(q, e8))


def test_decoder_with_image_tokens_matches_transformers():
    """Prefill over text + image placeholders (soft tokens, three-stream rotary positions) and one decode step whose
    rotary position runs behind its cache index."""
    from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch

    hf_cfg, hf = _hf(1)
    _round_text_linears(hf)
    IMG = 300
    grids = [(1, 4, 6), (1, 2, 4)]
    ids = [5, 6, 302] + [IMG] * 6 + [303, 7, 8, 9, 302] + [IMG] * 2 + [303, 10, 11, 12]
    S = len(ids) - 1
    n_patches = sum(t * h * w for t, h, w in grids)
    patches = torch.randn(n_patches, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor(grids),
                  mm_token_type_ids=torch.tensor([[int(t == IMG) for t in ids]])).logits[0].float()

    d = hf_cfg.text_config.to_dict()
    cfg = LlamaConfig.from_hf(d)
    assert cfg.mrope_sections == [4, 6, 6] and cfg.qkv_bias
    sd = hf.state_dict()
    model = LlamaModel.from_state_dict(cfg, QV.text_state_dict(sd), device="cpu")
    vision = QV.Qwen2VLVisionModel.from_state_dict(QV.Qwen2VLVisionConfig.from_hf(hf_cfg.vision_config.to_dict()), sd,
                                                   device="cpu", dtype=torch.float32)
    soft = vision.forward(patches, grids)
    pos3, delta = QV.rope_index(ids[:S], grids, IMG)
    assert delta < 0 and soft.shape[0] == ids.count(IMG)

    page, nblk = 16, 3
    k_cache = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    table = torch.arange(nblk, dtype=torch.int32)[None]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    idx = torch.arange(S, dtype=torch.int32)
    rows = torch.tensor([i for i, t in enumerate(ids[:S]) if t == IMG])
    prefill = StepBatch(i32(ids[:S]), idx, idx.clone(), i32([0]), i32([S]), i32([S]), table, idx.clone(), S, 1,
                        embed_rows=rows, embed_vals=soft, pos3=pos3)
    a = model.forward(prefill, k_cache, v_cache).float()
    decode = StepBatch(i32(ids[S:]), i32([S + delta]), i32([S]), i32([0]), i32([1]), i32([S + 1]), table, i32([0]), 1, 1)
    got = torch.cat([a, model.forward(decode, k_cache, v_cache).float()], 0)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.99, cos
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.8
    assert float((got - want).abs().max()) < 0.08 * max(float(want.abs().max()), 1.0)


def test_engine_generates_from_image_prompts():
    """The adapter widens placeholders and describes the soft tokens; the engine prefills in chunks that cut through
    the image, decodes with the rotary delta, and serves a text request in the same steps.  Greedy tokens must
    equal a straight run of the model (one prefill over the whole prompt, then single-token steps)."""
    from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch
    from antfly_b200.pipelines.vlm import Qwen2VLAdapter, VlmTokens, split_content
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    hf_cfg, hf = _hf(2)
    sd = hf.state_dict()
    cfg = LlamaConfig.from_hf(hf_cfg.text_config.to_dict())
    model = LlamaModel.from_state_dict(cfg, QV.text_state_dict(sd), device="cpu")
    vision = QV.Qwen2VLVisionModel.from_state_dict(QV.Qwen2VLVisionConfig.from_hf(hf_cfg.vision_config.to_dict()), sd,
                                                   device="cpu", dtype=torch.float32)
    adapter = Qwen2VLAdapter(vision, VlmTokens(300, 302, 303), min_pixels=28 * 28, max_pixels=28 * 28 * 16)
    img = torch.randint(0, 256, (60, 110, 3), generator=torch.Generator().manual_seed(7), dtype=torch.uint8)
    prompt = [5, 6, 302, 300, 303, 7, 8, 9]
    ids, soft = adapter.expand(prompt, [img])
    n_img = ids.count(300)
    assert n_img == soft["vals"].shape[0] == len(soft["rows"]) and n_img > 1 and soft["delta"] < 0
    assert adapter.expand([1, 2], []) == ([1, 2], None)
    with pytest.raises(ValueError):
        adapter.expand(prompt, [])
    with pytest.raises(ValueError):
        adapter.expand([1, 2], [img])

    # straight run
    N_NEW = 5
    page, nblk = 16, 8
    k_cache = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    table = torch.arange(nblk, dtype=torch.int32)[None]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    S = len(ids)
    idx = torch.arange(S, dtype=torch.int32)
    b = StepBatch(i32(ids), idx, idx.clone(), i32([0]), i32([S]), i32([S]), table, i32([S - 1]), S, 1,
                  embed_rows=torch.tensor(soft["rows"]), embed_vals=soft["vals"], pos3=soft["pos3"])
    want = [int(model.forward(b, k_cache, v_cache).float().argmax(-1)[0])]
    for j in range(N_NEW - 1):
        c = S + j
        d = StepBatch(i32([want[-1]]), i32([c + soft["delta"]]), i32([c]), i32([0]), i32([1]), i32([c + 1]), table,
                      i32([0]), 1, 1)
        want.append(int(model.forward(d, k_cache, v_cache).float().argmax(-1)[0]))

    eng = LLMEngine(model, num_blocks=32, max_batch=4, use_cuda_graph=False, prefill_chunk=8, max_step_tokens=16)
    sp = SamplingParams(max_tokens=N_NEW, temperature=0.0)
    res = eng.generate([ids, [11, 12, 13, 14]], sp, soft=[soft, None])
    assert res[0].token_ids == want, (res[0].token_ids, want)
    text_only = LLMEngine(model, num_blocks=32, max_batch=4, use_cuda_graph=False).generate([[11, 12, 13, 14]], sp)
    assert res[1].token_ids == text_only[0].token_ids          # the text request is unaffected by its neighbour
    with pytest.raises(ValueError):
        eng.add_request(ids, sp, {**soft, "rows": soft["rows"][:-1]})

    # chat content parts: images are collected in reading order
    msgs = [{"role": "user", "content": [{"type": "text", "text": "what is"}, {"type": "image", "image": img},
                                         {"type": "image_url", "image_url": {"url": "x.png"}}]}]
    found = split_content(msgs)
    assert len(found) == 2 and found[0] is img and found[1] == "x.png"


def test_generator_with_image_adapter_and_chat_parts():
    """Generator level: a chat message with an image part renders the placeholder, the adapter widens it, and the
    reply equals what the same prompt gives through the engine directly; a text-only model refuses images."""
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.pipelines.generation import ChatTemplate, Generator
    from antfly_b200.pipelines.vlm import Qwen2VLAdapter, VlmTokens
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    hf_cfg, hf = _hf(3)
    sd = hf.state_dict()
    model = LlamaModel.from_state_dict(LlamaConfig.from_hf(hf_cfg.text_config.to_dict()), QV.text_state_dict(sd),
                                       device="cpu")
    vision = QV.Qwen2VLVisionModel.from_state_dict(QV.Qwen2VLVisionConfig.from_hf(hf_cfg.vision_config.to_dict()), sd,
                                                   device="cpu", dtype=torch.float32)
    adapter = Qwen2VLAdapter(vision, VlmTokens(300), min_pixels=28 * 28, max_pixels=28 * 28 * 4)

    class Tok(ByteTokenizer):                      # a byte tokenizer that knows the image placeholder as one token
        def encode_prompt(self, text, add_bos=True):
            ids = []
            for i, piece in enumerate(text.split(adapter.placeholder)):
                if i:
                    ids += [302, 300, 303]
                ids += self.encode(piece)
            return ids

    tok = Tok(290)
    tmpl = "{% for m in messages %}{{ m['content'] }}{% endfor %}"
    assert ChatTemplate(tmpl).apply([{"role": "user", "content": [{"type": "image", "image": 1},
                                                                  {"type": "text", "text": "hi"}]}],
                                    image_placeholder="<I>") == "<I>hi"
    eng = LLMEngine(model, num_blocks=32, max_batch=2, use_cuda_graph=False)
    gen = Generator(eng, tok, tmpl, add_bos=False, vlm=adapter)
    img = torch.randint(0, 256, (50, 50, 3), generator=torch.Generator().manual_seed(1), dtype=torch.uint8)
    sp = SamplingParams(max_tokens=4, temperature=0.0)
    out = gen.generate([{"role": "user", "content": [{"type": "image", "image": img},
                                                     {"type": "text", "text": "hi"}]}], sp)
    ids, soft = adapter.expand([302, 300, 303] + tok.encode("hi"), [img])
    want = eng.generate([ids], sp, soft=[soft])[0].token_ids
    assert out.token_ids == want and out.prompt_tokens == len(ids)
    same = gen.generate("hi", sp, images=[img], raw_prompt=True)             # placeholder put in front
    assert same.token_ids == want
    plain = Generator(eng, tok, tmpl, add_bos=False)
    with pytest.raises(ValueError):
        plain.generate("hi", sp, images=[img])
    assert len(plain.generate("hi", sp).token_ids) == 4


def test_colqwen_token_embeddings_and_maxsim_match_transformers():
    """ColQwen2: per-token projected, normalised decoder states for a page image and for a text query; the
    late-interaction score equals the sum over query tokens of the best page-token dot product."""
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.pipelines.vlm import ColQwenEmbedder, Qwen2VLAdapter, VlmTokens

    vlm_cfg, _ = _hf(5)
    torch.manual_seed(5)
    cfg = transformers.ColQwen2Config(vlm_config=vlm_cfg, embedding_dim=24)
    hf = transformers.ColQwen2ForRetrieval(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
    _round_text_linears(hf.vlm)
    sd = {k[len("vlm."):] if k.startswith("vlm.") else k: v for k, v in hf.state_dict().items()}
    model = LlamaModel.from_state_dict(LlamaConfig.from_hf(vlm_cfg.text_config.to_dict()), QV.text_state_dict(
        {k: v for k, v in sd.items() if not k.startswith("embedding_proj_layer")}), device="cpu")
    vision = QV.Qwen2VLVisionModel.from_state_dict(QV.Qwen2VLVisionConfig.from_hf(vlm_cfg.vision_config.to_dict()), sd,
                                                   device="cpu", dtype=torch.float32)

    class FixedPatches(Qwen2VLAdapter):              # feed the same patches to both implementations
        def encode_images(self, images):
            return self.vision.forward(images[0][0], [images[0][1]]), [images[0][1]]

    ad = FixedPatches(vision, VlmTokens(300, 302, 303))
    emb = ColQwenEmbedder(model, ad, sd["embedding_proj_layer.weight"].float(), sd["embedding_proj_layer.bias"].float())
    grid = (1, 4, 6)
    patches = torch.randn(24, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(6))
    page_ids = [302, 300, 303, 7, 8]
    got_page = emb.embed_ids(page_ids, [(patches, grid)])
    full = [302] + [300] * 6 + [303, 7, 8]
    with torch.no_grad():
        want_page = hf(input_ids=torch.tensor([full]), pixel_values=patches[None], image_grid_thw=torch.tensor([grid]),
                       attention_mask=torch.ones(1, len(full), dtype=torch.long),
                       mm_token_type_ids=torch.tensor([[int(t == 300) for t in full]])).embeddings[0]
        q_ids = [11, 12, 13, 14]
        want_q = hf(input_ids=torch.tensor([q_ids]), attention_mask=torch.ones(1, 4, dtype=torch.long)).embeddings[0]
    got_q = emb.embed_ids(q_ids)
    assert got_page.shape == want_page.shape == (10, 24) and emb.dim == 24
    assert float(torch.nn.functional.cosine_similarity(got_page, want_page, dim=-1).min()) > 0.98
    assert float(torch.nn.functional.cosine_similarity(got_q, want_q, dim=-1).min()) > 0.98
    other = torch.nn.functional.normalize(torch.randn(7, 24, generator=torch.Generator().manual_seed(8)), dim=-1)
    s = emb.score(got_q, [got_page, other])
    ref = [float((got_q.bfloat16().float() @ p.bfloat16().float().T).max(-1).values.sum()) for p in (got_page, other)]
    assert s == pytest.approx(ref, abs=2e-2) and emb.score(got_q, []) == []


def test_colqwen_rerank_pages_through_the_endpoint():
    import base64
    import io

    pil = pytest.importorskip("PIL.Image")
    import numpy as np
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.pipelines.vlm import ColQwenEmbedder, Qwen2VLAdapter, VlmTokens
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    hf_cfg, hf = _hf(6)
    sd = hf.state_dict()
    model = LlamaModel.from_state_dict(LlamaConfig.from_hf(hf_cfg.text_config.to_dict()), QV.text_state_dict(sd),
                                       device="cpu")
    vision = QV.Qwen2VLVisionModel.from_state_dict(QV.Qwen2VLVisionConfig.from_hf(hf_cfg.vision_config.to_dict()), sd,
                                                   device="cpu", dtype=torch.float32)

    class Tok(ByteTokenizer):
        def encode_prompt(self, text, add_bos=True):
            ids = []
            for i, piece in enumerate(text.split("<|image_pad|>")):
                if i:
                    ids.append(300)
                ids += self.encode(piece)
            return ids

    g = torch.Generator().manual_seed(0)
    emb = ColQwenEmbedder(model, Qwen2VLAdapter(vision, VlmTokens(300), 28 * 28, 28 * 28 * 4),
                          torch.randn(16, 128, generator=g) * 0.1, None, Tok(290))
    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register("tiny-colqwen", "embedder", emb, emb.tokenizer)
    c = TestClient(create_app(mgr))
    buf = io.BytesIO()
    pil.fromarray(np.random.default_rng(0).integers(0, 256, size=(40, 60, 3), dtype=np.uint8)).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    r = c.post("/ai/v1/rerank_multimodal", json={"model": "tiny-colqwen", "query": "invoice total", "documents": [
        {"content": [{"type": "image_url", "image_url": {"url": url}}]},
        {"content": [{"type": "text", "text": "invoice total"}, {"type": "image_url", "image_url": {"url": url}}]}]})
    assert r.status_code == 200, r.text
    d = r.json()["data"]
    want, _ = emb.rerank_pages("invoice total", [([], [__import__("antfly_b200.pipelines.multimodal", fromlist=["x"])
                                                       .decode_data_url(url)])])
    assert d[0]["score"] == pytest.approx(want[0], abs=1e-3)
    assert d[1]["score"] >= d[0]["score"] - 1e-6           # the second document also holds the query text itself
