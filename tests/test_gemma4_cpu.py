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


def _assistant(target, hf_target_cfg, seed=3, **extra_cfg):
    """A random query-only assistant whose head geometry fits the target's caches."""
    from antfly_b200.models.gemma4 import Gemma4Assistant

    torch.manual_seed(seed)
    acfg = transformers.Gemma4TextConfig(
        vocab_size=hf_target_cfg.vocab_size, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=hf_target_cfg.num_key_value_heads, head_dim=hf_target_cfg.head_dim,
        global_head_dim=hf_target_cfg.global_head_dim, sliding_window=hf_target_cfg.sliding_window,
        hidden_size_per_layer_input=0, vocab_size_per_layer_input=hf_target_cfg.vocab_size, num_kv_shared_layers=0,
        layer_types=["sliding_attention", "full_attention"], tie_word_embeddings=True)
    hf_a = transformers.Gemma4ForCausalLM(acfg).eval().float()
    sd = {k: v for k, v in hf_a.state_dict().items()
          if not any(s in k for s in ("k_proj", "v_proj", "k_norm"))}
    sd["pre_projection.weight"] = torch.randn(32, 2 * hf_target_cfg.hidden_size) * 0.2
    sd["post_projection.weight"] = torch.randn(hf_target_cfg.hidden_size, 32) * 0.2
    conf = {"model_type": "gemma4_assistant", "backbone_hidden_size": hf_target_cfg.hidden_size,
            "text_config": acfg.to_dict(), **extra_cfg}
    if extra_cfg.get("num_centroids"):
        nc = extra_cfg["num_centroids"]
        sd["masked_embedding.centroids.weight"] = torch.randn(nc, 32)
        sd["masked_embedding.token_ordering"] = torch.randperm(hf_target_cfg.vocab_size).float()
    return Gemma4Assistant.from_state_dict(conf, sd, target, device="cpu", dtype=torch.float32), sd


def test_mtp_assistant_drafts_from_the_targets_caches_and_never_changes_the_output():
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel, kv_donor_layers

    hf_cfg, hf = _hf()
    cfg = Gemma4Config.from_hf(hf_cfg.to_dict())
    target = Gemma4TextModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    assert kv_donor_layers(cfg) == (3, 2)
    asst, _ = _assistant(target, hf_cfg)
    assert asst.body.kv_source == {0: 3, 1: 2} and asst.body.query_only
    prompt = [5, 9, 17, 33, 2, 71, 8]
    plain = target.generate(prompt, 14)
    for k in (1, 3, 5):
        assert asst.generate(prompt, 14, k=k) == plain
    assert asst.rounds > 0 and asst.drafted >= asst.matched >= 0
    # a draft step reads the caches and leaves them alone; chained steps feed the projected activation forward
    logits, st = target.forward(torch.tensor(prompt))
    before = {l: (k.clone(), v.clone()) for l, (k, v) in st.kv.items()}
    d3 = asst.draft(prompt[-1], st.last_hidden, st, 3)
    assert len(d3) == 3 and st.length == len(prompt)
    assert all(torch.equal(st.kv[l][0], before[l][0]) and torch.equal(st.kv[l][1], before[l][1]) for l in before)
    assert asst.draft(prompt[-1], st.last_hidden, st, 1) == d3[:1]
    # an assistant that always agrees with the target is accepted whole: k drafts + 1 bonus token per round
    n0 = len(prompt)
    asst.draft = lambda token, act, state, k: (plain + [0] * 8)[state.length - n0: state.length - n0 + k]
    asst.rounds = asst.drafted = asst.matched = 0
    assert asst.generate(prompt, 13, k=4) == plain[:13]
    assert asst.matched == asst.drafted and asst.rounds == 3           # 1 + 3 * (4 + 1) >= 13


def test_mtp_masked_embedding_argmax_only_sees_the_best_clusters():
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel

    hf_cfg, hf = _hf()
    target = Gemma4TextModel.from_state_dict(Gemma4Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                             dtype=torch.float32)
    asst, sd = _assistant(target, hf_cfg, num_centroids=10, centroid_intermediate_top_k=2,
                          use_ordered_embeddings=True)
    g = torch.Generator().manual_seed(0)
    hidden, logits = torch.randn(32, generator=g), torch.randn(200, generator=g)
    got = asst._pick(hidden, logits)
    cl = sd["masked_embedding.centroids.weight"] @ hidden
    best = cl.topk(2).indices.tolist()
    order = sd["masked_embedding.token_ordering"].long().view(10, 20)
    cand = torch.cat([order[b] for b in best])
    assert got == int(cand[logits[cand].argmax()])
    assert got != int(logits.argmax()) or int(logits.argmax()) in cand.tolist()
    asst.ordered = False
    assert asst._pick(hidden, logits) == int(logits.argmax())


def test_mtp_needs_a_target_with_shared_kv_donors():
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel

    hf_cfg, hf = _hf(num_kv_shared_layers=0)
    target = Gemma4TextModel.from_state_dict(Gemma4Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                             dtype=torch.float32)
    with pytest.raises(ValueError):
        _assistant(target, hf_cfg)


def test_mtp_assistant_as_the_draft_model_of_a_request(tmp_path):
    import json

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import safetensors_io as st
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel
    from antfly_b200.runtime.sampling_params import SamplingParams

    hf_cfg, hf = _hf(vocab_size=600, vocab_size_per_layer_input=600)
    d = tmp_path / "generators" / "tiny-g4"
    d.mkdir(parents=True)
    st.save_file({k: v.contiguous() for k, v in hf.state_dict().items() if k != "lm_head.weight"},
                 str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(dict(hf_cfg.to_dict(), model_type="gemma4_text"), default=str))
    target = Gemma4TextModel.from_state_dict(Gemma4Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                             dtype=torch.float32)
    asst, sd = _assistant(target, hf_cfg)
    a = tmp_path / "generators" / "tiny-g4-assistant"
    a.mkdir(parents=True)
    st.save_file({k: v.contiguous() for k, v in sd.items() if k != "lm_head.weight"}, str(a / "model.safetensors"))
    conf = {"model_type": "gemma4_assistant", "backbone_hidden_size": hf_cfg.hidden_size,
            "text_config": asst.body.cfg.__dict__ | {"model_type": "gemma4_text"}}
    (a / "config.json").write_text(json.dumps(conf, default=str))
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    plain = mgr.get_generator("tiny-g4").pipeline.generate("hello world", sp, raw_prompt=True)
    lm = mgr.get_generator("tiny-g4", draft_model="tiny-g4-assistant")
    assert lm is mgr.get_generator("tiny-g4", draft_model="tiny-g4-assistant")        # cached variant
    pipe = lm.pipeline
    deltas = []
    fast = pipe.generate("hello world", sp, raw_prompt=True, on_delta=deltas.append)
    assert fast.token_ids == plain.token_ids and fast.text == plain.text and len(fast.token_ids) == 12
    assert "".join(deltas) == fast.text[: len("".join(deltas))] and pipe.assistant.rounds > 0
    # sampling requests decode without the assistant
    rounds = pipe.assistant.rounds
    pipe.generate("hello world", SamplingParams(max_tokens=4, temperature=0.8, seed=1, ignore_eos=True), raw_prompt=True)
    assert pipe.assistant.rounds == rounds
    with pytest.raises(ValueError):
        mgr.get_generator("tiny-g4", cache_dtype="fp8")
    with pytest.raises(ValueError):
        mgr.get_generator("tiny-g4", draft_model="tiny-g4")                           # not an assistant checkpoint
