"""Florence-2 (DaViT tower, projector, BART text half) against transformers' Florence2ForConditionalGeneration."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf(image=64):
    from transformers.models.florence2 import modeling_florence2 as M

    torch.manual_seed(0)
    v = transformers.Florence2VisionConfig(depths=(1, 1, 2, 1), embed_dim=(16, 32, 48, 64), num_heads=(2, 2, 4, 4),
                                           num_groups=(2, 4, 4, 8), window_size=3, projection_dim=40,
                                           max_position_embeddings=12, max_temporal_embeddings=5, drop_path_rate=0.0)
    t = transformers.BartConfig(vocab_size=120, d_model=40, encoder_layers=2, decoder_layers=2,
                                encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=64,
                                decoder_ffn_dim=64, max_position_embeddings=64, decoder_start_token_id=2,
                                eos_token_id=2, bos_token_id=0, pad_token_id=1, forced_eos_token_id=None)
    c = transformers.Florence2Config(text_config=t, vision_config=v, image_token_id=119)
    m = M.Florence2ForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n or n.endswith(".bias"):
                p.add_(torch.randn_like(p) * 0.1)
    return c, m


def test_florence2_tower_projector_and_logits_match_transformers():
    from antfly_b200.models.florence2 import Florence2Model

    c, hf = _hf()
    model = Florence2Model.from_state_dict(c.to_dict(), hf.state_dict(), device="cpu", dtype=torch.float32)
    px = torch.randn(2, 3, 80, 64)            # feature map 3 x 2: windows need padding at every stage but the first
    with torch.no_grad():
        want_map = hf.model.vision_tower(px).last_hidden_state                # [B, C, H, W]
        want_tok = hf.model.get_image_features(px).pooler_output
    got_map = model.tower.forward(px)
    torch.testing.assert_close(got_map.permute(0, 3, 1, 2), want_map, atol=2e-4, rtol=2e-3)
    got_tok = model.image_tokens(px)
    torch.testing.assert_close(got_tok, want_tok, atol=2e-4, rtol=2e-3)
    n_img = want_tok.shape[1]
    prompt = [0, 17, 33, 51, 2]
    ids = torch.tensor([[119] * n_img + prompt])
    dec = torch.tensor([[2, 9, 14, 77]])
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=px[:1], decoder_input_ids=dec).logits[0]
    state = model.start_decoding(model.encode(prompt, px[0]))
    got = model.decode(state, dec[0].tolist())
    torch.testing.assert_close(got, want, atol=1e-2, rtol=1e-2)              # the CPU attention wrapper rounds to bf16
    # step-by-step decoding continues from the cache
    state = model.start_decoding(model.encode(prompt, px[0]))
    rows = [model.decode(state, [t])[0] for t in dec[0].tolist()]
    torch.testing.assert_close(torch.stack(rows), want, atol=1e-2, rtol=1e-2)


def test_original_checkpoint_names_load_the_same_model():
    """The original release's tensor names (``vision_tower.convs.0.proj``, ``...conv1.fn.dw``, ``window_attn.fn.qkv``,
    ``ffn.fn.net.fc1``, a bare [C, proj] ``image_projection``, ``language_model.model.*``) map onto the same weights."""
    from antfly_b200.models.florence2 import Florence2Model

    c, hf = _hf()
    sd = hf.state_dict()
    orig = {}
    for k, v in sd.items():
        if k.startswith("model.vision_tower."):
            n = k[len("model."):]
            n = n.replace(".conv.", ".proj.") if ".convs." in n else n
            n = n.replace(".conv1.", ".conv1.fn.dw.").replace(".conv2.", ".conv2.fn.dw.")
            attn = "window_attn" if ".spatial_block." in n else "channel_attn"
            n = n.replace(".norm1.", f".{attn}.norm.").replace(f".{attn}.qkv.", f".{attn}.fn.qkv.")
            n = n.replace(f".{attn}.proj.", f".{attn}.fn.proj.")
            n = n.replace(".norm2.", ".ffn.norm.").replace(".ffn.fc", ".ffn.fn.net.fc")
            orig[n] = v
        elif k == "model.multi_modal_projector.image_projection.weight":
            orig["image_projection"] = v.t().contiguous()
        elif k.startswith("model.multi_modal_projector.image_proj_norm."):
            orig[k[len("model.multi_modal_projector."):]] = v
        elif k.startswith("model.multi_modal_projector.image_position_embed."):
            orig["image_pos_embed." + k[len("model.multi_modal_projector.image_position_embed."):]] = v
        elif k.startswith("model.multi_modal_projector.visual_temporal_embed."):
            orig[k[len("model.multi_modal_projector."):]] = v
        elif k.startswith("model.language_model."):
            orig["language_model.model." + k[len("model.language_model."):]] = v
        elif k == "lm_head.weight":
            orig["language_model.lm_head.weight"] = v
    a = Florence2Model.from_state_dict(c.to_dict(), sd, device="cpu", dtype=torch.float32)
    b = Florence2Model.from_state_dict(c.to_dict(), orig, device="cpu", dtype=torch.float32)
    assert set(a.tower.w) == set(b.tower.w) and all(torch.equal(a.tower.w[k], b.tower.w[k]) for k in a.tower.w)
    assert all(torch.equal(a.p[k], b.p[k]) for k in a.p)
    assert all(torch.equal(a.text.w[k], b.text.w[k]) for k in a.text.w)


def test_no_repeat_ngram_guard():
    from antfly_b200.models.florence2 import banned_next_tokens

    assert banned_next_tokens([1, 2, 3, 1, 2], 3) == [3]
    assert banned_next_tokens([1, 2, 3, 1, 2], 2) == [3]
    assert sorted(banned_next_tokens([5, 6, 5, 7, 5], 2)) == [6, 7]
    assert banned_next_tokens([1, 2], 4) == [] and banned_next_tokens([1, 2, 3], 0) == []
    assert banned_next_tokens([4, 4, 4], 1) == [4, 4, 4]


def test_generate_matches_transformers_greedy_search():
    from antfly_b200.models.florence2 import Florence2Model

    c, hf = _hf()
    model = Florence2Model.from_state_dict(c.to_dict(), hf.state_dict(), device="cpu", dtype=torch.float32)
    px = torch.randn(1, 3, 64, 64)
    n_img = model.image_tokens(px).shape[1]
    prompt = [0, 40, 41, 42, 2]
    seq = [2]
    for _ in range(6):
        with torch.no_grad():
            lg = hf(input_ids=torch.tensor([[119] * n_img + prompt]), pixel_values=px,
                    decoder_input_ids=torch.tensor([seq])).logits[0, -1]
        seq.append(int(lg.argmax()))
    want = seq[1:]
    if 2 in want:
        want = want[:want.index(2)]
    assert model.generate(prompt, px[0], max_new_tokens=6) == want


def test_florence2_reader_through_the_http_endpoint(tmp_path):
    import base64
    import io
    import json

    import numpy as np
    from fastapi.testclient import TestClient
    from PIL import Image as pil

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app
    from antfly_b200.formats import safetensors_io as st

    c, hf = _hf()
    d = tmp_path / "readers" / "tiny-florence"
    d.mkdir(parents=True)
    c.text_config.vocab_size = 600
    from transformers.models.florence2 import modeling_florence2 as M

    torch.manual_seed(1)
    c.image_token_id = 599
    hf = M.Florence2ForConditionalGeneration(c).eval().float()
    sd = {k: v.contiguous() for k, v in hf.state_dict().items() if k != "lm_head.weight"}
    st.save_file(sd, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(c.to_dict(), default=str))
    (d / "preprocessor_config.json").write_text(json.dumps({"size": {"height": 64, "width": 64}, "resample": 3}))
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")
    client = TestClient(create_app(mgr))
    buf = io.BytesIO()
    img = np.random.default_rng(0).integers(0, 256, size=(30, 50, 3), dtype=np.uint8)
    pil.fromarray(img).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    r = client.post("/ai/v1/read", json={"model": "tiny-florence", "images": [url], "prompt": "<CAPTION>",
                                         "max_tokens": 6})
    assert r.status_code == 200, r.text
    body = r.json()
    pipe = mgr.get("tiny-florence", "reader").pipeline
    # the task token was rewritten to its sentence and wrapped in the begin / end markers
    ids = pipe.prompt_ids("<CAPTION>")
    assert ids[0] == 0 and ids[-1] == 2 and ids[1:-1] == list(pipe.tokenizer.encode("What does the image describe?"))
    assert pipe.prompt_ids("free text")[1:-1] == list(pipe.tokenizer.encode("free text"))
    px = pipe.preprocess(torch.from_numpy(img))
    assert px.shape == (3, 64, 64)
    direct = pipe.model.generate(ids, px, 6, pipe.no_repeat_ngram_size)
    assert body["usage"]["completion_tokens"] == len(direct)
    assert body["data"][0]["text"] == pipe.tokenizer.decode(direct).replace("<s>", "").replace("</s>", "").strip()
    # a different task prompt changes the encoder input (and, for this random model, usually the output)
    r2 = client.post("/ai/v1/read", json={"model": "tiny-florence", "images": [url], "max_tokens": 6})
    assert r2.status_code == 200


def test_location_tokens_become_pixel_regions():
    from antfly_b200.pipelines.reading import parse_location_text

    od = "car<loc_100><loc_200><loc_500><loc_600>person<loc_0><loc_0><loc_999><loc_999><loc_10><loc_20><loc_30><loc_40>"
    r = parse_location_text(od, 1000, 500)
    assert [x["text"] for x in r] == ["car", "person", "person"]
    assert r[0]["bbox"] == [100.5, 100.2, 500.5, 300.2] and r[1]["bbox"] == [0.5, 0.2, 999.5, 499.8]
    ocr = "</s><s>Hello<loc_10><loc_20><loc_110><loc_20><loc_110><loc_60><loc_10><loc_60>"
    q = parse_location_text(ocr, 1000, 1000, quads=True)
    assert len(q) == 1 and q[0]["text"] == "Hello" and q[0]["bbox"] == [10.5, 20.5, 110.5, 60.5]
    assert parse_location_text("no boxes here", 10, 10) == []
