"""LayoutLMv3 against the Hugging Face implementation: text + boxes + page image, and text + boxes alone."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models.layoutlmv3 import Document, LayoutLMv3Config, LayoutLMv3Model, distance_bucket


def _hf(num_labels):
    torch.manual_seed(9)
    cfg = transformers.LayoutLMv3Config(
        vocab_size=300, hidden_size=96, num_hidden_layers=2, num_attention_heads=4, intermediate_size=192,
        max_position_embeddings=80, coordinate_size=16, shape_size=16, input_size=64, patch_size=16,
        rel_pos_bins=16, max_rel_pos=32, rel_2d_pos_bins=16, max_rel_2d_pos=64, num_labels=num_labels,
        hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, classifier_dropout=0.0)
    hf = transformers.LayoutLMv3ForTokenClassification(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias") or "rel_pos" in n or n.endswith("cls_token") or n.endswith("pos_embed"):
                p.normal_(0, 0.2)
    return cfg, hf


def _doc(g, n, with_image=True):
    ids = [0] + torch.randint(3, 290, (n,), generator=g).tolist() + [2]
    x0 = torch.randint(0, 800, (n + 2,), generator=g)
    y0 = torch.randint(0, 800, (n + 2,), generator=g)
    boxes = torch.stack([x0, y0, x0 + torch.randint(1, 200, (n + 2,), generator=g),
                         y0 + torch.randint(1, 200, (n + 2,), generator=g)], 1).tolist()
    px = torch.randn(3, 64, 64, generator=g) if with_image else None
    return Document(ids, boxes, px)


@pytest.mark.parametrize("num_labels,with_image", [(5, True), (12, True), (5, False)])
def test_layoutlmv3_token_logits_match_transformers(num_labels, with_image):
    hf_cfg, hf = _hf(num_labels)
    cfg = LayoutLMv3Config.from_hf(hf_cfg.to_dict())
    model = LayoutLMv3Model.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    assert cfg.num_labels == num_labels and ("cls.dense.w" in model.w) == (num_labels >= 10)
    g = torch.Generator().manual_seed(num_labels)
    docs = [_doc(g, 9, with_image), _doc(g, 21, with_image)]
    got = model.token_logits(docs)
    for d, lg in zip(docs, got):
        kw = dict(input_ids=torch.tensor([d.ids]), bbox=torch.tensor([d.boxes]))
        if with_image:
            kw["pixel_values"] = d.pixels[None]
        with torch.no_grad():
            want = hf(**kw).logits[0]
        assert lg.shape == want.shape == (len(d.ids), num_labels)
        assert float(torch.nn.functional.cosine_similarity(lg.flatten(), want.flatten(), dim=0)) > 0.999
        torch.testing.assert_close(lg, want, atol=5e-2, rtol=5e-2)
    h = model.encode(docs[:1])[0]
    assert h.shape[0] == len(docs[0].ids) + (17 if with_image else 0)
    with pytest.raises(ValueError):
        model.encode([Document([0, 5, 2], [[0, 0, 10, 10]] * 2)])
    with pytest.raises(ValueError):
        model.encode([Document([0, 5, 2], [[0, 0, 10, 2000]] * 3)])


def test_distance_buckets():
    r = torch.tensor([-200, -9, -3, 0, 3, 9, 200])
    b = distance_bucket(r, 16, 32)
    assert b.tolist()[3] == 0 and b.tolist()[2] == 3 and b.tolist()[4] == 8 + 3
    assert b.max() == 15 and b.tolist()[0] == 7 and b.tolist()[-1] == 15


def test_layout_word_labelling_pipeline():
    from antfly_b200.pipelines.layout import (LayoutTokenClassifier, WordLabel, group_entities, normalize_box,
                                              page_pixels)
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    hf_cfg, hf = _hf(5)
    cfg = LayoutLMv3Config.from_hf(hf_cfg.to_dict())
    model = LayoutLMv3Model.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    labels = {0: "O", 1: "B-KEY", 2: "I-KEY", 3: "B-VALUE", 4: "I-VALUE"}
    pipe = LayoutTokenClassifier(model, ByteTokenizer(290), labels)
    assert normalize_box((50, 100, 150, 300), 500, 1000) == (100, 100, 300, 300)
    page = torch.randint(0, 256, (120, 90, 3), generator=torch.Generator().manual_seed(0), dtype=torch.uint8)
    px = page_pixels(page, 64)
    assert px.shape == (3, 64, 64) and float(px.min()) >= -1.0 and float(px.max()) <= 1.0
    words = ["Invoice", "No", ":", "12345", "Total", "due"] * 6           # longer than one 77-token window
    boxes = [(10 * i % 900, 20, 10 * i % 900 + 40, 40) for i in range(len(words))]
    got = pipe.label_words(words, boxes, page)
    assert [g.word for g in got] == words and all(g.label in labels.values() and 0 < g.score <= 1 for g in got)
    # the first window's words agree with a direct run of the model on that window
    ids, bx, firsts = [0], [(0, 0, 0, 0)], []
    for w, b in zip(words, boxes):
        t = ByteTokenizer(290).encode(w)
        if len(ids) + len(t) + 1 > pipe.window:
            break
        firsts.append(len(ids)); ids += t; bx += [b] * len(t)
    lg = model.token_logits([Document(ids + [2], bx + [(0, 0, 0, 0)], px)])[0]
    assert [labels[int(lg[f].argmax())] for f in firsts] == [g.label for g in got[: len(firsts)]]
    ents = group_entities([WordLabel("Invoice", (0, 0, 10, 10), "B-KEY", 0.9), WordLabel("No", (12, 0, 20, 10), "I-KEY", 0.7),
                           WordLabel(":", (21, 0, 22, 10), "O", 0.9), WordLabel("12345", (30, 0, 60, 12), "B-VALUE", 0.8),
                           WordLabel("77", (70, 0, 80, 12), "B-VALUE", 0.6)])
    assert [(e["label"], e["text"], e["box"]) for e in ents] == [
        ("KEY", "Invoice No", [0, 0, 20, 10]), ("VALUE", "12345", [30, 0, 60, 12]), ("VALUE", "77", [70, 0, 80, 12])]
    assert abs(ents[0]["score"] - 0.8) < 1e-9
    with pytest.raises(ValueError):
        pipe.label_words(["a"], [])


def test_layout_endpoint():
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app
    from antfly_b200.pipelines.layout import LayoutTokenClassifier
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    hf_cfg, hf = _hf(5)
    model = LayoutLMv3Model.from_state_dict(LayoutLMv3Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                            dtype=torch.float32)
    tok = ByteTokenizer(290)
    pipe = LayoutTokenClassifier(model, tok, {0: "O", 1: "B-KEY", 2: "I-KEY", 3: "B-VALUE", 4: "I-VALUE"})
    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register("tiny-layout", "recognizer", pipe, tok)
    c = TestClient(create_app(mgr))
    page = {"words": ["Total", ":", "42"], "boxes": [[10, 10, 60, 30], [62, 10, 66, 30], [80, 10, 120, 30]],
            "width": 200, "height": 100}
    r = c.post("/ai/v1/layout", json={"model": "tiny-layout", "pages": [page]})
    assert r.status_code == 200, r.text
    rec = r.json()["data"][0]
    assert [w["word"] for w in rec["words"]] == page["words"] and rec["words"][0]["box"] == [50, 100, 300, 300]
    assert isinstance(rec["entities"], list)
    want = pipe.label_words(page["words"], [(50, 100, 300, 300), (310, 100, 330, 300), (400, 100, 600, 300)])
    assert [w["label"] for w in rec["words"]] == [w.label for w in want]
    bad = dict(page, boxes=page["boxes"][:2])
    assert c.post("/ai/v1/layout", json={"model": "tiny-layout", "pages": [bad]}).status_code == 400
    far = {"words": ["x"], "boxes": [[0, 0, 5000, 10]]}
    assert c.post("/ai/v1/layout", json={"model": "tiny-layout", "pages": [far]}).status_code == 400


def test_document_classification_head_matches_transformers():
    from antfly_b200.pipelines.layout import DocumentClassifier
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    torch.manual_seed(4)
    hf_cfg, _ = _hf(4)
    hf = transformers.LayoutLMv3ForSequenceClassification(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias") or "rel_pos" in n:
                p.normal_(0, 0.2)
    model = LayoutLMv3Model.from_state_dict(LayoutLMv3Config.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                            dtype=torch.float32)
    g = torch.Generator().manual_seed(1)
    docs = [_doc(g, 7), _doc(g, 15)]
    got = model.sequence_logits(docs)
    for d, lg in zip(docs, got):
        with torch.no_grad():
            want = hf(input_ids=torch.tensor([d.ids]), bbox=torch.tensor([d.boxes]), pixel_values=d.pixels[None]).logits[0]
        torch.testing.assert_close(lg, want, atol=5e-2, rtol=5e-2)
    clf = DocumentClassifier(model, ByteTokenizer(290), {0: "invoice", 1: "letter", 2: "form", 3: "memo"})
    out = clf.classify(["Total", "due"], [(10, 10, 60, 30), (70, 10, 100, 30)], top_k=2)
    assert len(out) == 2 and out[0]["score"] >= out[1]["score"] and out[0]["label"] in ("invoice", "letter", "form", "memo")
    token_only = LayoutLMv3Model.from_state_dict(LayoutLMv3Config.from_hf(_hf(5)[0].to_dict()), _hf(5)[1].state_dict(),
                                                 device="cpu", dtype=torch.float32)
    with pytest.raises(ValueError):
        token_only.sequence_logits(docs)
