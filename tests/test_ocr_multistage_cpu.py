"""Multi-stage OCR: region extraction from a probability map, reading order, text assembly, CTC decoding, and the
whole pipeline on a synthetic page with a stand-in recogniser."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from antfly_b200.pipelines import ocr_multistage as O


def test_connected_components_merge_and_diagonals():
    m = np.zeros((7, 9), dtype=bool)
    m[1, 1] = m[2, 2] = True                    # diagonal neighbours are one component
    m[1:5, 5] = m[1:5, 8] = True                # a U shape: two arms joined at the bottom
    m[4, 5:9] = True
    m[6, 0] = True                              # a single pixel
    comps = O.connected_components(m)
    assert comps == [(1, 1, 2, 2, 2), (5, 1, 8, 4, 10), (0, 6, 0, 6, 1)]
    assert O.connected_components(m, min_area=2) == comps[:2]
    assert O.connected_components(np.zeros((3, 3), dtype=bool)) == []


def test_region_post_processing_scores_and_unclip():
    p = torch.zeros(20, 40)
    p[4:8, 5:25] = 0.9                          # a confident line
    p[12:16, 5:25] = 0.35                       # above the pixel threshold, below the box threshold
    regs = O.RegionPostProcessor(threshold=0.3, box_threshold=0.6, unclip_ratio=1.5, min_box_area=4).process(p, 400, 100)
    assert len(regs) == 1 and abs(regs[0].confidence - 0.9) < 1e-6
    bw, bh = 20 * 10.0, 4 * 5.0                 # the box in page units (the map is 10x / 5x smaller than the page)
    d = bw * bh * 1.5 / (2 * (bw + bh))
    assert regs[0].bbox == pytest.approx((50 - d, 20 - d, 250 + d, 40 + d))
    edge = torch.zeros(10, 10); edge[0:3, 0:6] = 1.0
    b = O.RegionPostProcessor(min_box_area=1).process(edge, 10, 10)[0].bbox
    assert b[0] == 0.0 and b[1] == 0.0          # grown boxes are clipped to the page


def test_reading_order_text_assembly_overlap_and_labels():
    R = lambda x0, y0, x1, y1, t: O.TextRegion((x0, y0, x1, y1), 1.0, t)
    regs = [R(200, 12, 300, 32, "world"), R(10, 60, 120, 80, "second"), R(10, 10, 150, 30, "hello"),
            R(130, 62, 200, 82, "line")]
    ordered = O.sort_reading_order(regs)
    assert [r.text for r in ordered] == ["hello", "world", "second", "line"]
    assert O.assemble_text(ordered) == "hello world\nsecond line" and O.assemble_text([]) == ""
    assert O.overlap((0, 0, 10, 10), (5, 0, 15, 10)) == pytest.approx(50 / 150) and O.overlap((0, 0, 1, 1), (2, 2, 3, 3)) == 0
    O.attach_layout_labels(ordered, [O.LayoutRegion((0, 0, 400, 40), "title"), O.LayoutRegion((0, 50, 400, 100), "body")])
    assert [r.label for r in ordered] == ["title", "title", "body", "body"]


def test_ctc_greedy_decoding():
    charset = ["a", "b", "c"]
    #            blank  a     a(repeat)  blank  a     c
    steps = [0, 1, 1, 0, 1, 3]
    logits = torch.full((6, 4), -5.0)
    for t, k in enumerate(steps):
        logits[t, k] = 2.0 + t
    text, conf = O.ctc_greedy(logits, charset)
    assert text == "aac" and conf == pytest.approx((3.0 + 6.0 + 7.0) / 3)
    assert O.ctc_greedy(torch.zeros(0, 4), charset) == ("", 0.0)
    assert O.ctc_greedy(torch.tensor([[1.0, 0.0]]), ["x"]) == ("", 0.0)


def test_pipeline_on_a_synthetic_page():
    page = torch.full((140, 420, 3), 250, dtype=torch.uint8)
    for (y0, y1, x0, x1) in ((30, 50, 20, 100), (30, 50, 112, 200), (32, 52, 300, 380), (90, 110, 20, 150)):
        page[y0:y1, x0:x1] = 20
    seen = []

    class Rec:
        def read(self, crops, max_new_tokens=64):
            seen.append(len(crops))
            return [SimpleNamespace(text=f" w{c.shape[1] // 10} ", confidence=0.5) for c in crops]

    ocr = O.MultiStageOCR(Rec(), layout=lambda p: [O.LayoutRegion((0, 0, 420, 70), "header")], batch_size=2)
    res = ocr.run(page)
    assert len(res.regions) == 3 and seen == [2, 1]
    a, b, c = res.regions
    assert a.bbox[0] < 20 and a.bbox[2] > 200 and a.bbox[2] < 300         # the two close words became one region
    assert b.bbox[0] > 250 and c.bbox[1] > 70
    assert res.full_text.count("\n") == 1 and res.full_text.split("\n")[0].count(" ") == 1
    assert [r.label for r in res.regions] == ["header", "header", None]
    assert all(r.rec_confidence == 0.5 and r.text.startswith("w") for r in res.regions)
    blank = O.MultiStageOCR(Rec()).run(torch.full((50, 50, 3), 255, dtype=torch.uint8))
    assert blank.full_text == "" and blank.regions == []


def test_read_endpoint_multistage_mode():
    import base64
    import io

    pil = pytest.importorskip("PIL.Image")
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    class Rec:
        def read(self, crops, max_new_tokens=64):
            return [SimpleNamespace(text=f"w{c.shape[1] // 10}", confidence=0.5, token_ids=[1]) for c in crops]

    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register("fake-reader", "reader", Rec(), None)
    c = TestClient(create_app(mgr))
    page = np.full((140, 420, 3), 250, dtype=np.uint8)
    page[30:50, 20:200] = 20
    page[90:110, 20:150] = 20
    buf = io.BytesIO()
    pil.fromarray(page).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    r = c.post("/ai/v1/read", json={"model": "fake-reader", "images": [url], "multistage": True, "min_box_area": 20})
    assert r.status_code == 200, r.text
    d = r.json()["data"][0]
    assert len(d["regions"]) == 2 and d["text"].count("\n") == 1
    assert d["regions"][0]["bbox"][1] < d["regions"][1]["bbox"][1]
