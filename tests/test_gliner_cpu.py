"""GLiNER head and pipeline: the head against torch.nn modules carrying the same weights, the encoder from
Hugging Face, and the decode rules on hand-made logits."""
import pytest
import torch
from torch import nn

transformers = pytest.importorskip("transformers")

from antfly_b200.models.deberta import DebertaConfig
from antfly_b200.models.gliner import GlinerInput, GlinerModel
from antfly_b200.pipelines import gliner as G
from antfly_b200.tokenizer.tokenizer import ByteTokenizer

H, D = 64, 32


class _Head(nn.Module):
    """The head as plain torch modules; attribute paths give the checkpoint's tensor names."""

    def __init__(self):
        super().__init__()
        mlp = lambda i, o: nn.Sequential(nn.Linear(i, 4 * H), nn.ReLU(), nn.Dropout(0.0), nn.Linear(4 * H, o))
        self.span_rep = nn.Module()
        self.span_rep.span_rep_layer = nn.Module()
        s = self.span_rep.span_rep_layer
        s.project_start, s.project_end, s.out_project = mlp(H, H), mlp(H, H), mlp(2 * H, H)
        self.count_embed = nn.Module()
        c = self.count_embed
        c.pos_embedding = nn.Embedding(4, H)
        c.gru = nn.GRU(H, H)
        c.transformer = nn.Module()
        c.transformer.in_projector = nn.Linear(H, D)
        c.transformer.transformer = nn.TransformerEncoder(
            nn.TransformerEncoderLayer(D, 4, 2 * D, dropout=0.0, batch_first=True), 2, enable_nested_tensor=False)
        c.transformer.out_projector = nn.Sequential(nn.Linear(D + H, H), nn.ReLU(), nn.Linear(H, H), nn.ReLU(),
                                                    nn.Linear(H, H))

    def spans(self, words, starts, ends):
        s = self.span_rep.span_rep_layer
        cat = torch.relu(torch.cat([s.project_start(words)[starts], s.project_end(words)[ends]], -1))
        return s.out_project(cat)

    def labels(self, h):
        c = self.count_embed
        x = c.pos_embedding.weight[0].expand(1, h.shape[0], H)
        out, _ = c.gru(x, h[None])
        comb = out[0] + h
        y = c.transformer.transformer(c.transformer.in_projector(comb)[None])[0]
        return c.transformer.out_projector(torch.cat([y, comb], -1))


def _build():
    torch.manual_seed(21)
    hf_cfg = transformers.DebertaV2Config(
        vocab_size=400, hidden_size=H, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
        max_position_embeddings=128, type_vocab_size=0, relative_attention=True, position_buckets=16,
        max_relative_positions=-1, pos_att_type=["p2c", "c2p"], share_att_key=True, norm_rel_ebd="layer_norm",
        position_biased_input=False, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-7)
    enc = transformers.DebertaV2Model(hf_cfg).eval()
    head = _Head().eval()
    with torch.no_grad():
        for n, p in list(enc.named_parameters()) + list(head.named_parameters()):
            if n.endswith("bias") or "bias_" in n:
                p.normal_(0, 0.05)
    sd = {"encoder." + k: v for k, v in enc.state_dict().items()}
    sd.update(head.state_dict())
    model = GlinerModel.from_state_dict(DebertaConfig.from_hf(hf_cfg.to_dict()), sd, device="cpu", dtype=torch.float32)
    return enc, head, model


def test_span_logits_match_torch_modules():
    enc, head, model = _build()
    E = 390                                              # the [E] marker id
    g = torch.Generator().manual_seed(1)
    inputs = []
    for n_labels, word_lens in ((3, [1, 2, 1, 3, 1]), (2, [2, 2, 1])):
        ids, mask = [5], [0]
        for _ in range(n_labels):
            ids += [E] + torch.randint(10, 380, (2,), generator=g).tolist()
            mask += [0, 0, 0]
        ids, mask = ids + [391], mask + [0]
        for wi, n in enumerate(word_lens):
            ids += torch.randint(10, 380, (n,), generator=g).tolist()
            mask += [wi + 1] * n
        inputs.append(GlinerInput(ids, mask, len(word_lens)))
    W = 3
    got = model.span_logits(inputs, [E], W)
    for inp, lg in zip(inputs, got):
        with torch.no_grad():
            hid = enc(input_ids=torch.tensor([inp.ids])).last_hidden_state[0]
            first = [inp.words_mask.index(i + 1) for i in range(inp.num_words)]
            words = hid[first]
            st = [w if w + k < inp.num_words else 0 for w in range(inp.num_words) for k in range(W)]
            en = [w + k if w + k < inp.num_words else 0 for w in range(inp.num_words) for k in range(W)]
            sv = head.spans(words, torch.tensor(st), torch.tensor(en))
            lv = head.labels(hid[[t for t, tok in enumerate(inp.ids) if tok == E]])
            want = (sv @ lv.T).view(inp.num_words, W, -1)
        assert lg.shape == want.shape
        # every GEMM output on the CPU path is rounded to bf16 like the kernels' outputs: compare loosely
        assert float(torch.nn.functional.cosine_similarity(lg.flatten(), want.flatten(), dim=0)) > 0.999
        torch.testing.assert_close(lg, want, atol=0.15, rtol=0.05)


def test_word_split_rules():
    ws = G.split_words("Dr. Anna-Lena Müller (@anna_m) visited https://x.io/a?b=1, twice!")
    assert [w for w, _, _ in ws] == ["Dr", ".", "Anna-Lena", "Müller", "(", "@anna_m", ")", "visited",
                                     "https://x.io/a?b=1,", "twice", "!"]
    raw = "Dr. Anna-Lena Müller (@anna_m) visited https://x.io/a?b=1, twice!".encode()
    assert all(raw[a:b].decode() == w for w, a, b in ws)          # offsets are byte offsets into the UTF-8 text
    assert G.split_words("  \t\n") == [] and [w for w, _, _ in G.split_words("a- b")] == ["a", "-", "b"]


def test_decode_flat_ner_dedup_and_relations():
    text = "Ada Lovelace met Ada in London"
    words = G.split_words(text)
    lg = torch.full((6, 3, 2), -9.0)
    lg[0, 1, 0] = 3.0        # "Ada Lovelace" person
    lg[0, 0, 0] = 1.0        # "Ada" person, overlaps the better span
    lg[3, 0, 0] = 2.0        # second "Ada" person
    lg[5, 0, 1] = 4.0        # "London" place
    lg[4, 1, 1] = 0.5        # "in London" place, overlaps
    flat = G.decode_entities(text, words, 6, lg, ["person", "place"], 0.5, True)
    assert [(e.text, e.label) for e in flat] == [("Ada Lovelace", "person"), ("Ada", "person"), ("London", "place")]
    assert flat[0].start == 0 and flat[0].end == 12 and abs(flat[2].score - torch.sigmoid(torch.tensor(4.0)).item()) < 1e-6
    nested = G.decode_entities(text, words, 6, lg, ["person", "place"], 0.5, False)
    # without flat NER overlaps stay, but the two "Ada" person spans merge into the better-scoring one
    assert [(e.text, e.start) for e in nested] == [("Ada Lovelace", 0), ("Ada", 17), ("in London", 21), ("London", 24)]
    # spans that run past the kept words are ignored
    assert G.decode_entities(text, words, 3, torch.full((6, 3, 2), 9.0), ["a", "b"], 0.5, True)[-1].end <= words[2][2]

    assert G.parse_relation_label("person::born in::place") == ("person", "born in", "place")
    assert G.parse_relation_label("person::knows") == ("person", "knows", None) and G.parse_relation_label("x") is None
    assert G.relation_candidates(["person", "place"], ["knows", "Person::lives in::place", "person::x::org"]) == [
        "person::knows", "place::knows", "person::lives in::place"]
    heads = [G.GlinerEntity("Ada Lovelace", "person::lives in::place", 0, 12, 0.9),
             G.GlinerEntity("London", "person::knows", 24, 30, 0.8)]      # a place under a person-headed relation
    rels = G.match_relations(flat, heads)
    assert len(rels) == 1 and rels[0].label == "lives in" and rels[0].tail.text == "London" and rels[0].head is flat[0]


def test_pipeline_end_to_end_with_random_weights():
    _, _, model = _build()
    tok = ByteTokenizer(380)
    cfg = G.GlinerConfig.from_files({"max_width": 4, "max_length": 96, "threshold": 0.3},
                                    {"[P]": 389, "[E]": 390, "[C]": 392, "[R]": 393, "[SEP_TEXT]": 391})
    pipe = G.GlinerPipeline(model, tok, cfg)
    inp, words = pipe.prepare("Ada met Bob", ["person", "city"], cfg.token_e)
    assert inp.ids.count(390) == 2 and inp.ids.count(391) == 1 and inp.num_words == 3 and max(inp.words_mask) == 3
    assert inp.words_mask[inp.ids.index(391)] == 0 and inp.words_mask[inp.ids.index(391) + 1] == 1
    texts = ["Ada met Bob in Paris", "x " * 60, ""]
    out = pipe.recognize(texts, ["person", "city"])
    assert len(out) == 3 and out[2] == []
    for t, ents in zip(texts, out):
        raw = t.encode()
        for e in ents:
            assert raw[e.start:e.end].decode() == e.text and e.label in ("person", "city") and e.score >= 0.3
        assert all(a.end <= b.start for a, b in zip(ents, ents[1:]))           # flat NER: no overlaps
    # a long text is cut at a word boundary so that the prompt fits max_length
    inp, _ = pipe.prepare("x " * 90, ["person"], cfg.token_e)
    assert len(inp.ids) <= 96 and 0 < inp.num_words < 90
    one = pipe.recognize([texts[0]], ["person", "city"])[0]
    assert [(e.start, e.end, e.label) for e in one] == [(e.start, e.end, e.label) for e in out[0]]   # batch == single
    scores = pipe.score_labels(texts[0], ["a", "b", "c"])
    assert len(scores) == 3 and all(0 <= s <= 1 for s in scores)
    best = pipe.classify(texts[0], ["a", "b", "c"])
    assert len(best) == 1 and best[0][1] == max(scores)
    assert len(pipe.classify(texts[0], ["a", "b", "c"], multi_label=True)) == 3
    ents, rels = pipe.extract_relations(texts[:1], ["person", "city"], ["lives in"])
    assert len(ents) == 1 and len(rels) == 1
    with pytest.raises(ValueError):
        pipe.recognize(["x"], [])


def test_extract_endpoint_with_a_span_model():
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    _, _, model = _build()
    tok = ByteTokenizer(380)
    cfg = G.GlinerConfig.from_files({"max_width": 4, "max_length": 128, "threshold": 0.3},
                                    {"[P]": 389, "[E]": 390, "[C]": 392, "[R]": 393, "[SEP_TEXT]": 391})
    pipe = G.GlinerPipeline(model, tok, cfg)
    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register("tiny-gliner", "recognizer", pipe, tok)
    c = TestClient(create_app(mgr))
    text = "Zoë met Bob in Paris"
    r = c.post("/ai/v1/extract", json={"model": "tiny-gliner", "inputs": [{"id": "a", "content": text}], "schema": {
        "entities": ["person", "city"], "relations": [{"type": "lives in"}],
        "classifications": [{"name": "topic", "labels": ["travel", "sport"]}]}})
    assert r.status_code == 200, r.text
    rec = r.json()["data"][0]
    want = pipe.recognize([text], ["person", "city"])[0]
    assert [(e["label"], e["text"]) for e in rec["entities"]] == [(e.label, e.text) for e in want]
    for e in rec["entities"]:
        assert text[e["start"]:e["end"]] == e["text"]          # character offsets, although "ë" is two bytes
    assert isinstance(rec["relations"], list)
    assert len(rec["classifications"]) == 1 and rec["classifications"][0]["label"] in ("travel", "sport")


def test_extract_resolve_option_builds_a_graph():
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    class Fake:                                   # a span model stand-in with fixed answers
        def recognize(self, texts, labels, threshold=None):
            E = G.GlinerEntity
            return [[E("Ada Lovelace", "person", 0, 12, 0.9), E("London", "city", 20, 26, 0.8)],
                    [E("ada lovelace", "person", 0, 12, 0.7)]][: len(texts)]

        def extract_relations(self, texts, ents, rels):
            e = self.recognize(texts, ents)
            return e, [[G.GlinerRelation(e[0][0], e[0][1], "lives in", 0.6)], []][: len(texts)]

        def classify(self, *a, **k):
            return []

    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register("fake", "recognizer", Fake(), None)
    c = TestClient(create_app(mgr))
    r = c.post("/ai/v1/extract", json={"model": "fake", "inputs": [{"content": "Ada Lovelace lived in London"},
                                                                    {"content": "ada lovelace again"}],
                                       "schema": {"entities": ["person", "city"], "relations": [{"type": "lives in"}]},
                                       "options": {"resolve": True}})
    assert r.status_code == 200, r.text
    kg = r.json()["knowledge_graph"]
    assert [e["name"] for e in kg["entities"]] == ["Ada Lovelace", "London"] and kg["entities"][0]["inputs"] == [0, 1]
    assert kg["relations"] == [{"source": "entity-0", "target": "entity-1", "type": "lives in", "score": 0.6,
                                "inputs": [0]}]


def test_extract_resolver_options_filter_and_shape_the_graph():
    """min_entity_confidence / min_relation_confidence drop weak mentions and relations, track_provenance switches
    the mention lists off, options may sit under options.resolver."""
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    class Fake:
        def recognize(self, texts, labels, threshold=None):
            E = G.GlinerEntity
            return [[E("Ada Lovelace", "person", 0, 12, 0.9), E("London", "city", 20, 26, 0.4)]][: len(texts)]

        def extract_relations(self, texts, ents, rels):
            e = self.recognize(texts, ents)
            return e, [[G.GlinerRelation(e[0][0], e[0][1], "lives in", 0.3)]][: len(texts)]

        def classify(self, *a, **k):
            return []

    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register("fake", "recognizer", Fake(), None)
    c = TestClient(create_app(mgr))
    body = {"model": "fake", "inputs": [{"content": "Ada Lovelace lived in London"}],
            "schema": {"entities": ["person", "city"], "relations": [{"type": "lives in"}]}}
    kg = c.post("/ai/v1/extract", json={**body, "options": {"resolve": True, "track_provenance": False}}
                ).json()["knowledge_graph"]
    assert len(kg["entities"]) == 2 and kg["entities"][0]["mentions"] is None and len(kg["relations"]) == 1
    kg = c.post("/ai/v1/extract", json={**body, "options": {"resolve": True, "resolver": {"min_entity_confidence": 0.5}}}
                ).json()["knowledge_graph"]
    assert [e["name"] for e in kg["entities"]] == ["Ada Lovelace"] and kg["relations"] == []   # London fell out
    kg = c.post("/ai/v1/extract", json={**body, "options": {"resolve": True, "min_relation_confidence": 0.5}}
                ).json()["knowledge_graph"]
    assert len(kg["entities"]) == 2 and kg["relations"] == []
