"""Classification / NER pipelines, the HBM planner and the parallel-strategy planner (all host-side logic)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models.bert import BertConfig, BertModel, pack_sequences
from antfly_b200.models.llama import LlamaConfig
from antfly_b200.parallel.strategy import plan_parallel
from antfly_b200.pipelines.classification import Entity, TextClassifier, TokenClassifier, aggregate_bio
from antfly_b200.runtime.memory import estimate_generation, plan_kv_blocks


def test_bio_aggregation_rules():
    tags = ["O", "B-PER", "I-PER", "O", "I-LOC", "I-LOC", "B-LOC", "I-ORG", "O"]
    ents = aggregate_bio(tags, [0.9] * len(tags))
    assert [(e.label, e.start_token, e.end_token) for e in ents] == [("PER", 1, 3), ("LOC", 4, 6), ("LOC", 6, 7),
                                                                      ("ORG", 7, 8)]
    # special tokens split entities; continuation pieces extend the open one regardless of their own tag
    ents = aggregate_bio(["B-PER", "O", "I-PER", "B-LOC"], [1.0, 0.2, 0.8, 0.6], is_special=[False, False, True, False],
                         is_continuation=[False, True, False, False])
    assert [(e.label, e.start_token, e.end_token) for e in ents] == [("PER", 0, 2), ("LOC", 3, 4)]
    assert abs(ents[0].score - 0.6) < 1e-6


def test_token_classifier_matches_transformers():
    torch.manual_seed(0)
    labels = ["O", "B-PER", "I-PER", "B-LOC", "I-LOC"]
    hf_cfg = transformers.BertConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                     intermediate_size=128, max_position_embeddings=64, num_labels=len(labels),
                                     hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    hf = transformers.BertForTokenClassification(hf_cfg).eval()
    cfg = BertConfig.from_hf(hf_cfg.to_dict())
    cfg.num_labels = len(labels)
    model = BertModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    seqs = [[101] + torch.randint(103, 300, (n,)).tolist() + [102] for n in (6, 13)]
    got = model.token_logits(pack_sequences(seqs, None)).float()
    o = 0
    for s in seqs:
        with torch.no_grad():
            want = hf(input_ids=torch.tensor([s])).logits[0]
        torch.testing.assert_close(got[o:o + len(s)], want, atol=2e-2, rtol=2e-2)
        o += len(s)
    tagger = TokenClassifier(model, dict(enumerate(labels)))
    ents = tagger.entities_ids(seqs, special_ids=[101, 102])
    assert len(ents) == 2 and all(isinstance(e, Entity) for row in ents for e in row)
    assert all(0 < e.start_token < e.end_token < len(s) for s, row in zip(seqs, ents) for e in row)


def test_text_classifier_probabilities():
    cfg = BertConfig(vocab_size=200, hidden_size=64, num_hidden_layers=1, num_attention_heads=4,
                     intermediate_size=128, max_position_embeddings=64, num_labels=3)
    model = BertModel.random_init(cfg, device="cpu", seed=0, dtype=torch.float32)
    clf = TextClassifier(model, id2label={0: "neg", 1: "neu", 2: "pos"})
    out = clf.classify_ids([[101, 5, 6, 102], [101, 9, 102]], top_k=3)
    assert len(out) == 2 and abs(sum(d["score"] for d in out[0]) - 1.0) < 1e-5
    assert {d["label"] for d in out[0]} == {"neg", "neu", "pos"}


def test_memory_planner():
    cfg = LlamaConfig.llama3_8b()
    est = estimate_generation(cfg)
    assert 8.0e9 < est.weight_bytes < 10.5e9              # ~8 B fp8 parameters + bf16 embedding table
    assert est.kv_bytes_per_token == 2 * 32 * 8 * 128 * 2  # K and V, 32 layers, 8 KV heads, bf16
    blocks = plan_kv_blocks(cfg, max_seq_len=8192)
    assert blocks * 16 * est.kv_bytes_per_token < 180e9 and blocks * 16 > 64 * 2304  # the headline workload fits
    est8 = estimate_generation(LlamaConfig.llama3_70b(), tp_size=8)
    assert est8.kv_bytes_per_token == 2 * 80 * 1 * 128 * 2 and est8.weight_bytes < 15e9
    with pytest.raises(MemoryError):
        plan_kv_blocks(LlamaConfig.llama3_70b(), hbm_bytes=40 * 10 ** 9, tp_size=1)


def test_parallel_strategy_planner():
    cfg = LlamaConfig.llama3_8b()
    assert plan_parallel(cfg, 1).strategy == "single"
    p = plan_parallel(cfg, 8)
    assert p.strategy == "tensor" and [r.tp_rank for r in p.ranks] == list(range(8)) and all(
        r.layers == (0, 32) for r in p.ranks)
    pp = plan_parallel(cfg, 3, "pipeline")
    assert [r.layers for r in pp.ranks] == [(0, 11), (11, 22), (22, 32)]
    assert pp.ranks[0].holds_embedding and not pp.ranks[0].holds_lm_head and pp.ranks[2].holds_lm_head
    with pytest.raises(ValueError):
        plan_parallel(cfg, 3, "tensor")
    assert plan_parallel(cfg, 3).strategy == "pipeline"
    assert plan_parallel(LlamaConfig.llama3_70b(), 8).notes == []      # 8 KV heads over 8 ranks: nothing replicated
    small_kv = LlamaConfig(num_attention_heads=32, num_key_value_heads=4, intermediate_size=14336)
    assert any("replicated" in n for n in plan_parallel(small_kv, 8).notes)


def test_sentencepiece_tokenizer_roundtrip_and_token_bytes(tmp_path):
    spm = pytest.importorskip("sentencepiece")
    from antfly_b200.tokenizer.tokenizer import SentencePieceTokenizer, load_tokenizer

    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(["the quick brown fox jumps over the lazy dog", "json {\"key\": [1, 2, 3]}",
                                 "vector search with paged attention", "hello world, hello tokens"] * 30))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "tokenizer"), vocab_size=340,
                                   model_type="bpe", byte_fallback=True, character_coverage=1.0,
                                   minloglevel=2)
    tok = load_tokenizer(str(tmp_path))
    assert isinstance(tok, SentencePieceTokenizer) and tok.vocab_size == 340
    text = "hello brown json {\"key\": 7} é"
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    # the per-token byte strings concatenate to the text (with SentencePiece's leading word-boundary space)
    joined = b"".join(tok.token_bytes(i) for i in ids).decode("utf-8")
    assert joined.lstrip(" ") == text
    assert tok.token_bytes(tok.special.eos_id) == b""


def test_clip_embedder_pipeline(tmp_path):
    import numpy as np

    from antfly_b200.models.clip import ClipConfig, ClipModel
    from antfly_b200.pipelines.multimodal import ClipEmbedder, load_image

    torch.manual_seed(0)
    hf_cfg = transformers.CLIPConfig(
        text_config=dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                         num_attention_heads=4, max_position_embeddings=16),
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                           image_size=32, patch_size=16), projection_dim=32)
    hf = transformers.CLIPModel(hf_cfg).eval()
    model = ClipModel.from_state_dict(ClipConfig.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                      dtype=torch.float32)
    emb = ClipEmbedder(model)
    rng = np.random.default_rng(0)
    arr = rng.integers(0, 256, size=(50, 70, 3), dtype=np.uint8)
    imgs = [arr, torch.from_numpy(rng.integers(0, 256, size=(33, 33, 4), dtype=np.uint8)), arr[:, :, 0]]
    pil = pytest.importorskip("PIL.Image")
    path = tmp_path / "img.png"
    pil.fromarray(arr).save(path)
    imgs.append(str(path))
    e = emb.embed_images(imgs)
    assert e.shape == (4, 32) and torch.allclose(e.norm(dim=-1), torch.ones(4), atol=1e-4)
    torch.testing.assert_close(e[0], e[3], atol=1e-5, rtol=1e-5)     # the PNG round trip is lossless
    assert load_image(arr[:, :, 0]).shape == (50, 70, 3)
    t = emb.embed_token_ids([[298, 5, 6, 299], [298, 7, 299]])
    assert t.shape == (2, 32) and (t @ e.T).shape == (2, 4)


def test_seq2seq_pipeline_t5_greedy_and_streaming():
    """Encoder-decoder text-to-text pipeline: same output as the model's own greedy loop, streamed deltas
    concatenate to the final text, chat messages are flattened."""
    import torch

    from antfly_b200.models.t5 import T5Config, T5Model
    from antfly_b200.pipelines.seq2seq import Seq2SeqGenerator
    from antfly_b200.runtime.sampling_params import SamplingParams
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    cfg = T5Config(vocab_size=300, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4,
                   relative_attention_num_buckets=8, relative_attention_max_distance=20, eos_token_id=2)
    g = torch.Generator().manual_seed(0)
    sd = {"shared.weight": torch.randn(300, 64, generator=g)}
    for stack, ff in (("encoder", 1), ("decoder", 2)):
        for l in range(2):
            s = f"{stack}.block.{l}.layer."
            for n in "qkvo":
                sd[s + f"0.SelfAttention.{n}.weight"] = torch.randn(64, 64, generator=g) * 0.2
                if stack == "decoder":
                    sd[s + f"1.EncDecAttention.{n}.weight"] = torch.randn(64, 64, generator=g) * 0.2
            sd[s + "0.layer_norm.weight"] = torch.ones(64)
            if stack == "decoder":
                sd[s + "1.layer_norm.weight"] = torch.ones(64)
            sd[s + f"{ff}.DenseReluDense.wi.weight"] = torch.randn(128, 64, generator=g) * 0.2
            sd[s + f"{ff}.DenseReluDense.wo.weight"] = torch.randn(64, 128, generator=g) * 0.2
            sd[s + f"{ff}.layer_norm.weight"] = torch.ones(64)
        sd[f"{stack}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"] = torch.randn(8, 4, generator=g)
        sd[f"{stack}.final_layer_norm.weight"] = torch.ones(64)
    model = T5Model.from_state_dict(cfg, sd, device="cpu", dtype=torch.float32)
    tok = ByteTokenizer(vocab_size=300)
    pipe = Seq2SeqGenerator(model, tok)
    deltas = []
    out = pipe.generate("rewrite: where is the cat", SamplingParams(max_tokens=12), on_delta=deltas.append)
    ids = pipe._encode("rewrite: where is the cat")
    assert ids[-1] == 2 and out.token_ids == model.generate(ids, max_new_tokens=12)
    assert out.completion_tokens == len(out.token_ids) <= 12 and out.prompt_tokens == len(ids)
    assert "".join(deltas) == out.text or out.text.endswith("�")
    out2 = pipe.generate([{"role": "user", "content": "rewrite: where is the cat"}], SamplingParams(max_tokens=12))
    assert out2.token_ids == out.token_ids


def test_relation_triplets_are_parsed_from_linearised_text():
    from antfly_b200.pipelines.relations import Triplet, parse_triplets, to_extraction

    text = ("<s><triplet> Punta Cana <subj> Dominican Republic <obj> country <subj> La Altagracia <obj> located in "
            "<triplet> Dominican Republic <subj> Punta Cana <obj> contains <triplet> dangling <subj> no relation</s>")
    tr = parse_triplets(text)
    assert tr == [Triplet("Punta Cana", "country", "Dominican Republic"),
                  Triplet("Punta Cana", "located in", "La Altagracia"),
                  Triplet("Dominican Republic", "contains", "Punta Cana")]
    assert parse_triplets("no markers at all") == [] and parse_triplets("<triplet> a <subj> b") == []
    assert parse_triplets("<triplet> a <subj> b <obj> r <triplet> a <subj> b <obj> r") == [Triplet("a", "r", "b")]
    src = "Punta Cana is a resort town in the Dominican Republic."
    ents, rels = to_extraction(tr, src, allowed=["COUNTRY", "contains"])
    assert [e["text"] for e in ents] == ["Punta Cana", "Dominican Republic"]
    assert src[ents[1]["start"]:ents[1]["end"]] == "Dominican Republic"
    assert rels == [{"type": "country", "source": {"entity_index": 0}, "target": {"entity_index": 1}},
                    {"type": "contains", "source": {"entity_index": 1}, "target": {"entity_index": 0}}]


def test_seq2seq_pipeline_drives_bart_with_a_forced_first_token():
    import torch

    transformers = __import__("pytest").importorskip("transformers")
    from antfly_b200.models.bart import BartConfig, BartModel
    from antfly_b200.pipelines.seq2seq import Seq2SeqGenerator
    from antfly_b200.runtime.sampling_params import SamplingParams
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    torch.manual_seed(0)
    hf_cfg = transformers.BartConfig(vocab_size=300, d_model=64, encoder_layers=1, decoder_layers=1,
                                     encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=128,
                                     decoder_ffn_dim=128, max_position_embeddings=64)
    cfg = BartConfig.from_hf({**hf_cfg.to_dict(), "forced_bos_token_id": 0})       # as in mBART-style config.json
    assert cfg.forced_bos_token_id == 0
    model = BartModel.from_state_dict(cfg, transformers.BartForConditionalGeneration(hf_cfg).state_dict(),
                                      device="cpu", dtype=torch.float32)
    pipe = Seq2SeqGenerator(model, ByteTokenizer(vocab_size=300))
    out = pipe.generate("summarize: a long story", SamplingParams(max_tokens=6))
    assert out.token_ids == model.generate(pipe._encode("summarize: a long story"), max_new_tokens=6)
