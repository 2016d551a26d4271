"""Architecture parity on CPU against Hugging Face `transformers` reference implementations with random weights:
decoder families (Llama GQA, Qwen2 with QKV bias, Qwen3 with per-head Q/K RMS norm and an explicit head size,
Mistral with a sliding window) through prefill + decode over the paged KV cache, and the BERT encoder with mean
pooling and a classification head.  The decoder's linear weights are block-fp8 in this engine, so the HF model
gets the same weights rounded to that grid first; what is compared is the wiring (RoPE convention, GQA, norms,
biases, masks, weight tying), not the quantiser."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models.bert import BertConfig, BertModel, pack_sequences
from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch
from antfly_b200.ops import reference as R


def _round_linears_to_fp8_grid(model):
    with torch.no_grad():
        for name, mod in model.named_modules():
            if isinstance(mod, torch.nn.Linear):
                q, e8 = R.quantize_block_fp8(mod.weight.data)
                mod.weight.data.copy_(R.dequantize_block_fp8(q, e8))
        for name, p in model.named_parameters():
            if p.dim() == 3 and "experts" in name:      # fused expert weights [E, out, in]
                for e in range(p.shape[0]):
                    q, e8 = R.quantize_block_fp8(p.data[e])
                    p.data[e].copy_(R.dequantize_block_fp8(q, e8))
            elif name.endswith("mlp.gate.weight") or name.endswith("shared_expert_gate.weight"):
                p.data.copy_(p.data.to(torch.bfloat16).float())   # router weights are kept in bf16


def _hf_decoder(kind: str):
    common = dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-5,
                  rope_theta=10000.0, tie_word_embeddings=False, attention_dropout=0.0)
    if kind == "llama":
        cfg = transformers.LlamaConfig(**common)
        m = transformers.LlamaForCausalLM(cfg)
    elif kind == "qwen2":
        cfg = transformers.Qwen2Config(**common)
        m = transformers.Qwen2ForCausalLM(cfg)
    elif kind == "qwen3":
        cfg = transformers.Qwen3Config(**common, head_dim=64)
        m = transformers.Qwen3ForCausalLM(cfg)
    elif kind == "mistral":
        cfg = transformers.MistralConfig(**common, sliding_window=8)
        m = transformers.MistralForCausalLM(cfg)
    elif kind == "gemma":
        cfg = transformers.GemmaConfig(**{**common, "head_dim": 64, "hidden_activation": "gelu_pytorch_tanh"})
        m = transformers.GemmaForCausalLM(cfg)
    elif kind == "gemma2":
        cfg = transformers.Gemma2Config(**{**common, "head_dim": 64, "query_pre_attn_scalar": 48, "sliding_window": 8,
                                           "num_hidden_layers": 3, "attn_logit_softcapping": 4.0,
                                           "final_logit_softcapping": 3.0,
                                           "hidden_activation": "gelu_pytorch_tanh"})
        cfg.tie_word_embeddings = False
        m = transformers.Gemma2ForCausalLM(cfg)
    elif kind == "gemma3":
        cfg = transformers.Gemma3TextConfig(**{**common, "head_dim": 64, "query_pre_attn_scalar": 48,
                                               "sliding_window": 8, "num_hidden_layers": 3,
                                               "layer_types": ["sliding_attention", "full_attention",
                                                               "sliding_attention"],
                                               "rope_parameters": {
                                                   "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                                   "full_attention": {"rope_type": "linear", "factor": 4.0,
                                                                      "rope_theta": 1000000.0}}})
        cfg.tie_word_embeddings = False
        m = transformers.Gemma3ForCausalLM(cfg)
    elif kind == "phi3":
        cfg = transformers.Phi3Config(**{**common, "pad_token_id": 0})
        m = transformers.Phi3ForCausalLM(cfg)
    elif kind == "mixtral":
        cfg = transformers.MixtralConfig(**common, num_local_experts=4, num_experts_per_tok=2)
        m = transformers.MixtralForCausalLM(cfg)
    elif kind == "qwen2_moe":
        cfg = transformers.Qwen2MoeConfig(**common, moe_intermediate_size=96, shared_expert_intermediate_size=160,
                                          num_experts=4, num_experts_per_tok=2, decoder_sparse_step=1,
                                          mlp_only_layers=[])
        m = transformers.Qwen2MoeForCausalLM(cfg)
    elif kind == "qwen3_moe":
        cfg = transformers.Qwen3MoeConfig(**common, head_dim=64, moe_intermediate_size=96, num_experts=4,
                                          num_experts_per_tok=2, decoder_sparse_step=1, mlp_only_layers=[],
                                          norm_topk_prob=True)
        m = transformers.Qwen3MoeForCausalLM(cfg)
    elif kind == "llama31":
        cfg = transformers.LlamaConfig(**common, rope_parameters={
            "rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0, "low_freq_factor": 1.0,
            "high_freq_factor": 4.0, "original_max_position_embeddings": 32})
        m = transformers.LlamaForCausalLM(cfg)
    elif kind == "llama_yarn":
        cfg = transformers.LlamaConfig(**common, rope_parameters={
            "rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0, "original_max_position_embeddings": 64,
            "beta_fast": 8.0, "beta_slow": 1.0})
        m = transformers.LlamaForCausalLM(cfg)
    elif kind == "phi3_long":
        g = torch.Generator().manual_seed(5)
        cfg = transformers.Phi3Config(**{**common, "pad_token_id": 0, "original_max_position_embeddings": 64,
                                         "rope_parameters": {
                                             "rope_type": "longrope", "rope_theta": 10000.0,
                                             "short_factor": (1.0 + torch.rand(16, generator=g)).tolist(),
                                             "long_factor": (2.0 + torch.rand(16, generator=g)).tolist()}})
        m = transformers.Phi3ForCausalLM(cfg)
    elif kind == "llama_tied":
        common["tie_word_embeddings"] = True
        cfg = transformers.LlamaConfig(**common)
        m = transformers.LlamaForCausalLM(cfg)
    else:
        raise ValueError(kind)
    return cfg, m.eval().float()


@pytest.mark.parametrize("kind", ["llama", "qwen2", "qwen3", "mistral", "llama_tied", "gemma", "gemma2", "gemma3", "phi3",
                                  "mixtral", "qwen2_moe", "qwen3_moe", "llama31", "llama_yarn", "phi3_long"])
def test_decoder_matches_transformers(kind):
    torch.manual_seed(0)
    hf_cfg, hf = _hf_decoder(kind)
    with torch.no_grad():  # make biases and norm gains non-trivial
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
            elif "norm" in n:
                p.uniform_(-0.3, 0.3) if kind.startswith("gemma") else p.uniform_(0.5, 1.5)
    _round_linears_to_fp8_grid(hf)
    cfg = LlamaConfig.from_hf(hf_cfg.to_dict())
    if kind == "llama_tied":
        assert cfg.tie_word_embeddings
    if kind in ("llama31", "llama_yarn", "phi3_long"):                  # a frequency table replaces the closed form
        assert cfg.rope_inv_freq is not None and len(cfg.rope_inv_freq) == cfg.rope_dim // 2
        assert (cfg.rope_mscale > 1.0) == (kind != "llama31")
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    if kind == "llama_tied":
        sd.pop("lm_head.weight", None)
    model = LlamaModel.from_state_dict(cfg, sd, device="cpu")

    S, page = 24, 16
    ids = torch.randint(0, hf_cfg.vocab_size, (S + 1,))
    with torch.no_grad():
        want = hf(ids[None]).logits[0].float()  # [S + 1, V]

    nblk = 3
    k_cache = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    table = torch.arange(nblk, dtype=torch.int32)[None]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    pos = torch.arange(S, dtype=torch.int32)
    prefill = StepBatch(ids[:S].int(), pos, pos.clone(), i32([0]), i32([S]), i32([S]), table, pos.clone(), S, 1)
    got_prefill = model.forward(prefill, k_cache, v_cache).float()
    decode = StepBatch(ids[S:].int(), i32([S]), i32([S]), i32([0]), i32([1]), i32([S + 1]), table, i32([0]), 1, 1)
    got_decode = model.forward(decode, k_cache, v_cache).float()
    got = torch.cat([got_prefill, got_decode], 0)

    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.99, (kind, cos)
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean()
    assert float(agree) >= 0.8, (kind, float(agree))
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) < 0.08 * max(scale, 1.0), (kind, float((got - want).abs().max()), scale)
    if kind in ("llama_yarn", "phi3_long"):
        # with the closed-form frequencies instead of the table the error is three to four times this bound
        assert float((got - want).abs().max()) < 0.012, float((got - want).abs().max())


@pytest.mark.parametrize("head", [False, True])
def test_bert_matches_transformers(head):
    torch.manual_seed(1)
    hf_cfg = transformers.BertConfig(vocab_size=400, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                     intermediate_size=128, max_position_embeddings=64, num_labels=3,
                                     hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    hf = (transformers.BertForSequenceClassification(hf_cfg) if head else transformers.BertModel(hf_cfg)).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
    cfg = BertConfig.from_hf(hf_cfg.to_dict())
    model = BertModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    seqs = [[101] + torch.randint(103, 400, (n,)).tolist() + [102] for n in (5, 17, 30)]
    types = [[0] * (len(s) // 2) + [1] * (len(s) - len(s) // 2) for s in seqs]
    batch = pack_sequences(seqs, types)
    L = max(len(s) for s in seqs)
    ids = torch.zeros((len(seqs), L), dtype=torch.long)
    tt = torch.zeros_like(ids)
    mask = torch.zeros_like(ids)
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.tensor(s)
        tt[i, : len(s)] = torch.tensor(types[i])
        mask[i, : len(s)] = 1
    with torch.no_grad():
        out = hf(input_ids=ids, token_type_ids=tt, attention_mask=mask)
    if head:
        got = model.classify(batch).float()
        torch.testing.assert_close(got, out.logits.float(), atol=3e-2, rtol=3e-2)
    else:
        hidden = out.last_hidden_state
        want = (hidden * mask[..., None]).sum(1) / mask.sum(1, keepdim=True)
        want = torch.nn.functional.normalize(want, dim=-1)
        got = model.embed(batch, pooling="mean", normalize=True).float()
        cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
        assert float(cos.min()) > 0.999, cos


def _hf_gpt(kind: str):
    if kind == "gpt2":
        cfg = transformers.GPT2Config(vocab_size=300, n_positions=64, n_embd=64, n_layer=2, n_head=4,
                                      resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        return cfg, transformers.GPT2LMHeadModel(cfg)
    if kind.startswith("neox"):
        cfg = transformers.GPTNeoXConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                         intermediate_size=128, max_position_embeddings=64, rotary_pct=0.25,
                                         use_parallel_residual=kind == "neox_parallel", hidden_dropout=0.0,
                                         attention_dropout=0.0, tie_word_embeddings=False)
        return cfg, transformers.GPTNeoXForCausalLM(cfg)
    if kind == "gptj":
        cfg = transformers.GPTJConfig(vocab_size=300, n_positions=64, n_embd=64, n_layer=2, n_head=4, rotary_dim=8,
                                      resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        return cfg, transformers.GPTJForCausalLM(cfg)
    if kind == "phi":
        cfg = transformers.PhiConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                     num_attention_heads=4, max_position_embeddings=64, partial_rotary_factor=0.5,
                                     resid_pdrop=0.0, embd_pdrop=0.0, attention_dropout=0.0)
        return cfg, transformers.PhiForCausalLM(cfg)
    if kind == "bloom":
        cfg = transformers.BloomConfig(vocab_size=300, hidden_size=64, n_layer=2, n_head=6 if False else 4,
                                       hidden_dropout=0.0, attention_dropout=0.0)
        return cfg, transformers.BloomForCausalLM(cfg)
    if kind == "bloom6":
        cfg = transformers.BloomConfig(vocab_size=300, hidden_size=96, n_layer=2, n_head=6, hidden_dropout=0.0,
                                       attention_dropout=0.0)
        return cfg, transformers.BloomForCausalLM(cfg)
    if kind == "gpt_neo":
        cfg = transformers.GPTNeoConfig(vocab_size=300, hidden_size=64, num_layers=4, num_heads=4, intermediate_size=128,
                                        max_position_embeddings=64, window_size=6,
                                        attention_types=[[["global", "local"], 2]], resid_dropout=0.0,
                                        embed_dropout=0.0, attention_dropout=0.0)
        return cfg, transformers.GPTNeoForCausalLM(cfg)
    if kind.startswith("falcon"):
        kw = {"falcon_mq": dict(multi_query=True, parallel_attn=True, new_decoder_architecture=False),
              "falcon_mha": dict(multi_query=False, parallel_attn=True, new_decoder_architecture=False),
              "falcon_new": dict(new_decoder_architecture=True, num_kv_heads=2),
              "falcon_seq": dict(multi_query=True, parallel_attn=False, new_decoder_architecture=False,
                                 bias=True)}[kind]
        cfg = transformers.FalconConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                        alibi=False, hidden_dropout=0.0, attention_dropout=0.0,
                                        max_position_embeddings=64, **kw)
        return cfg, transformers.FalconForCausalLM(cfg)
    cfg = transformers.OPTConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                 ffn_dim=128, max_position_embeddings=64, word_embed_proj_dim=64, dropout=0.0,
                                 attention_dropout=0.0)
    return cfg, transformers.OPTForCausalLM(cfg)


@pytest.mark.parametrize("kind", ["gpt2", "neox_parallel", "neox_sequential", "opt", "gptj", "phi", "gpt_neo",
                                  "falcon_mq", "falcon_mha", "falcon_new", "falcon_seq", "bloom", "bloom6"])
def test_layernorm_decoders_match_transformers(kind):
    from antfly_b200.models.gpt import GptConfig, GptModel

    torch.manual_seed(2)
    hf_cfg, hf = _hf_gpt(kind)
    hf = hf.eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
    cfg = GptConfig.from_hf(hf_cfg.to_dict())
    model = GptModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    S, page, nblk = 20, 16, 2
    ids = torch.randint(0, hf_cfg.vocab_size, (S + 1,))
    with torch.no_grad():
        want = hf(ids[None]).logits[0].float()
    k_cache = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, model.D), dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    table = torch.arange(nblk, dtype=torch.int32)[None]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    pos = torch.arange(S, dtype=torch.int32)
    got = torch.cat([
        model.forward(StepBatch(ids[:S].int(), pos, pos.clone(), i32([0]), i32([S]), i32([S]), table, pos.clone(),
                                S, 1), k_cache, v_cache).float(),
        model.forward(StepBatch(ids[S:].int(), i32([S]), i32([S]), i32([0]), i32([1]), i32([S + 1]), table,
                                i32([0]), 1, 1), k_cache, v_cache).float()], 0)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.995, (kind, cos)
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.85


@pytest.mark.parametrize("kind", ["roberta", "xlm-roberta"])
def test_roberta_family_matches_transformers(kind):
    """Position ids start after the padding index, one token type, same encoder otherwise."""
    torch.manual_seed(3)
    C, M = ((transformers.RobertaConfig, transformers.RobertaModel) if kind == "roberta"
            else (transformers.XLMRobertaConfig, transformers.XLMRobertaModel))
    hf_cfg = C(vocab_size=400, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
               max_position_embeddings=70, type_vocab_size=1, pad_token_id=1, hidden_dropout_prob=0.0,
               attention_probs_dropout_prob=0.0)
    hf = M(hf_cfg, add_pooling_layer=False).eval()
    cfg = BertConfig.from_hf(hf_cfg.to_dict())
    assert cfg.position_offset == 2
    model = BertModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    seqs = [[0] + torch.randint(3, 400, (n,)).tolist() + [2] for n in (4, 19, 33)]
    batch = pack_sequences(seqs, None, position_offset=cfg.position_offset)
    L = max(len(s) for s in seqs)
    ids = torch.full((len(seqs), L), 1, dtype=torch.long)
    mask = torch.zeros_like(ids)
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.tensor(s)
        mask[i, : len(s)] = 1
    with torch.no_grad():
        hidden = hf(input_ids=ids, attention_mask=mask).last_hidden_state
    want = torch.nn.functional.normalize((hidden * mask[..., None]).sum(1) / mask.sum(1, keepdim=True), dim=-1)
    got = model.embed(batch, pooling="mean", normalize=True).float()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.999, cos


def test_clip_text_and_vision_towers_match_transformers():
    from antfly_b200.models.clip import ClipConfig, ClipModel
    from antfly_b200.ops import image_ops as I

    torch.manual_seed(4)
    hf_cfg = transformers.CLIPConfig(
        text_config=dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, max_position_embeddings=24, eos_token_id=2, bos_token_id=0,
                         pad_token_id=1, attention_dropout=0.0),
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                           image_size=32, patch_size=8, attention_dropout=0.0),
        projection_dim=48)
    hf = transformers.CLIPModel(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
    cfg = ClipConfig.from_hf(hf_cfg.to_dict())
    assert cfg.text.hidden_act == "quick_gelu" and cfg.vision.patch_size == 8 and cfg.projection_dim == 48
    model = ClipModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)

    # text: sequences of different lengths, the end-of-text token has the highest id (original tokenizer layout)
    seqs = [[298] + torch.randint(3, 290, (n,)).tolist() + [299] for n in (3, 9, 15)]
    L = max(len(s) for s in seqs)
    ids = torch.full((len(seqs), L), 1, dtype=torch.long)
    mask = torch.zeros_like(ids)
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.tensor(s)
        mask[i, : len(s)] = 1
    with torch.no_grad():
        want_t = hf.get_text_features(input_ids=ids, attention_mask=mask)
    want_t = getattr(want_t, "pooler_output", want_t)
    got_t = model.embed_text(seqs, normalize=False)
    # (the CPU path rounds every GEMM output to bf16 like the kernels do: compare directions and magnitudes)
    assert float(torch.nn.functional.cosine_similarity(got_t, want_t.float(), dim=-1).min()) > 0.9995
    torch.testing.assert_close(got_t, want_t.float(), atol=3e-2, rtol=3e-2)

    # vision: uint8 images through our preprocessing, the same pixels into the reference
    g = torch.Generator().manual_seed(0)
    imgs = torch.randint(0, 256, (2, 40, 52, 3), generator=g, dtype=torch.uint8)
    pixels = I.clip_preprocess(imgs, size=32, mode="bicubic")
    with torch.no_grad():
        want_v = hf.get_image_features(pixel_values=pixels)
    want_v = getattr(want_v, "pooler_output", want_v)
    got_v = model.embed_images(pixels, normalize=False)
    assert float(torch.nn.functional.cosine_similarity(got_v, want_v.float(), dim=-1).min()) > 0.9995
    torch.testing.assert_close(got_v, want_v.float(), atol=3e-2, rtol=3e-2)
    # normalised embeddings give the usual similarity matrix
    sim = model.embed_text(seqs) @ model.embed_images(pixels).T
    assert sim.shape == (3, 2) and float(sim.abs().max()) <= 1.0 + 1e-5


def test_decoder_embedder_last_token_pooling_matches_transformers():
    """Qwen3-Embedding style: last-token hidden state after the final norm, L2-normalised."""
    from antfly_b200.pipelines.embedding import DecoderEmbedder

    torch.manual_seed(5)
    hf_cfg, hf = _hf_decoder("qwen3")
    _round_linears_to_fp8_grid(hf)
    model = LlamaModel.from_state_dict(LlamaConfig.from_hf(hf_cfg.to_dict()),
                                       {k: v.detach().clone() for k, v in hf.state_dict().items()}, device="cpu")
    seqs = [torch.randint(0, 320, (n,)).tolist() for n in (7, 21, 12)]
    emb = DecoderEmbedder(model)
    got = emb.embed_ids(seqs)
    want = []
    for s in seqs:
        with torch.no_grad():
            h = hf.model(torch.tensor([s])).last_hidden_state[0, -1]
        want.append(torch.nn.functional.normalize(h.float(), dim=-1))
    want = torch.stack(want)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.995, cos
    assert emb.embed_ids(seqs, dimensions=32).shape == (3, 32)
    assert model.return_hidden is False


@pytest.mark.parametrize("head", ["embed", "sequence", "token"])
def test_modernbert_matches_transformers(head):
    """Alternating global / local (two-sided window) attention with two rotary bases, pre-norm blocks, gated-GELU
    MLP, prediction head; sequences longer than the local window so the window mask matters."""
    from antfly_b200.models.modernbert import ModernBertConfig, ModernBertModel

    torch.manual_seed(2)
    hf_cfg = transformers.ModernBertConfig(vocab_size=400, hidden_size=64, num_hidden_layers=4,
                                           num_attention_heads=4, intermediate_size=96,
                                           max_position_embeddings=128, local_attention=16,
                                           global_attn_every_n_layers=3, num_labels=3, pad_token_id=0,
                                           bos_token_id=1, eos_token_id=2, cls_token_id=1, sep_token_id=2,
                                           attention_dropout=0.0, mlp_dropout=0.0, embedding_dropout=0.0,
                                           classifier_dropout=0.0, classifier_pooling="mean",
                                           attn_implementation="eager")
    cls = {"embed": transformers.ModernBertModel, "sequence": transformers.ModernBertForSequenceClassification,
           "token": transformers.ModernBertForTokenClassification}[head]
    hf = cls(hf_cfg).eval()
    cfg = ModernBertConfig.from_hf(hf_cfg.to_dict())
    assert [cfg.is_global(l) for l in range(4)] == [True, False, False, True]
    model = ModernBertModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    seqs = [[1] + torch.randint(3, 400, (n,)).tolist() + [2] for n in (5, 40, 61)]
    batch = pack_sequences(seqs)
    L = max(len(s) for s in seqs)
    ids = torch.zeros((len(seqs), L), dtype=torch.long)
    mask = torch.zeros_like(ids)
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.tensor(s)
        mask[i, : len(s)] = 1
    with torch.no_grad():
        out = hf(input_ids=ids, attention_mask=mask)
    if head == "sequence":
        torch.testing.assert_close(model.classify(batch).float(), out.logits.float(), atol=3e-2, rtol=3e-2)
    elif head == "token":
        want = torch.cat([out.logits[i, : len(s)] for i, s in enumerate(seqs)])
        torch.testing.assert_close(model.token_logits(batch).float(), want.float(), atol=3e-2, rtol=3e-2)
    else:
        hidden = out.last_hidden_state
        want = torch.nn.functional.normalize((hidden * mask[..., None]).sum(1) / mask.sum(1, keepdim=True), dim=-1)
        got = model.embed(batch, pooling="mean", normalize=True).float()
        cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
        assert float(cos.min()) > 0.999, cos


@pytest.mark.parametrize("variant", ["v3_embed", "v3_sequence", "v2_token"])
def test_deberta_matches_transformers(variant):
    """Disentangled attention (content-to-position and position-to-content terms over log-bucketed relative
    distances), shared or separate position projections, with / without absolute positions and token types."""
    from antfly_b200.models.deberta import DebertaConfig, DebertaModel

    torch.manual_seed(3)
    v3 = variant.startswith("v3")
    hf_cfg = transformers.DebertaV2Config(
        vocab_size=400, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
        max_position_embeddings=64, type_vocab_size=0 if v3 else 2, relative_attention=True,
        position_buckets=16 if v3 else -1, max_relative_positions=-1 if v3 else 24, pos_att_type=["p2c", "c2p"],
        share_att_key=v3, norm_rel_ebd="layer_norm" if v3 else "none", position_biased_input=not v3,
        hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, pooler_dropout=0.0, num_labels=3,
        pooler_hidden_size=64, layer_norm_eps=1e-7)
    cls = {"v3_embed": transformers.DebertaV2Model, "v3_sequence": transformers.DebertaV2ForSequenceClassification,
           "v2_token": transformers.DebertaV2ForTokenClassification}[variant]
    hf = cls(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
    cfg = DebertaConfig.from_hf(hf_cfg.to_dict())
    model = DebertaModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    seqs = [[1] + torch.randint(3, 400, (n,)).tolist() + [2] for n in (5, 28, 45)]
    types = None if v3 else [[0] * (len(s) // 2) + [1] * (len(s) - len(s) // 2) for s in seqs]
    batch = pack_sequences(seqs, types)
    L = max(len(s) for s in seqs)
    ids = torch.zeros((len(seqs), L), dtype=torch.long)
    mask = torch.zeros_like(ids)
    tt = torch.zeros_like(ids)
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.tensor(s)
        mask[i, : len(s)] = 1
        if types:
            tt[i, : len(s)] = torch.tensor(types[i])
    with torch.no_grad():
        out = hf(input_ids=ids, attention_mask=mask, token_type_ids=None if v3 else tt)
    if variant == "v3_sequence":
        torch.testing.assert_close(model.classify(batch).float(), out.logits.float(), atol=3e-2, rtol=3e-2)
    elif variant == "v2_token":
        want = torch.cat([out.logits[i, : len(s)] for i, s in enumerate(seqs)])
        torch.testing.assert_close(model.token_logits(batch).float(), want.float(), atol=3e-2, rtol=3e-2)
    else:
        hidden = out.last_hidden_state
        want = torch.nn.functional.normalize((hidden * mask[..., None]).sum(1) / mask.sum(1, keepdim=True), dim=-1)
        got = model.embed(batch, pooling="mean", normalize=True).float()
        cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
        assert float(cos.min()) > 0.999, cos


@pytest.mark.parametrize("ff,tied", [("relu", True), ("gated-gelu", False)])
def test_t5_matches_transformers(ff, tied):
    """Encoder-decoder with bucketed relative-position bias, unscaled scores, ReLU / gated-GELU FFN, tied (scaled)
    or separate vocabulary projection; teacher-forced logits, incremental decoding with caches, greedy output."""
    from antfly_b200.models.t5 import T5Config, T5Model

    torch.manual_seed(4)
    hf_cfg = transformers.T5Config(vocab_size=300, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_decoder_layers=3,
                                   num_heads=4, relative_attention_num_buckets=8, relative_attention_max_distance=20,
                                   feed_forward_proj=ff, tie_word_embeddings=tied, dropout_rate=0.0,
                                   decoder_start_token_id=0, eos_token_id=1, pad_token_id=0)
    hf = transformers.T5ForConditionalGeneration(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "relative_attention_bias" in n:
                p.normal_(0, 1.0)
            elif "layer_norm" not in n:
                p.mul_(1.5)                                    # default init gives near-uniform logits
    cfg = T5Config.from_hf(hf_cfg.to_dict())
    model = T5Model.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    src = torch.randint(2, 300, (40,)).tolist()
    tgt = [0] + torch.randint(2, 300, (12,)).tolist()
    with torch.no_grad():
        out = hf(input_ids=torch.tensor([src]), decoder_input_ids=torch.tensor([tgt]))
    enc = model.encode(src)
    torch.testing.assert_close(enc.float(), out.encoder_last_hidden_state[0], atol=8e-2, rtol=3e-2)
    state = model.start_decoding(enc)
    full = model.decode(state, tgt)
    ref_l = out.logits[0]
    assert float((full - ref_l).norm() / ref_l.norm()) < 0.02
    assert bool((full.argmax(-1) == ref_l.argmax(-1)).all())
    # token-by-token decoding through the caches gives the same logits as one teacher-forced pass
    state = model.start_decoding(enc)
    step = torch.cat([model.decode(state, [t]) for t in tgt])
    torch.testing.assert_close(step, full, atol=8e-2, rtol=3e-2)    # bf16-rounded activations on both sides
    dec, want = [0], []
    with torch.no_grad():
        for _ in range(10):                                    # greedy decoding by re-running the full decoder
            nxt = int(hf(input_ids=torch.tensor([src]), decoder_input_ids=torch.tensor([dec])).logits[0, -1].argmax())
            if nxt == 1:
                break
            want.append(nxt)
            dec.append(nxt)
    assert model.generate(src, max_new_tokens=10) == want


def test_whisper_matches_transformers():
    """Convolutional stem as GEMMs over unfolded windows, sinusoidal / learned positions, encoder, decoder with
    self- and cross-attention caches, tied output projection, greedy transcription; log-mel front end against the
    Hugging Face feature extractor."""
    import numpy as np

    from antfly_b200.models.whisper import WhisperConfig, WhisperModel
    from antfly_b200.ops import audio_ops as AO

    torch.manual_seed(6)
    hf_cfg = transformers.WhisperConfig(vocab_size=300, num_mel_bins=80, d_model=64, encoder_layers=2,
                                        encoder_attention_heads=4, decoder_layers=2, decoder_attention_heads=4,
                                        encoder_ffn_dim=128, decoder_ffn_dim=128, max_source_positions=100,
                                        max_target_positions=32, dropout=0.0, attention_dropout=0.0,
                                        activation_dropout=0.0, decoder_start_token_id=1, eos_token_id=2,
                                        pad_token_id=0, bos_token_id=1, suppress_tokens=None,
                                        begin_suppress_tokens=None)
    hf = transformers.WhisperForConditionalGeneration(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
            elif "layer_norm" not in n and "embed_positions" not in n:
                p.mul_(2.0)
    cfg = WhisperConfig.from_hf(hf_cfg.to_dict())
    model = WhisperModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    mel = torch.randn(80, 200) * 0.5
    tgt = [1] + torch.randint(3, 300, (9,)).tolist()
    with torch.no_grad():
        out = hf(input_features=mel[None], decoder_input_ids=torch.tensor([tgt]))
    enc = model.encode(mel)
    ref = out.encoder_last_hidden_state[0]
    assert enc.shape == (100, 64) and float((enc.float() - ref).norm() / ref.norm()) < 0.02
    full = model.decode(model.start_decoding(enc), tgt)
    assert float((full - out.logits[0]).norm() / out.logits[0].norm()) < 0.03
    assert float((full.argmax(-1) == out.logits[0].argmax(-1)).float().mean()) >= 0.9
    state = model.start_decoding(enc)
    step = torch.cat([model.decode(state, [t]) for t in tgt])
    assert float((step - full).norm() / full.norm()) < 0.02
    dec, want = [1], []
    with torch.no_grad():
        for _ in range(8):
            nxt = int(hf(input_features=mel[None], decoder_input_ids=torch.tensor([dec])).logits[0, -1].argmax())
            if nxt == 2:
                break
            want.append(nxt)
            dec.append(nxt)
    assert model.transcribe_ids(mel, [1], max_new_tokens=8) == want
    # front end
    fe = transformers.WhisperFeatureExtractor()
    t = torch.arange(16000 * 2) / 16000
    x = 0.3 * torch.sin(2 * np.pi * 440 * t) + 0.05 * torch.randn(t.numel())
    want_f = torch.from_numpy(fe(x.numpy(), sampling_rate=16000, return_tensors="np")["input_features"][0])
    got_f = AO.log_mel(x)
    assert got_f.shape == (80, 3000) and float((got_f - want_f).abs().max()) < 1e-4


@pytest.mark.parametrize("scale", [False, True])
def test_bart_matches_transformers(scale):
    """Post-LayerNorm encoder-decoder with offset learned positions, embedding LayerNorm (and optional embedding
    scale), cross attention, shared output projection with a logit bias; cached decoding and greedy output."""
    from antfly_b200.models.bart import BartConfig, BartModel

    torch.manual_seed(7)
    hf_cfg = transformers.BartConfig(vocab_size=300, d_model=64, encoder_layers=2, decoder_layers=2,
                                     encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=128,
                                     decoder_ffn_dim=128, max_position_embeddings=64, scale_embedding=scale,
                                     dropout=0.0, attention_dropout=0.0, activation_dropout=0.0, pad_token_id=1,
                                     bos_token_id=0, eos_token_id=2, decoder_start_token_id=2,
                                     forced_eos_token_id=None)
    hf = transformers.BartForConditionalGeneration(hf_cfg).eval()
    with torch.no_grad():
        hf.final_logits_bias.normal_(0, 0.5)
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
            elif "layer_norm" not in n and "layernorm" not in n:
                p.mul_(3.0)
    cfg = BartConfig.from_hf(hf_cfg.to_dict())
    model = BartModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    src = [0] + torch.randint(3, 300, (30,)).tolist() + [2]
    tgt = [2, 0] + torch.randint(3, 300, (9,)).tolist()
    with torch.no_grad():
        out = hf(input_ids=torch.tensor([src]), decoder_input_ids=torch.tensor([tgt]))
    enc = model.encode(src)
    ref = out.encoder_last_hidden_state[0]
    assert float((enc.float() - ref).norm() / ref.norm()) < 0.02
    full = model.decode(model.start_decoding(enc), tgt)
    assert float((full - out.logits[0]).norm() / out.logits[0].norm()) < 0.03
    assert float((full.argmax(-1) == out.logits[0].argmax(-1)).float().mean()) >= 0.9
    state = model.start_decoding(enc)
    step = torch.cat([model.decode(state, [t]) for t in tgt])
    assert float((step - full).norm() / full.norm()) < 0.02
    dec, want = [2], []
    with torch.no_grad():
        for _ in range(8):
            nxt = int(hf(input_ids=torch.tensor([src]), decoder_input_ids=torch.tensor([dec])).logits[0, -1].argmax())
            if nxt == 2:
                break
            want.append(nxt)
            dec.append(nxt)
    assert model.generate(src, max_new_tokens=8) == want


@pytest.mark.parametrize("learned_pos", [True, False])
def test_trocr_vision_encoder_decoder_matches_transformers(learned_pos):
    """ViT encoder (patch GEMM, class token, pre-LayerNorm) + TrOCR decoder (cross attention from a different
    width, learned or sinusoidal positions, embedding LayerNorm / scale), cached greedy decoding."""
    from antfly_b200.models.trocr import TrOCRConfig, TrOCRModel

    torch.manual_seed(8)
    enc = transformers.ViTConfig(hidden_size=48, num_hidden_layers=2, num_attention_heads=4, intermediate_size=96,
                                 image_size=32, patch_size=8, hidden_dropout_prob=0.0,
                                 attention_probs_dropout_prob=0.0)
    dec = transformers.TrOCRConfig(vocab_size=300, d_model=64, decoder_layers=2, decoder_attention_heads=4,
                                   decoder_ffn_dim=128, max_position_embeddings=40, dropout=0.0,
                                   attention_dropout=0.0, activation_dropout=0.0, cross_attention_hidden_size=48,
                                   use_learned_position_embeddings=learned_pos, layernorm_embedding=learned_pos,
                                   scale_embedding=not learned_pos, decoder_start_token_id=2, eos_token_id=2,
                                   pad_token_id=1)
    hf_cfg = transformers.VisionEncoderDecoderConfig.from_encoder_decoder_configs(enc, dec)
    hf = transformers.VisionEncoderDecoderModel(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.05)
            elif "norm" not in n and "position" not in n and "cls_token" not in n:
                p.mul_(2.0)
    cfg = TrOCRConfig.from_hf(hf_cfg.to_dict())
    assert cfg.encoder.patch_size == 8 and cfg.decoder.use_learned_position_embeddings == learned_pos
    model = TrOCRModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    pixels = torch.randn(3, 32, 32)
    tgt = [2] + torch.randint(3, 300, (9,)).tolist()
    with torch.no_grad():
        out = hf(pixel_values=pixels[None], decoder_input_ids=torch.tensor([tgt]))
    enc_h = model.encode(pixels)
    ref = out.encoder_last_hidden_state[0]
    assert enc_h.shape == (17, 48) and float((enc_h.float() - ref).norm() / ref.norm()) < 0.02
    full = model.decode(model.start_decoding(enc_h), tgt)
    assert float((full - out.logits[0]).norm() / out.logits[0].norm()) < 0.03
    state = model.start_decoding(enc_h)
    step = torch.cat([model.decode(state, [t]) for t in tgt])
    assert float((step - full).norm() / full.norm()) < 0.02
    dec_ids, want = [2], []
    with torch.no_grad():
        for _ in range(6):
            nxt = int(hf(pixel_values=pixels[None], decoder_input_ids=torch.tensor([dec_ids])).logits[0, -1].argmax())
            if nxt == 2:
                break
            want.append(nxt)
            dec_ids.append(nxt)
    assert model.read_ids(pixels, max_new_tokens=6) == want
