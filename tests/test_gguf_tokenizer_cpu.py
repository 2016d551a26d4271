"""Tokenizers carried in GGUF metadata: byte-level BPE (``gpt2``) and SentencePiece-style BPE (``llama``) rebuilt from
the token / merge / score lists, against the libraries that produced those lists."""
import pytest

CORPUS = ["the quick brown fox jumps over the lazy dog", "hello world, hello tokenizer!", "numbers 12345 and 67890",
          "naïve café déjà vu", "tabs\tand  double  spaces", "ünïcödé ≠ ascii — dashes", "def f(x): return x + 1"] * 8
PROBES = ["hello world", " the fox", "naïve dog 123", "unseen: žluťoučký kůň 🙂", "", "a", "def  f(x):\n    return x"]


def test_gpt2_model_from_metadata_matches_the_tokenizers_library(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    from antfly_b200.tokenizer import GGUFTokenizer

    tk = Tokenizer(models.BPE())
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    tk.train_from_iterator(CORPUS, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|bos|>", "<|eos|>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    import json

    model = json.loads(tk.to_str())["model"]
    vocab = sorted(model["vocab"], key=model["vocab"].get)
    merges = [m if isinstance(m, str) else " ".join(m) for m in model["merges"]]
    md = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": vocab, "tokenizer.ggml.merges": merges,
          "tokenizer.ggml.token_type": [3 if t in ("<|bos|>", "<|eos|>") else 1 for t in vocab],
          "tokenizer.ggml.bos_token_id": vocab.index("<|bos|>"), "tokenizer.ggml.eos_token_id": vocab.index("<|eos|>"),
          "tokenizer.chat_template": "{{ messages }}"}
    g = GGUFTokenizer(md)
    assert g.special.bos_id == vocab.index("<|bos|>") and g.chat_template == "{{ messages }}"
    for text in PROBES:
        want = tk.encode(text, add_special_tokens=False).ids
        assert g.encode(text) == want, text
        assert g.decode(want) == text
        assert b"".join(g.token_bytes(i) for i in want).decode("utf-8") == text
    assert g.encode_prompt("hi")[0] == g.special.bos_id and g.decode([g.special.bos_id] + g.encode("hi")) == "hi"
    assert g.encode("<|eos|>") == [vocab.index("<|eos|>")]                 # control tokens match as a whole


def test_llama_model_from_metadata_matches_sentencepiece(tmp_path):
    spm = pytest.importorskip("sentencepiece")
    from antfly_b200.tokenizer import GGUFTokenizer

    corpus = tmp_path / "c.txt"
    corpus.write_text("\n".join(CORPUS))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "m"), vocab_size=420,
                                   model_type="bpe", byte_fallback=True, character_coverage=1.0, bos_id=1, eos_id=2,
                                   unk_id=0, minloglevel=2, split_digits=True, normalization_rule_name="identity",
                                   remove_extra_whitespaces=False, add_dummy_prefix=True)
    sp = spm.SentencePieceProcessor(model_file=str(tmp_path / "m.model"))
    n = sp.get_piece_size()
    types = [2 if sp.is_unknown(i) else 3 if sp.is_control(i) else 6 if sp.is_byte(i) else 1 for i in range(n)]
    md = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": [sp.id_to_piece(i) for i in range(n)],
          "tokenizer.ggml.scores": [sp.get_score(i) for i in range(n)], "tokenizer.ggml.token_type": types,
          "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0}
    g = GGUFTokenizer(md)
    for text in PROBES:
        want = list(sp.encode(text))
        assert g.encode(text) == want, (text, g.encode(text), want)
        assert g.decode(want) == sp.decode(want)
    assert g.special.bos_id == 1 and g.special.eos_id == 2 and g.token_bytes(1) == b""


def test_model_directory_with_only_a_gguf_file_uses_its_tokenizer(tmp_path):
    import torch

    from antfly_b200.formats import gguf as GG
    from antfly_b200.tokenizer import GGUFTokenizer, load_tokenizer

    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "a", "b", "▁a", "ab", "▁ab"]
    md = {"general.architecture": "llama", "llama.block_count": 1, "tokenizer.ggml.model": "llama",
          "tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": [0.0] * 259 + [-1.0, -2.0, -3.0, -0.5, -0.7, -0.1],
          "tokenizer.ggml.token_type": [2, 3, 3] + [6] * 256 + [1] * 6,
          "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0}
    GG.write_gguf(str(tmp_path / "model.gguf"), md, {"token_embd.weight": (0, torch.zeros(4, 4))})
    tok = load_tokenizer(str(tmp_path), 0)
    assert isinstance(tok, GGUFTokenizer) and tok.vocab_size == len(toks)
    # "ab ab": pieces by score: (_a, b) vs (a, b) -> "ab" scores -0.7 < "_a" -0.5, then "_a"+"b" -> "_ab" (-0.1)
    assert tok.encode("ab ab") == [toks.index("▁ab")] * 2
    assert tok.encode("é") == [toks.index("▁")] + [3 + b for b in "é".encode()]     # byte fallback
    assert tok.decode(tok.encode("ab é")) == "ab é"


def test_gguf_only_generator_gets_tokenizer_and_chat_template_from_the_file(tmp_path):
    import torch
    import transformers

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import gguf as GG
    from antfly_b200.runtime.sampling_params import SamplingParams

    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "a", "b", "▁a", "ab", "▁ab"]
    template = "{% for m in messages %}<s>{{ m['role'] }}: {{ m['content'] }}</s>{% endfor %}assistant:"
    md = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.scores": [0.0] * 259 + [-1.0, -2.0, -3.0, -0.5, -0.7, -0.1],
          "tokenizer.ggml.token_type": [2, 3, 3] + [6] * 256 + [1] * 6, "tokenizer.ggml.bos_token_id": 1,
          "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0, "tokenizer.chat_template": template}
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=len(toks), hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128)
    hf = transformers.LlamaForCausalLM(cfg)
    d = tmp_path / "generators" / "chatty"
    d.mkdir(parents=True)
    GG.export_llama_gguf(str(d / "model.gguf"), hf.state_dict(), cfg.to_dict(), tokens=toks, extra_metadata=md)
    lm = ModelManager(models_dir=str(tmp_path), device="cpu").get("chatty", "generator")
    assert lm.pipeline.template.source == template and lm.tokenizer.vocab_size == len(toks)
    out = lm.pipeline.generate([{"role": "user", "content": "ab"}], SamplingParams(max_tokens=3, ignore_eos=True))
    assert len(out.token_ids) == 3 and out.prompt_tokens > 4
