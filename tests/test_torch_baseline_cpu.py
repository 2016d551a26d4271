"""The constructed library baseline (baseline/torch_nccl.py) is a faithful model of the same architectures: its
tiny-shape Llama decode agrees with Hugging Face's LlamaForCausalLM given the same weights, and its exact search
agrees with a brute-force top-k.  (It is a comparison arm of the benchmark, not part of the package.)"""
import importlib.util
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    spec = importlib.util.spec_from_file_location("torch_nccl", os.path.join(ROOT, "baseline", "torch_nccl.py"))
    m = importlib.util.module_from_spec(spec)
    sys.modules["torch_nccl"] = m
    spec.loader.exec_module(m)
    return m


def test_tiny_llama_greedy_decode_matches_transformers():
    from transformers import LlamaConfig, LlamaForCausalLM

    T = _load()
    s = T.LlamaShape(layers=2, hidden=64, heads=4, kv_heads=2, ffn=128, vocab=256, theta=10000.0)
    m = T.TorchLlama(s, 0, 1, torch.device("cpu"), torch.float32, seed=3)
    cfg = LlamaConfig(vocab_size=s.vocab, hidden_size=s.hidden, intermediate_size=s.ffn, num_hidden_layers=s.layers,
                      num_attention_heads=s.heads, num_key_value_heads=s.kv_heads, rope_theta=s.theta,
                      rms_norm_eps=s.eps, tie_word_embeddings=False, attention_bias=False)
    hf = LlamaForCausalLM(cfg).eval()
    sd = {"model.embed_tokens.weight": m.embed, "model.norm.weight": m.norm, "lm_head.weight": m.head}
    hd = s.hidden // s.heads
    for i, L in enumerate(m.layers):
        q, k, v = L["qkv"].split([s.heads * hd, s.kv_heads * hd, s.kv_heads * hd], 0)
        g, u = L["gu"].chunk(2, 0)
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                   p + "self_attn.o_proj.weight": L["o"], p + "mlp.gate_proj.weight": g, p + "mlp.up_proj.weight": u,
                   p + "mlp.down_proj.weight": L["d"], p + "input_layernorm.weight": L["n1"],
                   p + "post_attention_layernorm.weight": L["n2"]})
    hf.load_state_dict(sd, strict=False)
    prompts = torch.randint(0, s.vocab, (3, 9), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        mine = T.decode_tokens(m, prompts, 6, prefill_batch=2)
        seq, ref = prompts, []
        for _ in range(6):  # plain greedy loop (generate() would stop a row at the end-of-sequence id)
            nxt = hf(seq).logits[:, -1].argmax(-1)
            ref.append(nxt)
            seq = torch.cat([seq, nxt[:, None]], 1)
        ref = torch.stack(ref, 1)
    assert torch.equal(mine, ref)


def test_exact_search_matches_brute_force():
    T = _load()
    g = torch.Generator().manual_seed(1)
    db = torch.nn.functional.normalize(torch.randn(5000, 32, generator=g), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(7, 32, generator=g), dim=-1)
    d, i = T.knn_search(db, q, 10, 100, 1, chunk=1024)
    ref = (q @ db.t()).topk(10, -1)
    assert torch.equal(i, ref.indices + 100)
    torch.testing.assert_close(d, 1 - ref.values)
