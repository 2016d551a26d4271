"""GPU end-to-end: BERT encoder and Llama decoder/engine on the CUDA kernels against the CPU fp32 oracle path."""
import pytest
import torch

from antfly_b200.models.bert import BertConfig, BertModel, pack_sequences
from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch
from antfly_b200.runtime.engine import LLMEngine
from antfly_b200.runtime.sampling_params import SamplingParams

pytestmark = pytest.mark.gpu


def _bert_pair(cfg):
    gpu = BertModel.random_init(cfg, device="cuda", seed=0)
    cpu = BertModel(cfg, {k: v.cpu() for k, v in gpu.w.items()})
    return gpu, cpu


def test_bert_embed_matches_oracle():
    cfg = BertConfig(hidden_size=256, num_hidden_layers=3, num_attention_heads=4, intermediate_size=1024,
                     vocab_size=2000)
    gpu, cpu = _bert_pair(cfg)
    g = torch.Generator().manual_seed(1)
    seqs = [torch.randint(5, 2000, (n,), generator=g).tolist() for n in (3, 17, 128, 64, 200, 1)]
    b = pack_sequences(seqs)
    e_gpu = gpu.embed(b.to("cuda")).cpu()
    e_cpu = cpu.embed(b)
    assert e_gpu.shape == (6, 256)
    torch.testing.assert_close(e_gpu.norm(dim=-1), torch.ones(6), atol=1e-3, rtol=1e-3)
    cos = (e_gpu * e_cpu).sum(-1)
    assert float(cos.min()) > 0.995, cos


def test_bert_cross_encoder_logits_match_oracle():
    cfg = BertConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512,
                     vocab_size=2000, num_labels=1, use_pooler=True)
    gpu, cpu = _bert_pair(cfg)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(5, 2000, (n,), generator=g).tolist() for n in (40, 77, 12)]
    types = [[0] * 10 + [1] * (len(s) - 10) for s in seqs]
    b = pack_sequences(seqs, types)
    torch.testing.assert_close(gpu.classify(b.to("cuda")).cpu(), cpu.classify(b), atol=3e-2, rtol=3e-2)


def _llama_pair(cfg, seed=0):
    gpu = LlamaModel.random_init(cfg, device="cuda", seed=seed, fast_init=False)
    w = {}
    for k, v in gpu.w.items():
        w[k] = v.to("cpu") if hasattr(v, "to") else v
    return gpu, LlamaModel(cfg, w)


def _prefill_batch(lens, device, max_blocks=8, page=16):
    T = sum(lens)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 512, (T,), generator=g, dtype=torch.int32)
    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
    ql = torch.tensor(lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int()
    tables = torch.zeros((len(lens), max_blocks), dtype=torch.int32)
    slots = []
    nb = 0
    for i, n in enumerate(lens):
        k = (n + page - 1) // page
        tables[i, :k] = torch.arange(nb, nb + k, dtype=torch.int32)
        slots.extend(range(nb * page, nb * page + n))
        nb += k
    rows = (qs + ql - 1).int()
    f = lambda t: t.to(device)
    return StepBatch(f(ids), f(pos), f(torch.tensor(slots, dtype=torch.int32)), f(qs), f(ql), f(ql.clone()),
                     f(tables), f(rows), max(lens), 1), nb


@pytest.mark.parametrize("variant", ["llama", "qwen2", "qwen3"])
def test_llama_forward_matches_oracle(variant):
    kw = {"qwen2": dict(qkv_bias=True), "qwen3": dict(qk_norm=True), "llama": {}}[variant]
    cfg = LlamaConfig.tiny(num_hidden_layers=2, **kw)
    gpu, cpu = _llama_pair(cfg)
    outs = []
    for m, dev in ((gpu, "cuda"), (cpu, "cpu")):
        b, nb = _prefill_batch([33, 5, 70], dev)
        kc = torch.zeros((2, nb + 1, 16, cfg.num_key_value_heads, cfg.head_dim), dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        outs.append((m.forward(b, kc, vc).float().cpu(), kc.float().cpu(), vc.float().cpu()))
    (lg, kg, vg), (lc, kc_, vc_) = outs
    torch.testing.assert_close(kg, kc_, atol=6e-2, rtol=5e-2)
    torch.testing.assert_close(vg, vc_, atol=6e-2, rtol=5e-2)
    torch.testing.assert_close(lg, lc, atol=8e-2, rtol=5e-2)
    assert float((lg.argmax(-1) == lc.argmax(-1)).float().mean()) >= 2 / 3


def _engine(model, **kw):
    return LLMEngine(model, num_blocks=128, page=16, max_batch=8, max_step_tokens=256, **kw)


def test_engine_graph_replay_matches_eager_and_chunked_prefill():
    cfg = LlamaConfig.tiny(num_hidden_layers=2)
    model = LlamaModel.random_init(cfg, device="cuda", seed=0, fast_init=False)
    prompts = [[5, 6, 7, 8, 9] * 9, [11, 12, 13], [3] * 40, [9, 8, 7, 6] * 20]
    sp = SamplingParams(max_tokens=24)
    a = _engine(model, use_cuda_graph=True).generate(prompts, sp)
    b = _engine(model, use_cuda_graph=False).generate(prompts, sp)
    c = _engine(model, use_cuda_graph=True, prefill_chunk=32).generate(prompts, sp)
    assert [r.token_ids for r in a] == [r.token_ids for r in b]
    # Chunk boundaries change the split-K factors and with them the fp32 summation order, so a near-tie may flip
    # late in a sequence; the prefill result (first token) must agree everywhere and most sequences fully.
    assert [x.token_ids[0] for x in a] == [y.token_ids[0] for y in c]
    assert sum(x.token_ids == y.token_ids for x, y in zip(a, c)) >= 2
    assert all(len(r.token_ids) == 24 for r in a)


def test_engine_speculative_decode_matches_greedy():
    cfg = LlamaConfig.tiny(num_hidden_layers=3)
    model = LlamaModel.random_init(cfg, device="cuda", seed=1, fast_init=False)
    prompts = [[7, 8, 9, 10] * 5, [100, 101, 102], [1, 2, 3, 4, 5, 6, 7, 8]]
    sp = SamplingParams(max_tokens=20)
    plain = _engine(model, use_cuda_graph=False).generate(prompts, sp)
    eng = _engine(model, use_cuda_graph=False, draft_layers=2, spec_k=4)
    spec = eng.generate(prompts, sp)
    agree = sum(x.token_ids == y.token_ids for x, y in zip(plain, spec))
    assert agree >= 2, (plain, spec)
    assert eng.spec.rounds > 0 and eng.spec.drafted == eng.spec.matched + eng.spec.rejected
    assert eng.cache.alloc.free_blocks == 128


def test_engine_sampling_path_on_gpu():
    cfg = LlamaConfig.tiny(num_hidden_layers=1)
    model = LlamaModel.random_init(cfg, device="cuda", seed=2, fast_init=False)
    sp = SamplingParams(max_tokens=8, temperature=0.8, top_k=30, top_p=0.95, min_p=0.01, repetition_penalty=1.3,
                        presence_penalty=0.2, seed=7)
    out = _engine(model).generate([[1, 2, 3], [4, 5, 6, 7]], sp)
    assert all(len(r.token_ids) == 8 and all(0 <= t < 512 for t in r.token_ids) for r in out)
