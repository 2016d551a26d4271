"""Generation engine on the CPU oracle path: scheduler + paged KV + model + sampler glue, no GPU."""
import torch

from antfly_b200.models.llama import LlamaConfig, LlamaModel
from antfly_b200.runtime.engine import LLMEngine
from antfly_b200.runtime.sampling_params import SamplingParams


def _engine(**kw):
    cfg = LlamaConfig.tiny(num_hidden_layers=2)
    model = LlamaModel.random_init(cfg, device="cpu", seed=0)
    return LLMEngine(model, num_blocks=64, page=16, max_batch=4, max_step_tokens=64, use_cuda_graph=False, **kw)


def test_greedy_generation_is_deterministic_and_chunking_invariant():
    prompts = [[5, 6, 7, 8, 9] * 9, [11, 12, 13], [3] * 40]
    sp = SamplingParams(max_tokens=6)
    a = _engine(prefill_chunk=2048).generate(prompts, sp)
    b = _engine(prefill_chunk=16).generate(prompts, sp)
    assert [r.token_ids for r in a] == [r.token_ids for r in b]
    assert all(len(r.token_ids) == 6 and r.finish_reason == "length" for r in a)


def test_stop_token_and_kv_blocks_are_released():
    eng = _engine()
    first = eng.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=4))[0].token_ids
    eng2 = _engine()
    res = eng2.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=8, stop_token_ids=[first[1]]))[0]
    assert res.token_ids == first[:2] and res.finish_reason == "stop"
    assert eng2.cache.alloc.free_blocks == 64


def test_speculative_decoding_reproduces_greedy_output():
    prompts = [[7, 8, 9, 10] * 5, [100, 101, 102]]
    sp = SamplingParams(max_tokens=12)
    plain = _engine().generate(prompts, sp)
    eng = _engine(draft_layers=1, spec_k=3)
    spec = eng.generate(prompts, sp)
    assert [r.token_ids for r in spec] == [r.token_ids for r in plain]
    st = eng.spec
    assert st.rounds > 0 and st.drafted == st.matched + st.rejected
    assert st.corrections + st.bonus == st.rounds * 2 or st.corrections + st.bonus >= st.rounds
    assert "speculative: rounds=" in st.line()


def test_sampling_with_penalties_runs_and_respects_limits():
    eng = _engine()
    sp = SamplingParams(max_tokens=5, temperature=0.9, top_k=20, top_p=0.9, min_p=0.01, repetition_penalty=1.2,
                        frequency_penalty=0.1, presence_penalty=0.1, seed=3)
    out = eng.generate([[1, 2, 3], [4, 5, 6, 7]], sp)
    assert all(len(r.token_ids) == 5 for r in out)
    assert all(0 <= t < 512 for r in out for t in r.token_ids)


def test_engine_generates_with_layernorm_decoder_family():
    """The paged-KV engine drives a GPT-2-style model (learned positions, LayerNorm, GELU MLP) exactly like a
    Llama-style one: greedy continuation equals a step-by-step full-recompute of the same model."""
    import torch

    from antfly_b200.models.gpt import GptConfig, GptModel
    from antfly_b200.models.llama import StepBatch
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    cfg = GptConfig("gpt2", vocab_size=200, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                    intermediate_size=128, max_position_embeddings=64)
    model = GptModel.random_init(cfg, device="cpu", seed=3, dtype=torch.float32)
    eng = LLMEngine(model, num_blocks=16, page=16, max_batch=2, max_step_tokens=64, prefill_chunk=8,
                    max_seq_len=48, use_cuda_graph=False)
    prompt = [5, 17, 99, 3, 42, 7, 150, 21, 8, 64, 11]
    rid = eng.add_request(prompt, SamplingParams(max_tokens=6, ignore_eos=True))
    while eng.has_work():
        eng.step()
    got = list(eng.reqs[rid].out)

    seq = list(prompt)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    for _ in range(6):
        n = len(seq)
        kc = torch.zeros((2, 4, 16, 4, 16), dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        pos = torch.arange(n, dtype=torch.int32)
        b = StepBatch(i32(seq), pos, pos.clone(), i32([0]), i32([n]), i32([n]), torch.arange(4, dtype=torch.int32)[None],
                      i32([n - 1]), n, 1)
        seq.append(int(model.forward(b, kc, vc).float().argmax(-1)))
    assert got == seq[len(prompt):], (got, seq[len(prompt):])


def test_prefix_cache_reuses_blocks_and_keeps_outputs():
    """Requests whose prompts share a block-aligned prefix skip prefilling it; generated tokens are the same as
    without the cache; entries are evicted when the pool runs short."""
    import torch

    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    cfg = LlamaConfig.tiny(vocab_size=256)
    model = LlamaModel.random_init(cfg, device="cpu", seed=5, fast_init=False)
    g = torch.Generator().manual_seed(0)
    system = torch.randint(0, 256, (70,), generator=g).tolist()           # 4 whole blocks + 6 tokens
    prompts = [system + torch.randint(0, 256, (n,), generator=g).tolist() for n in (5, 9, 3)]

    def run(prefix_cache, num_blocks=64):
        eng = LLMEngine(model, num_blocks=num_blocks, page=16, max_batch=4, max_step_tokens=128, prefill_chunk=32,
                        max_seq_len=128, use_cuda_graph=False, prefix_cache=prefix_cache)
        outs = []
        for p in prompts:   # one after the other so the later ones can hit
            rid = eng.add_request(p, SamplingParams(max_tokens=6, ignore_eos=True))
            while eng.has_work():
                eng.step()
            outs.append(list(eng.reqs[rid].out))
        return eng, outs

    base_eng, base = run(False)
    eng, got = run(True)
    assert got == base
    st = eng.prefix.stats()
    assert st["hits"] == 2 and st["misses"] == 1 and st["tokens_reused"] == 2 * 64
    # the shared prompt blocks are held once by the cache entries, not once per request
    assert eng.sched.stats()["step_query_tokens_total"] < base_eng.sched.stats()["step_query_tokens_total"] - 100
    free_with_entries = eng.cache.alloc.free_blocks
    eng.prefix.clear()
    assert eng.cache.alloc.free_blocks > free_with_entries and eng.cache.alloc.free_blocks == 64

    # a pool too small to keep every cached prefix: entries are dropped on demand and generation still completes
    prompts = [torch.randint(0, 256, (70 + i,), generator=g).tolist() for i in range(3)]   # unrelated prompts
    _, want = run(False, num_blocks=64)
    small, got_small = run(True, num_blocks=10)
    assert got_small == want and small.prefix.stats()["evictions"] >= 1 and small.prefix.stats()["hits"] == 0


def _draft_model(seed=5, layers=1):
    cfg = LlamaConfig.tiny(num_hidden_layers=layers)
    return LlamaModel.random_init(cfg, device="cpu", seed=seed)


def test_speculative_decoding_with_a_separate_draft_model_reproduces_greedy_output():
    """A second, independently initialised model drafts; the target verifies.  Whatever the draft proposes, the
    output must be the target's own greedy continuation, both KV caches must stay consistent across rounds with
    rejections (random drafts rarely match) and every block must be released at the end."""
    prompts = [[7, 8, 9, 10] * 5, [100, 101, 102], [42] * 33]
    sp = SamplingParams(max_tokens=14)
    plain = _engine().generate(prompts, sp)
    eng = _engine(draft_model=_draft_model(), spec_k=4)
    spec = eng.generate(prompts, sp)
    assert [r.token_ids for r in spec] == [r.token_ids for r in plain]
    st = eng.spec
    assert st.rounds > 0 and st.drafted == st.matched + st.rejected and st.accepted == st.matched + st.corrections + st.bonus
    assert eng.cache.alloc.free_blocks == 64 and eng.draft_cache.alloc.free_blocks == 64


def test_separate_draft_that_equals_the_target_is_always_accepted_and_k_is_per_request():
    """The target's own weights as the 'separate' draft: every draft matches, every round ends with a bonus token
    (which exercises the catch-up of the draft cache's missing last entry); speculative_k of the request sets the
    round's draft length."""
    prompts = [[7, 8, 9, 10] * 3, [1, 2, 3]]
    sp = SamplingParams(max_tokens=11, speculative_k=2)
    plain = _engine().generate(prompts, SamplingParams(max_tokens=11))
    twin = LlamaModel.random_init(LlamaConfig.tiny(num_hidden_layers=2), device="cpu", seed=0)
    eng = _engine(draft_model=twin, spec_k=4)
    spec = eng.generate(prompts, sp)
    assert [r.token_ids for r in spec] == [r.token_ids for r in plain]
    st = eng.spec
    assert st.rejected == 0 and st.matched == st.drafted and st.corrections == 0
    assert st.bonus > 0 and st.drafted % 2 == 0      # rounds of exactly two draft tokens per sequence


def test_draft_model_with_another_vocabulary_is_refused():
    import pytest

    other = LlamaModel.random_init(LlamaConfig.tiny(num_hidden_layers=1, vocab_size=300), device="cpu", seed=1)
    with pytest.raises(ValueError):
        _engine(draft_model=other)


# ---------------------------------------------------------------------------------------------------------------
# Quantised KV caches through the whole engine (prefill chunks, decode, speculative verification, prefix sharing).
# The reference for "the cache works" is an engine with a full-precision cache into which every key / value row is
# written after a round trip through the same codec: both engines then attend over identical numbers, so their
# greedy tokens must agree.
# ---------------------------------------------------------------------------------------------------------------
import pytest  # noqa: E402


class _RoundTripCache:
    """f32 cache whose writes pass through a codec's encode + decode (the dequantised-cache reference)."""

    def __init__(self, codec, cache):
        from antfly_b200.ops import kv_quant as KQ

        self.codec, self.KQ = codec, KQ
        self.k, self.v = _RoundTripTensor(self, cache.k, False), _RoundTripTensor(self, cache.v, True)


class _RoundTripTensor:
    def __init__(self, owner, t, value):
        self.owner, self.t, self.value = owner, t, value
        self.shape = t.shape

    def __getitem__(self, l):
        return _RoundTripLayer(self.owner, self.t[l], self.value)


class _RoundTripLayer(torch.Tensor):
    """A view of the f32 cache layer whose index-assignment (what the CPU KV-write path does) quantises rows."""

    @staticmethod
    def __new__(cls, owner, t, value):
        obj = torch.Tensor._make_subclass(cls, t)
        obj.owner, obj.value = owner, value
        return obj

    def view(self, *shape):
        v = torch.Tensor.view(self.as_subclass(torch.Tensor), *shape)
        out = torch.Tensor._make_subclass(_RoundTripLayer, v)
        out.owner, out.value = self.owner, self.value
        return out

    def __setitem__(self, idx, rows):
        KQ, codec = self.owner.KQ, self.owner.codec
        T, H, D = rows.shape
        enc = KQ.encode_rows_torch(codec, rows.float(), value=self.value)
        dec = KQ.decode_rows(codec, enc, H, D, value=self.value)
        torch.Tensor.__setitem__(self.as_subclass(torch.Tensor), idx, dec)


@pytest.mark.parametrize("codec", ["fp8", "int8", "int4"])
def test_quantised_kv_cache_generates_the_tokens_of_the_dequantised_cache_reference(codec):
    prompts = [[7, 8, 9, 10] * 9, [100, 101, 102], [5] * 21]
    sp = SamplingParams(max_tokens=10)
    ref_eng = _engine(kv_dtype="f32", prefill_chunk=16)
    rt = _RoundTripCache(codec, ref_eng.cache)
    ref_eng.cache.k, ref_eng.cache.v = rt.k, rt.v
    want = [r.token_ids for r in ref_eng.generate(prompts, sp)]
    eng = _engine(kv_dtype=codec, prefill_chunk=16)
    got = [r.token_ids for r in eng.generate(prompts, sp)]
    assert got == want
    assert eng.cache.codec == codec and eng.cache.k.data.dtype == torch.uint8
    assert eng.cache.alloc.free_blocks == 64
    # smaller than a bf16 cache by the codec's ratio
    bf16 = _engine().cache.nbytes()
    assert eng.cache.nbytes() < {"fp8": 0.52, "int8": 0.55, "int4": 0.3}[codec] * bf16


@pytest.mark.parametrize("codec", ["polar4", "turbo3"])
def test_compressed_key_codecs_run_end_to_end(codec):
    """polar4 / turbo3 clamp keys to [-1, 1]; with random weights the output differs from bf16, but generation must
    run through prefill, decode and block release."""
    eng = _engine(kv_dtype=codec)
    res = eng.generate([[1, 2, 3, 4, 5, 6, 7] * 3, [9, 9]], SamplingParams(max_tokens=6))
    assert all(len(r.token_ids) == 6 for r in res)
    assert eng.cache.alloc.free_blocks == 64


def test_quantised_kv_with_speculative_decoding_and_prefix_cache():
    prompts = [[3, 4, 5, 6] * 10 + [11], [3, 4, 5, 6] * 10 + [12]]
    sp = SamplingParams(max_tokens=8)
    plain = [r.token_ids for r in _engine(kv_dtype="int8").generate(prompts, sp)]
    eng = _engine(kv_dtype="int8", draft_layers=1, spec_k=3, prefix_cache=True)
    assert [r.token_ids for r in eng.generate(prompts, sp)] == plain
    with pytest.raises(ValueError):
        _engine(kv_dtype="int8").compact_request(1, 0.5)
