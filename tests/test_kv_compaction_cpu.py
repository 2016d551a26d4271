"""KV compaction by attention matching: the fitted small cache reproduces attention better than plain eviction,
and the engine keeps generating with logical positions over the compacted cache."""
import torch

from antfly_b200.runtime.kv_compaction import attention_output, compact_head, compact_layer


def _structured_kv(n, d, seed):
    g = torch.Generator().manual_seed(seed)
    centers = torch.randn(6, d, generator=g)
    assign = torch.randint(0, 6, (n,), generator=g)
    K = centers[assign] * 1.5 + 0.4 * torch.randn(n, d, generator=g)
    V = torch.randn(6, d, generator=g)[assign] + 0.3 * torch.randn(n, d, generator=g)
    return K, V


def test_fitted_values_beat_plain_eviction():
    d, n = 32, 400
    K, V = _structured_kv(n, d, 0)
    g = torch.Generator().manual_seed(1)
    Q = K[torch.randint(0, n, (50,), generator=g)] + 0.2 * torch.randn(50, d, generator=g)  # held-out probes
    full = attention_output(Q, K, V)
    for ratio in (0.1, 0.25):
        idx, K_hat, V_hat = compact_head(K, V, ratio)
        assert idx.numel() == int(-(-n * ratio // 1)) and torch.equal(idx, idx.sort().values)
        fitted = attention_output(Q, K_hat, V_hat)
        evicted = attention_output(Q, K_hat, V[idx])                       # same keys, original values
        recent = attention_output(Q, K[-idx.numel():], V[-idx.numel():])   # sliding-window baseline
        e_fit = float((fitted - full).norm() / full.norm())
        e_evict = float((evicted - full).norm() / full.norm())
        e_recent = float((recent - full).norm() / full.norm())
        assert e_fit < e_evict and e_fit < e_recent and e_fit < 0.35, (ratio, e_fit, e_evict, e_recent)


def test_ratio_one_and_recent_window_and_layer_shape():
    K, V = _structured_kv(64, 16, 2)
    idx, K_hat, V_hat = compact_head(K, V, 1.0)
    assert torch.equal(K_hat, K) and torch.equal(V_hat, V) and idx.numel() == 64
    idx, _, _ = compact_head(K, V, 0.25, keep_recent=8)
    assert set(range(56, 64)) <= set(idx.tolist())
    Kl, Vl = torch.randn(100, 3, 16).bfloat16(), torch.randn(100, 3, 16).bfloat16()
    Kc, Vc = compact_layer(Kl, Vl, 0.2)
    assert Kc.shape == (20, 3, 16) and Vc.shape == (20, 3, 16) and Kc.dtype == torch.float32


def test_engine_compacts_after_prefill_and_keeps_generating():
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.runtime.engine import LLMEngine
    from antfly_b200.runtime.sampling_params import SamplingParams

    cfg = LlamaConfig.tiny(vocab_size=256)
    model = LlamaModel.random_init(cfg, device="cpu", seed=2, fast_init=False)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 256, (96,), generator=g).tolist()

    def run(ratio):
        eng = LLMEngine(model, num_blocks=32, page=16, max_batch=2, max_step_tokens=128, prefill_chunk=64,
                        max_seq_len=160, use_cuda_graph=False)
        rid = eng.add_request(prompt, SamplingParams(max_tokens=10, ignore_eos=True, cache_compaction_ratio=ratio))
        while eng.has_work():
            eng.step()
        return eng, eng.reqs[rid]

    _, base = run(None)
    eng, r = run(0.5)
    assert len(r.out) == 10 and r.kv_removed == 48
    assert r.out[0] == base.out[0]               # the first token is sampled before the cache is compacted
    # blocks were given back: 96 prompt tokens -> 48 kept (3 blocks) instead of 6
    eng2, r2 = run(1.0)
    assert r2.kv_removed == 0 and r2.out == base.out
