"""GPU runs of the audio, vision and span models against their own CPU (fp32-accumulate) paths, plus attention with
head widths the kernel does not have natively (run zero-padded)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

transformers = pytest.importorskip("transformers")


def _close(got, want, cos_min=0.995):
    got, want = got.float().cpu(), want.float().cpu()
    c = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    assert float(c) > cos_min, float(c)


@pytest.mark.parametrize("D", [32, 80])
def test_varlen_attention_padded_head_width(D):
    from antfly_b200.ops import attention as A
    from antfly_b200.ops import reference as R

    g = torch.Generator().manual_seed(D)
    lens = torch.tensor([37, 5, 90], dtype=torch.int32)
    starts = (torch.cumsum(lens, 0) - lens).to(torch.int32)
    T = int(lens.sum())
    q, k, v = (torch.randn(T, 4, D, generator=g).to(torch.bfloat16) for _ in range(3))
    cu = torch.cat([starts.long(), torch.tensor([T])])
    want = R.varlen_attention(q, k, v, cu)
    got = A.varlen_attention(q.cuda(), k.cuda(), v.cuda(), starts.cuda(), lens.cuda(), 90)
    assert got.shape == (T, 4, D)
    torch.testing.assert_close(got.float().cpu(), want, atol=2e-2, rtol=2e-2)


def test_qwen2vl_vision_tower_on_gpu():
    from antfly_b200.models import qwen2vl as QV
    import tests.test_qwen2vl_cpu as T

    hf_cfg, hf = T._hf()
    vc = QV.Qwen2VLVisionConfig.from_hf(hf_cfg.vision_config.to_dict())
    sd = {k: v.to(torch.bfloat16).float() for k, v in hf.state_dict().items()}
    cpu = QV.Qwen2VLVisionModel.from_state_dict(vc, sd, device="cpu", dtype=torch.float32)
    gpu = QV.Qwen2VLVisionModel.from_state_dict(vc, sd, device="cuda")
    grids = [(1, 4, 6), (1, 2, 2)]
    patches = torch.randn(28, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).float()
    _close(gpu.forward(patches, grids), cpu.forward(patches, grids))


@pytest.mark.parametrize("fusion", [False, True])
def test_clap_audio_tower_on_gpu(fusion):
    from antfly_b200.models.clap import ClapConfig, ClapModel
    import tests.test_clap_cpu as T

    hf_cfg, hf = T._tiny(fusion)
    cfg = ClapConfig.from_hf(hf_cfg.to_dict())
    sd = {k: (v.to(torch.bfloat16).float() if v.is_floating_point() else v) for k, v in hf.state_dict().items()}
    cpu = ClapModel.from_state_dict(cfg, sd, device="cpu", dtype=torch.float32)
    gpu = ClapModel.from_state_dict(cfg, sd, device="cuda")
    feats = torch.randn(3, 4 if fusion else 1, 250, 16, generator=torch.Generator().manual_seed(3)) * 10 - 20
    longer = [True, False, True]
    _close(gpu.embed_audio(feats, longer), cpu.embed_audio(feats, longer), 0.99)
    seqs = [[0, 5, 9, 2], [0, 7, 8, 11, 30, 2]]
    _close(gpu.embed_text(seqs), cpu.embed_text(seqs), 0.99)


def test_gliner_span_logits_on_gpu():
    from antfly_b200.models.deberta import DebertaConfig
    from antfly_b200.models.gliner import GlinerInput, GlinerModel
    import tests.test_gliner_cpu as T

    enc, head, cpu = T._build()
    sd = {"encoder." + k: v for k, v in enc.state_dict().items()}
    sd.update(head.state_dict())
    gpu = GlinerModel.from_state_dict(DebertaConfig.from_hf(enc.config.to_dict()), sd, device="cuda")
    inp = GlinerInput([5, 390, 20, 21, 390, 30, 391, 40, 41, 42, 43, 44], [0] * 7 + [1, 2, 2, 3, 4], 4)
    a = gpu.span_logits([inp], [390], 3)[0]
    b = cpu.span_logits([inp], [390], 3)[0]
    assert a.shape == b.shape == (4, 3, 2)
    _close(a, b, 0.98)


def test_bitnet_forward_on_gpu():
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    import tests.test_bitnet_cpu as T

    hf_cfg, hf = T._hf()
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    sd.pop("lm_head.weight", None)
    cfg = LlamaConfig.from_hf(hf_cfg.to_dict())
    ids = torch.randint(0, hf_cfg.vocab_size, (25,), generator=torch.Generator().manual_seed(5))
    want = T._run(LlamaModel.from_state_dict(cfg, dict(sd), device="cpu"), cfg, ids, 24)
    gpu = LlamaModel.from_state_dict(cfg, dict(sd), device="cuda")
    got = T._run(gpu, cfg, ids.cuda(), 24, device="cuda")
    cos = torch.nn.functional.cosine_similarity(got.float().cpu(), want, dim=-1)
    assert float(cos.min()) > 0.99, cos


# -- 256-wide heads (Gemma-class decoders) through the same attention kernels ----------------------------------
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_attention_head_width_256(causal):
    from antfly_b200.ops import attention as A
    from antfly_b200.ops import reference as R
    from tests.test_attention_gpu import _rand

    D, Hq, Hkv = 256, 4, 2
    lens = torch.tensor([1, 17, 64, 65, 200, 33], dtype=torch.int32)
    starts = (torch.cumsum(lens, 0) - lens).int()
    T = int(lens.sum())
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=1, scale=0.5)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    out = A.varlen_attention(q, k, v, starts.cuda(), lens.cuda(), int(lens.max()), causal=causal)
    cu = torch.cat([starts, torch.tensor([T], dtype=torch.int32)])
    torch.testing.assert_close(out.float(), R.varlen_attention(q, k, v, cu, causal=causal), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("Hq,Hkv", [(8, 1), (8, 2), (16, 1)])
@pytest.mark.parametrize("splits", [1, 4])
def test_paged_decode_head_width_256(Hq, Hkv, splits):
    from antfly_b200.ops import attention as A
    from antfly_b200.ops import reference as R
    from tests.test_attention_gpu import _build_paged, _rand

    D = 256
    kv_lens = [1, 15, 16, 17, 300, 1030, 64]
    B = len(kv_lens)
    kc, vc, bt = _build_paged(B, kv_lens, Hkv, D, 16, seed=5)
    q = _rand(B, Hq, D, seed=9, scale=0.5)
    q_starts = torch.arange(B, dtype=torch.int32, device="cuda")
    q_lens = torch.ones(B, dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    out = A.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl, 1, num_splits=splits)
    torch.testing.assert_close(out.float(), R.paged_attention(q, kc, vc, bt, q_starts, q_lens, kvl), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("window", [0, 40])
def test_paged_attention_without_causal_mask(window):
    """Runs of image tokens attend in both directions: paged keys, no causal mask, optionally a two-sided window."""
    from antfly_b200.ops import attention as A
    from antfly_b200.ops import reference as R
    from tests.test_attention_gpu import _build_paged, _rand

    D, Hq, Hkv = 64, 8, 2
    kv_lens, q_lens = [70, 300, 33], [64, 256, 33]
    B = len(kv_lens)
    kc, vc, bt = _build_paged(B, kv_lens, Hkv, D, 16, seed=3)
    T = sum(q_lens)
    q = _rand(T, Hq, D, seed=4)
    ql = torch.tensor(q_lens, dtype=torch.int32, device="cuda")
    qs = (torch.cumsum(ql, 0) - ql).int()
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    out = A.paged_attention(q, kc, vc, bt, qs, ql, kvl, max(q_lens), window=window, causal=False, decode=False)
    ref = R.paged_attention(q, kc, vc, bt, qs, ql, kvl, sliding_window=window, causal=False)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


def _prefill_logits(model, cfg, ids, device, **extra):
    from antfly_b200.models.llama import StepBatch

    S, page, nblk = len(ids), 16, 4
    kc = torch.zeros((cfg.num_hidden_layers, nblk, page, model.Hkv, cfg.head_dim), dtype=torch.bfloat16, device=device)
    vc = torch.zeros_like(kc)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    idx = torch.arange(S, dtype=torch.int32, device=device)
    mv = lambda v: tuple(t.to(device) if isinstance(t, torch.Tensor) else t for t in v) if isinstance(v, tuple) else (
        v.to(device) if isinstance(v, torch.Tensor) else v)
    b = StepBatch(i32(ids), idx, idx.clone(), i32([0]), i32([S]), i32([S]),
                  torch.arange(nblk, dtype=torch.int32, device=device)[None], idx.clone(), S, 1,
                  **{k: mv(v) for k, v in extra.items()})
    return model.forward(b, kc, vc).float().cpu()


def test_qwen2vl_decoder_with_image_tokens_on_gpu():
    from antfly_b200.models import qwen2vl as QV
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    import tests.test_qwen2vl_cpu as T

    hf_cfg, hf = T._hf(1)
    sd = QV.text_state_dict(hf.state_dict())
    cfg = LlamaConfig.from_hf(hf_cfg.text_config.to_dict())
    grids = [(1, 4, 6)]
    ids = [5, 6, 302] + [300] * 6 + [303, 7, 8, 9]
    pos3, _ = QV.rope_index(ids, grids, 300)
    soft = torch.randn(6, cfg.hidden_size, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    rows = torch.tensor([3, 4, 5, 6, 7, 8])
    extra = dict(embed_rows=rows, embed_vals=soft, pos3=pos3)
    want = _prefill_logits(LlamaModel.from_state_dict(cfg, dict(sd), device="cpu"), cfg, ids, "cpu", **extra)
    got = _prefill_logits(LlamaModel.from_state_dict(cfg, dict(sd), device="cuda"), cfg, ids, "cuda", **extra)
    assert float(torch.nn.functional.cosine_similarity(got, want, dim=-1).min()) > 0.99


def test_gemma3_decoder_with_two_way_image_attention_on_gpu():
    from antfly_b200.models.llama import LlamaConfig, LlamaModel
    from antfly_b200.models.qwen2vl import text_state_dict
    import tests.test_gemma3v_cpu as T

    hf_cfg, hf = T._hf(1)
    sd = text_state_dict(hf.state_dict())
    cfg = LlamaConfig.from_hf(hf_cfg.text_config.to_dict())
    ids = [2, 5, 6, 301] + [300] * 4 + [302, 7, 8, 9, 10, 11, 12]
    soft = torch.randn(4, cfg.hidden_size, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    rows = torch.tensor([4, 5, 6, 7])

    def extra(dev):
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        table = torch.arange(4, dtype=torch.int32, device=dev)[None]
        return dict(embed_rows=rows, embed_vals=soft, bidir=(i32([4]), i32([4]), i32([8]), table, 4, rows.to(dev)))

    want = _prefill_logits(LlamaModel.from_state_dict(cfg, dict(sd), device="cpu"), cfg, ids, "cpu", **extra("cpu"))
    got = _prefill_logits(LlamaModel.from_state_dict(cfg, dict(sd), device="cuda"), cfg, ids, "cuda", **extra("cuda"))
    assert float(torch.nn.functional.cosine_similarity(got, want, dim=-1).min()) > 0.99
