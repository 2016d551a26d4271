"""GPU runs of the decoders that keep their own sequence state (Qwen3.5, Gemma-4 text / vision / assistant,
DeepSeek-V4), of Florence-2, and of the Llama-family variants with soft caps and sinks, each against the same model
on the CPU (fp32)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

transformers = pytest.importorskip("transformers")


def _close(got, want, cos_min=0.99):
    got, want = got.float().cpu(), want.float().cpu()
    c = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    assert float(c) > cos_min, float(c)


def _steps(model, ids, cuts):
    st, out, at = None, [], 0
    for n in cuts:
        lg, st = model.forward(ids[at:at + n].to(model.device), st)
        out.append(lg.float().cpu())
        at += n
    return torch.cat(out)


def test_gemma4_text_prefill_and_decode_on_gpu():
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel
    from tests.test_gemma4_cpu import _hf

    for over in ({}, dict(enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=48)):
        hf_cfg, hf = _hf(**over)
        cfg = Gemma4Config.from_hf(hf_cfg.to_dict())
        ids = torch.randint(1, 200, (19,), generator=torch.Generator().manual_seed(1))
        cpu = Gemma4TextModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
        gpu = Gemma4TextModel.from_state_dict(cfg, hf.state_dict(), device="cuda", dtype=torch.bfloat16)
        _close(_steps(gpu, ids, [15, 1, 1, 2]), _steps(cpu, ids, [15, 1, 1, 2]))


def test_gemma4_vision_tower_and_assistant_on_gpu():
    from antfly_b200.models.gemma4 import Gemma4Config, Gemma4TextModel
    from antfly_b200.models.gemma4v import Gemma4VisionConfig, Gemma4VisionTower
    from tests.test_gemma4_cpu import _assistant, _hf
    from transformers.models.gemma4 import modeling_gemma4 as M

    torch.manual_seed(0)
    vcfg = transformers.Gemma4VisionConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                           num_attention_heads=1, num_key_value_heads=1, head_dim=64, patch_size=4,
                                           pooling_kernel_size=2, position_embedding_size=32)
    hf = M.Gemma4VisionModel(vcfg).eval().float()
    ys, xs = torch.meshgrid(torch.arange(4), torch.arange(4), indexing="ij")
    pos = torch.stack([xs.flatten(), ys.flatten()], -1)[None]
    pix = torch.rand(1, 16, 48)
    cfg = Gemma4VisionConfig.from_hf(vcfg.to_dict())
    cpu = Gemma4VisionTower.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    gpu = Gemma4VisionTower.from_state_dict(cfg, hf.state_dict(), device="cuda", dtype=torch.bfloat16)
    _close(gpu.forward(pix.cuda(), pos.cuda()), cpu.forward(pix, pos))
    hf_cfg, hft = _hf()
    target = Gemma4TextModel.from_state_dict(Gemma4Config.from_hf(hf_cfg.to_dict()), hft.state_dict(), device="cuda",
                                             dtype=torch.bfloat16)
    asst, sd = _assistant(target, hf_cfg)          # built on the CPU helper's dtype; rebuild on the device
    from antfly_b200.models.gemma4 import Gemma4Assistant

    conf = {"model_type": "gemma4_assistant", "text_config": asst.body.cfg.__dict__}
    asst = Gemma4Assistant.from_state_dict(conf, sd, target, device="cuda", dtype=torch.bfloat16)
    prompt = [5, 9, 17, 33, 2, 71, 8]
    assert asst.generate(prompt, 10, k=3) == target.generate(prompt, 10)


def test_qwen35_and_deepseek_v4_on_gpu():
    from antfly_b200.models import deepseek_v4 as V4
    from tests.test_deepseek_v4_cpu import _tiny

    cfg, sd = _tiny()
    ids = torch.randint(0, cfg.vocab_size, (9,), generator=torch.Generator().manual_seed(5))
    cpu = V4.DeepseekV4Model.from_state_dict(cfg, sd, device="cpu", dtype=torch.float32)
    gpu = V4.DeepseekV4Model.from_state_dict(cfg, sd, device="cuda", dtype=torch.bfloat16)
    _close(_steps(gpu, ids, [4, 1, 3, 1]), _steps(cpu, ids, [4, 1, 3, 1]), cos_min=0.98)
    from antfly_b200.models.qwen35 import Qwen35Config, Qwen35Model
    from tests.test_qwen35_cpu import _hf as _hf35

    hf_cfg, hf = _hf35()
    qcfg = Qwen35Config.from_hf(hf_cfg.to_dict())
    ids = torch.randint(1, hf_cfg.vocab_size, (14,), generator=torch.Generator().manual_seed(2))
    cpu = Qwen35Model.from_state_dict(qcfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    gpu = Qwen35Model.from_state_dict(qcfg, hf.state_dict(), device="cuda", dtype=torch.bfloat16)
    _close(_steps(gpu, ids, [10, 1, 3]), _steps(cpu, ids, [10, 1, 3]), cos_min=0.98)


def test_florence2_on_gpu():
    from antfly_b200.models.florence2 import Florence2Model
    from tests.test_florence2_cpu import _hf

    c, hf = _hf()
    px = torch.randn(1, 3, 80, 64)
    cpu = Florence2Model.from_state_dict(c.to_dict(), hf.state_dict(), device="cpu", dtype=torch.float32)
    gpu = Florence2Model.from_state_dict(c.to_dict(), hf.state_dict(), device="cuda", dtype=torch.bfloat16)
    _close(gpu.image_tokens(px.cuda()), cpu.image_tokens(px), cos_min=0.98)
    prompt = [0, 17, 33, 51, 2]
    a = gpu.decode(gpu.start_decoding(gpu.encode(prompt, px[0].cuda())), [2, 9, 14])
    b = cpu.decode(cpu.start_decoding(cpu.encode(prompt, px[0])), [2, 9, 14])
    _close(a, b, cos_min=0.98)


@pytest.mark.parametrize("kind", ["gemma2", "sinks"])
def test_llama_family_with_soft_caps_and_sinks_on_gpu(kind):
    from antfly_b200.models.llama import LlamaConfig, LlamaModel, StepBatch

    torch.manual_seed(0)
    if kind == "gemma2":
        hf_cfg = transformers.Gemma2Config(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                           num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                           query_pre_attn_scalar=48, sliding_window=8, attn_logit_softcapping=4.0,
                                           final_logit_softcapping=3.0, max_position_embeddings=256)
        sd = transformers.Gemma2ForCausalLM(hf_cfg).state_dict()
    else:
        hf_cfg = transformers.LlamaConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                          num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                          tie_word_embeddings=False)
        sd = dict(transformers.LlamaForCausalLM(hf_cfg).state_dict())
        for l in range(2):
            sd[f"model.layers.{l}.self_attn.sinks"] = torch.tensor([0.5, -0.3, 1.0, 0.0])
    outs = []
    for dev in ("cpu", "cuda"):
        model = LlamaModel.from_state_dict(LlamaConfig.from_hf(hf_cfg.to_dict()), {k: v.clone() for k, v in sd.items()},
                                           device=dev)
        kc = torch.zeros((2, 3, 16, model.Hkv, model.cfg.head_dim), dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        ids = torch.arange(7, 31, dtype=torch.int32, device=dev)
        pos = torch.arange(24, dtype=torch.int32, device=dev)
        table = torch.arange(3, dtype=torch.int32, device=dev)[None]
        pre = StepBatch(ids, pos, pos.clone(), i32([0]), i32([24]), i32([24]), table, pos.clone(), 24, 1)
        a = model.forward(pre, kc, vc).float().cpu()
        dec = StepBatch(i32([40]), i32([24]), i32([24]), i32([0]), i32([1]), i32([25]), table, i32([0]), 1, 1)
        outs.append(torch.cat([a, model.forward(dec, kc, vc).float().cpu()]))
    _close(outs[1], outs[0], cos_min=0.98)
