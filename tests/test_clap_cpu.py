"""CLAP audio / text towers and the audio front end against the Hugging Face implementation (CPU, fp32 weights)."""
import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from antfly_b200.models.clap import ClapConfig, ClapModel
from antfly_b200.ops import audio_ops as A


def _tiny(fusion: bool):
    torch.manual_seed(11)
    cfg = transformers.ClapConfig(
        text_config=dict(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, max_position_embeddings=40, pad_token_id=1, projection_dim=48,
                         hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0),
        audio_config=dict(spec_size=64, num_mel_bins=16, patch_size=4, patch_stride=[4, 4], window_size=4,
                          patch_embeds_hidden_size=16, depths=[2, 2], num_attention_heads=[2, 4], hidden_size=32,
                          projection_dim=48, enable_fusion=fusion, fusion_type="aff_2d" if fusion else None,
                          aff_block_r=4, drop_path_rate=0.0, attention_probs_dropout_prob=0.0),
        projection_dim=48)
    hf = transformers.ClapModel(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias") or "relative_position_bias_table" in n:
                p.normal_(0, 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("running_mean"):
                b.normal_(0, 0.5)
            elif n.endswith("running_var"):
                b.uniform_(0.5, 2.0)
    return cfg, hf


@pytest.mark.parametrize("fusion", [False, True])
def test_clap_towers_match_transformers(fusion):
    hf_cfg, hf = _tiny(fusion)
    cfg = ClapConfig.from_hf(hf_cfg.to_dict())
    assert cfg.audio.depths == [2, 2] and cfg.audio.enable_fusion == fusion and cfg.text.position_offset == 2
    model = ClapModel.from_state_dict(cfg, hf.state_dict(), device="cpu", dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    # 250 frames of 16 mel bins are stretched to 256 frames and folded into a 64 x 64 image
    feats = torch.randn(3, 4 if fusion else 1, 250, 16, generator=g) * 10 - 20
    longer = [True, False, True]
    with torch.no_grad():
        want = hf.get_audio_features(input_features=feats, is_longer=torch.tensor(longer)[:, None])
    want = getattr(want, "pooler_output", want).float()
    got = model.embed_audio(feats, longer)
    assert float(torch.nn.functional.cosine_similarity(got, want, dim=-1).min()) > 0.999
    torch.testing.assert_close(got, want, atol=3e-2, rtol=3e-2)

    seqs = [[0] + torch.randint(3, 190, (n,), generator=g).tolist() + [2] for n in (4, 11, 7)]
    L = max(len(s) for s in seqs)
    ids = torch.full((3, L), 1, dtype=torch.long)
    mask = torch.zeros_like(ids)
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.tensor(s)
        mask[i, : len(s)] = 1
    with torch.no_grad():
        want_t = hf.get_text_features(input_ids=ids, attention_mask=mask)
    want_t = getattr(want_t, "pooler_output", want_t).float()
    got_t = model.embed_text(seqs)
    assert float(torch.nn.functional.cosine_similarity(got_t, want_t, dim=-1).min()) > 0.999
    sim = got_t @ got.T
    assert sim.shape == (3, 3) and float(sim.abs().max()) <= 1 + 1e-5


def test_clap_front_end_matches_feature_extractor():
    fe = transformers.ClapFeatureExtractor(truncation="fusion", frequency_min=50, frequency_max=14000)
    g = torch.Generator().manual_seed(0)
    short = torch.randn(48000 * 3 + 123, generator=g) * 0.1
    want = fe(short.numpy(), sampling_rate=48000, return_tensors="pt")["input_features"][0]
    got, longer = A.clap_features(short, 4)
    assert not longer and got.shape == (4, 1001, 64)
    torch.testing.assert_close(got, want.float(), atol=2e-3, rtol=1e-4)
    # a long clip: plane 0 is the whole spectrogram shrunk to ten seconds' worth of frames; the three crops sit
    # at the front, the middle and the back (the training recipe draws them at random within those thirds)
    long = torch.randn(480000 + 48000 * 7, generator=g) * 0.1
    np.random.seed(0)
    want = fe(long.numpy(), sampling_rate=48000, return_tensors="pt")["input_features"][0]
    got, longer = A.clap_features(long, 4)
    assert longer and got.shape == (4, 1001, 64)
    torch.testing.assert_close(got[0], want[0].float(), atol=2e-3, rtol=1e-4)
    mel = A.clap_log_mel(long)
    total = mel.shape[0]
    torch.testing.assert_close(got[1], mel[:1001])
    torch.testing.assert_close(got[2], mel[(total - 1001) // 2:(total - 1001) // 2 + 1001])
    torch.testing.assert_close(got[3], mel[total - 1001:])
    # silence and a one-sample clip do not divide by zero
    assert torch.isfinite(A.clap_features(torch.zeros(0), 1)[0]).all()
    assert A.clap_features(torch.ones(1), 1)[0].shape == (1, 1001, 64)


def test_embed_endpoint_takes_audio_media_parts():
    """WAV bytes as a ``media`` content part beside text, through a CLAP embedder registered with the server."""
    import base64
    import io
    import wave

    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app
    from antfly_b200.pipelines.multimodal import ClapEmbedder
    from antfly_b200.tokenizer.tokenizer import ByteTokenizer

    hf_cfg, hf = _tiny(True)
    model = ClapModel.from_state_dict(ClapConfig.from_hf(hf_cfg.to_dict()), hf.state_dict(), device="cpu",
                                      dtype=torch.float32)
    # the tiny tower takes 16 mel bins x 256 frames; give the embedder a matching front end
    pipe = ClapEmbedder(model, ByteTokenizer(200), bos_id=0, eos_id=2)
    calls = []

    def fake_features(wave_48k, channels=4):
        calls.append(int(wave_48k.numel()))
        g = torch.Generator().manual_seed(int(wave_48k.numel()))
        return torch.randn(channels, 250, 16, generator=g) * 10 - 20, wave_48k.numel() > 480000

    import antfly_b200.ops.audio_ops as Au
    real = Au.clap_features
    Au.clap_features = fake_features
    try:
        mgr = ModelManager(models_dir="/nonexistent", device="cpu")
        mgr.register("tiny-clap", "embedder", pipe, pipe.tokenizer)
        c = TestClient(create_app(mgr))
        buf = io.BytesIO()
        with wave.open(buf, "wb") as w:
            w.setnchannels(1); w.setsampwidth(2); w.setframerate(16000)
            w.writeframes((np.sin(np.arange(8000) / 10.0) * 12000).astype("<i2").tobytes())
        b64 = base64.b64encode(buf.getvalue()).decode()
        r = c.post("/ai/v1/embed", json={"model": "tiny-clap", "input": [
            {"type": "text", "text": "a dog barking"},
            {"type": "media", "mime_type": "audio/wav", "data": b64},
            {"type": "audio", "data": "data:audio/wav;base64," + b64}]})
        assert r.status_code == 200, r.text
        data = r.json()["data"]
        assert len(data) == 3 and all(len(d["embedding"]) == 48 for d in data)
        assert all(abs(sum(v * v for v in d["embedding"]) - 1.0) < 1e-3 for d in data)
        assert data[1]["embedding"] == data[2]["embedding"]           # the same clip twice
        assert calls == [24000, 24000]                                # 0.5 s at 16 kHz resampled to 48 kHz
        r = c.post("/ai/v1/embed", json={"model": "tiny-clap", "input": [
            {"type": "media", "mime_type": "audio/wav", "data": "data:image/png;base64," + b64}]})
        assert r.status_code == 400 and "does not match" in r.json()["message"]
        r = c.post("/ai/v1/embed", json={"model": "tiny-clap", "input": [{"type": "media", "data": b64}]})
        assert r.status_code == 400 and "mime_type" in r.json()["message"]
    finally:
        Au.clap_features = real
