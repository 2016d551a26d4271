"""Audio front end (WAV decoding, resampling), the transcription pipeline's forced prompt, and the /transcribe
endpoint with a tiny random Whisper checkpoint."""
import base64
import io
import json
import math
import struct
import wave

import pytest
import torch
from fastapi.testclient import TestClient

from antfly_b200.ops import audio_ops as AO


def _wav_bytes(x: torch.Tensor, rate: int, width: int = 2, channels: int = 1) -> bytes:
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(channels)
        w.setsampwidth(width)
        w.setframerate(rate)
        pcm = (x.clamp(-1, 1) * (2 ** (8 * width - 1) - 1)).round().long()
        if width == 1:
            data = bytes(((pcm + 128) & 0xFF).tolist())
        else:
            data = b"".join(int(v).to_bytes(width, "little", signed=True) for v in pcm.tolist())
        w.writeframes(data if channels == 1 else b"".join(
            data[i:i + width] * channels for i in range(0, len(data), width)))
    return buf.getvalue()


@pytest.mark.parametrize("width", [1, 2, 3, 4])
def test_wav_decoding_by_sample_width_and_channels(width):
    t = torch.arange(800) / 8000
    x = 0.5 * torch.sin(2 * math.pi * 300 * t)
    got, rate = AO.read_wav(_wav_bytes(x, 8000, width, channels=2))
    assert rate == 8000 and got.shape == x.shape
    assert float((got - x).abs().max()) < (0.02 if width == 1 else 1e-3)
    with pytest.raises(ValueError):
        AO.read_wav(b"not a wav file at all")
    # 32-bit float WAV (format tag 3)
    data = x.numpy().astype("float32").tobytes()
    hdr = b"RIFF" + struct.pack("<I", 36 + len(data)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 3, 1, 8000, 32000, 4,
                                                                                    32) + b"data" + struct.pack(
        "<I", len(data))
    got, rate = AO.read_wav(hdr + data)
    assert rate == 8000 and torch.equal(got, x)


def test_resampling_keeps_tones_and_length():
    t = torch.arange(44100) / 44100
    x = 0.5 * torch.sin(2 * math.pi * 1000 * t)
    y = AO.resample(x, 44100)
    assert abs(y.numel() - 16000) <= 1
    ref = 0.5 * torch.sin(2 * math.pi * 1000 * torch.arange(y.numel()) / 16000)
    mid = slice(2000, 14000)                                   # away from the filter's edge transients
    assert float((y[mid] - ref[mid]).abs().max()) < 0.01
    # a tone above the new Nyquist frequency is removed, not aliased
    hi = AO.resample(0.5 * torch.sin(2 * math.pi * 12000 * t), 44100)
    assert float(hi[mid].abs().max()) < 0.02
    assert AO.resample(x, 16000) is x


def _write_whisper(dirpath):
    transformers = pytest.importorskip("transformers")
    from antfly_b200.formats import safetensors_io as st

    torch.manual_seed(0)
    cfg = transformers.WhisperConfig(vocab_size=300, num_mel_bins=80, d_model=64, encoder_layers=1,
                                     encoder_attention_heads=4, decoder_layers=1, decoder_attention_heads=4,
                                     encoder_ffn_dim=128, decoder_ffn_dim=128, max_source_positions=50,
                                     max_target_positions=32, decoder_start_token_id=258, eos_token_id=2,
                                     pad_token_id=0, bos_token_id=1, suppress_tokens=None, begin_suppress_tokens=None)
    hf = transformers.WhisperForConditionalGeneration(cfg)
    dirpath.mkdir(parents=True)
    sd = {k: v.contiguous() for k, v in hf.state_dict().items() if k != "proj_out.weight"}
    st.save_file(sd, str(dirpath / "model.safetensors"))
    (dirpath / "config.json").write_text(json.dumps({**{k: v for k, v in cfg.to_dict().items()
                                                        if isinstance(v, (int, float, str, bool))},
                                                     "model_type": "whisper"}))
    (dirpath / "generation_config.json").write_text(json.dumps({
        "decoder_start_token_id": 258, "lang_to_id": {"<|en|>": 259, "<|de|>": 260},
        "task_to_id": {"transcribe": 261, "translate": 262}, "no_timestamps_token_id": 263,
        "suppress_tokens": [1, 5000], "is_multilingual": True}))


def test_transcription_pipeline_and_endpoint(tmp_path):
    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    _write_whisper(tmp_path / "transcribers" / "tiny-whisper")
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")
    pipe = mgr.get("tiny-whisper", "transcriber").pipeline
    assert pipe.prompt() == [258] and pipe.prompt("en") == [258, 259, 261, 263]
    assert pipe.prompt("<|de|>", "translate") == [258, 260, 262, 263]
    with pytest.raises(ValueError):
        pipe.prompt("xx")
    t = torch.arange(8000 * 2) / 8000                          # 2 s at 8 kHz: resampled, one 1 s-window model
    x = 0.4 * torch.sin(2 * math.pi * 220 * t)
    out = pipe.transcribe(_wav_bytes(x, 8000), language="en", max_new_tokens=6)
    assert len(out.segments) == 1 and out.completion_tokens <= 6 and out.prompt_tokens == 4
    assert all(tok != 1 for s in out.segments for tok in s["tokens"])             # suppressed token never sampled
    direct = pipe.model.transcribe_ids(
        AO.log_mel(AO.resample(x, 8000), n_samples=pipe.frames * 160), [258, 259, 261, 263], 6, [1])
    assert out.segments[0]["tokens"] == direct
    c = TestClient(create_app(mgr))
    r = c.post("/ai/v1/transcribe", json={"model": "tiny-whisper", "language": "en", "max_tokens": 6,
                                          "audio": base64.b64encode(_wav_bytes(x, 8000)).decode()})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "list" and body["data"][0]["object"] == "transcription"
    assert body["data"][0]["text"] == out.text and body["usage"]["completion_tokens"] == out.completion_tokens
    assert c.post("/ai/v1/transcribe", json={"model": "tiny-whisper", "audio": "!!!"}).status_code == 400
    assert c.post("/ai/v1/transcribe", json={"model": "tiny-whisper",
                                             "audio": base64.b64encode(b"junk").decode()}).status_code == 400
    assert c.post("/ai/v1/transcribe", json={"model": "none", "audio": "AAAA"}).status_code == 404
    # the forced language is echoed; with none forced the decoder's most likely language token is used
    assert body["data"][0]["language"] == "en" and out.language == "en"
    auto = pipe.transcribe(_wav_bytes(x, 8000), max_new_tokens=4)
    mel = AO.log_mel(AO.resample(x, 8000), n_samples=pipe.frames * 160)
    logits = pipe.model.decode(pipe.model.start_decoding(pipe.model.encode(mel)), [258])[-1]
    want = "en" if float(logits[259]) >= float(logits[260]) else "de"
    assert auto.language == want and auto.prompt_tokens == 4
    assert auto.segments[0]["tokens"] == pipe.model.transcribe_ids(
        mel, [258, 259 if want == "en" else 260, 261, 263], 4, [1])
    r = c.post("/ai/v1/transcribe", json={"model": "tiny-whisper", "max_tokens": 4,
                                          "audio": base64.b64encode(_wav_bytes(x, 8000)).decode()})
    assert r.json()["data"][0]["language"] == want


def test_transcription_with_voice_activity_segments(tmp_path):
    """With vad options only the speech spans are decoded: two bursts separated by silence give two segments at the
    bursts' times; a silent recording gives none; the endpoint takes the same section."""
    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    _write_whisper(tmp_path / "transcribers" / "tiny-whisper")
    mgr = ModelManager(models_dir=str(tmp_path), device="cpu")
    pipe = mgr.get("tiny-whisper", "transcriber").pipeline
    rate = 16000
    t = torch.arange(rate * 4) / rate
    x = 0.002 * torch.randn(rate * 4, generator=torch.Generator().manual_seed(0))
    for a, b in ((0.5, 1.2), (2.5, 3.3)):
        m = (t >= a) & (t < b)
        x[m] += 0.4 * torch.sin(2 * math.pi * 220 * t[m])
    out = pipe.transcribe(_wav_bytes(x, rate), language="en", max_new_tokens=4, vad={})
    assert len(out.segments) == 2
    assert abs(out.segments[0]["start"] - 0.5) < 0.1 and abs(out.segments[0]["end"] - 1.2) < 0.1
    assert abs(out.segments[1]["start"] - 2.5) < 0.1 and abs(out.segments[1]["end"] - 3.3) < 0.1
    plain = pipe.transcribe(_wav_bytes(x, rate), language="en", max_new_tokens=4)
    assert len(plain.segments) == 1 and plain.segments[0]["end"] == 4.0   # without it: one window over everything
    quiet = pipe.transcribe(_wav_bytes(0.001 * torch.randn(rate * 2), rate), language="en", vad={})
    assert quiet.segments == [] and quiet.text == "" and quiet.completion_tokens == 0
    c = TestClient(create_app(mgr))
    r = c.post("/ai/v1/transcribe", json={"model": "tiny-whisper", "language": "en", "max_tokens": 4,
                                          "audio": base64.b64encode(_wav_bytes(x, rate)).decode(),
                                          "vad": {"min_silence_duration_ms": 200}})
    assert r.status_code == 200 and len(r.json()["data"][0]["segments"]) == 2
