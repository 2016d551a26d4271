"""The fixed chunker and the chunk endpoint in the reference's contract (request: input + config; response: a list of
chunk objects with character or time spans), with the reference's own worked cases
(zig/pkg/inference/src/pipelines/chunking.zig tests, zig/lib/chunker/src/fixed_multimodal.zig tests)."""
import base64
import io
import wave

import numpy as np
import pytest
from fastapi.testclient import TestClient

from antfly_b200.api.model_manager import ModelManager
from antfly_b200.api.server import create_app
from antfly_b200.pipelines.chunking import chunk_binary, chunk_text


def test_fixed_text_chunker_worked_cases():
    assert chunk_text("") == []
    one = chunk_text("Hello world.", target_tokens=100)
    assert len(one) == 1 and one[0]["text"] == "Hello world." and (one[0]["start_char"], one[0]["end_char"]) == (0, 12)
    text = "alpha beta gamma delta epsilon zeta eta theta"
    ch = chunk_text(text, target_tokens=4, overlap_tokens=1, separator=" ")
    assert len(ch) >= 2 and ch[0]["start_char"] == 0
    assert all(text[c["start_char"]:c["end_char"]] == c["text"] for c in ch)
    assert all(len(c["text"].split()) <= 4 for c in ch)
    # every chunk after the first starts with the last token of its predecessor
    for a, b in zip(ch, ch[1:]):
        assert b["text"].split()[0] == a["text"].split()[-1] and b["start_char"] < a["end_char"]
    assert ch[-1]["text"].endswith("theta")
    with pytest.raises(ValueError):
        chunk_text(text, target_tokens=4, overlap_tokens=4)


def test_sections_fall_back_from_paragraphs_to_lines_to_sentences_and_cap_at_fifty():
    paras = "\n\n".join(f"Paragraph {i} has a few words in it." for i in range(6))
    ch = chunk_text(paras, target_tokens=20, overlap_tokens=0)
    assert all(c["text"].count("Paragraph") <= 2 for c in ch) and len(ch) >= 3
    assert "".join(c["text"] for c in ch).count("Paragraph") == 6               # nothing lost, nothing repeated
    lines = "\n".join(f"line {i} of the file" for i in range(8))              # no blank lines: newline sections
    assert len(chunk_text(lines, target_tokens=10, overlap_tokens=0)) == 4
    sent = "One two three. Four five six. Seven eight nine. Ten eleven twelve."
    ch = chunk_text(sent, target_tokens=8, overlap_tokens=0)
    assert [c["text"] for c in ch] == ["One two three. Four five six.", "Seven eight nine. Ten eleven twelve."]
    long_word_run = " ".join(str(i) for i in range(400))                       # one section far above the target
    ch = chunk_text(long_word_run, target_tokens=5, overlap_tokens=0)
    assert len(ch) == 50                                                       # the default cap
    assert len(chunk_text(long_word_run, target_tokens=5, overlap_tokens=0, max_chunks=7)) == 7


def _wav(samples, rate):
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(rate)
        w.writeframes((np.asarray(samples) * 32767).astype("<i2").tobytes())
    return buf.getvalue()


def test_audio_windows_and_gif_frames():
    data = _wav([0.0, 0.2, 0.4, 0.6, 0.8, 1.0], 1000)
    ch = chunk_binary("audio/wav", data, window_ms=3, overlap_ms=1, max_chunks=8)
    assert len(ch) == 3 and ch[0]["mime_type"] == "audio/wav"
    assert (ch[0]["start_time_ms"], ch[0]["end_time_ms"]) == (0.0, 3.0) and ch[1]["start_time_ms"] == 2.0
    with wave.open(io.BytesIO(ch[1]["data"]), "rb") as w:
        assert w.getnframes() == 3 and w.getframerate() == 1000
    with pytest.raises(ValueError):
        chunk_binary("audio/wav", data, window_ms=3, overlap_ms=3)
    gif = bytes.fromhex("4749463839610100010000000021ff0b4e45545343415045322e30030100000021f90401050000002c00000000"
                        "0100010081000000ff000000ff0000000002024c010021f90401070000002c000000000100010081000000ff0000"
                        "00ff0000000002025401003b")
    frames = chunk_binary("image/gif", gif, max_chunks=8)
    assert len(frames) == 2 and frames[0]["mime_type"] == "image/png" and frames[0]["frame_index"] == 0
    assert frames[0]["data"][:8] == b"\x89PNG\r\n\x1a\n" and frames[1]["frame_index"] == 1
    assert frames[1]["frame_delay_ms"] > 0
    assert chunk_binary("application/pdf", b"%PDF") == [{"id": 0, "mime_type": "application/pdf", "data": b"%PDF"}]


def test_chunk_endpoint_contract():
    c = TestClient(create_app(ModelManager(models_dir="/nonexistent", device="cpu")))
    text = "alpha beta gamma delta epsilon zeta eta theta"
    r = c.post("/ai/v1/chunk", json={"input": text, "config": {"model": "fixed", "text": {
        "target_tokens": 4, "overlap_tokens": 1, "separator": " "}}})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "list" and body["model"] == "fixed" and body["cache_hit"] is False
    assert body["usage"] == {"prompt_tokens": 8, "completion_tokens": 0, "total_tokens": 8}
    d = body["data"]
    assert [x["index"] for x in d] == list(range(len(d))) and all(x["object"] == "chunk" for x in d)
    assert all(x["mime_type"] == "text/plain" and text[x["start_char"]:x["end_char"]] == x["text"] for x in d)
    # content-part input, the deprecated ``text`` field and the older flat options give the same chunks
    same = c.post("/ai/v1/chunk", json={"input": {"type": "text", "text": text}, "config": {"text": {
        "target_tokens": 4, "overlap_tokens": 1, "separator": " "}}}).json()["data"]
    assert same == d
    flat = c.post("/ai/v1/chunk", json={"text": text, "target_tokens": 4, "overlap_tokens": 1}).json()
    assert [x["text"] for x in flat["chunks"]] == [x["text"] for x in flat["data"]] and len(flat["data"]) >= 2
    wav = base64.b64encode(_wav([0.0] * 50, 1000)).decode()
    r = c.post("/ai/v1/chunk", json={"input": {"type": "media", "mime_type": "audio/wav", "data": wav},
                                     "config": {"audio": {"window_duration_ms": 20, "overlap_duration_ms": 5}}})
    a = r.json()["data"]
    assert r.status_code == 200 and len(a) == 4 and a[1]["start_time_ms"] == 15.0 and a[0]["mime_type"] == "audio/wav"
    assert base64.b64decode(a[0]["data"])[:4] == b"RIFF"
    assert c.post("/ai/v1/chunk", json={"config": {}}).status_code == 400
    assert c.post("/ai/v1/chunk", json={"input": text, "config": {"text": {"target_tokens": 3, "overlap_tokens": 3}}}
                  ).status_code == 400


def _tone_wav(rate, spans, total_s, amp=0.3, noise=0.002, seed=0):
    import io
    import wave

    import numpy as np

    rng = np.random.default_rng(seed)
    n = int(rate * total_s)
    x = rng.normal(0, noise, n).astype(np.float32)
    t = np.arange(n) / rate
    for a, b in spans:
        m = (t >= a) & (t < b)
        x[m] += amp * np.sin(2 * np.pi * 220 * t[m]) * (0.6 + 0.4 * np.sin(2 * np.pi * 3 * t[m]))
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1); w.setsampwidth(2); w.setframerate(rate)
        w.writeframes((np.clip(x, -1, 1) * 32767).astype("<i2").tobytes())
    return buf.getvalue()


def test_vad_frame_merging_rules():
    from antfly_b200.pipelines.chunking import merge_vad_frames

    F, R = 512, 16000
    # frames: 10 speech, 3 silence, 10 speech, 30 silence, 2 speech (too short), 30 silence, 100 speech
    probs = [0.9] * 10 + [0.1] * 3 + [0.9] * 10 + [0.1] * 30 + [0.9] * 2 + [0.1] * 30 + [0.9] * 100
    segs = merge_vad_frames(probs, F, R, 0.5, 300, 250, 30, 0)
    # 3 silent frames = 96 ms < 300 ms: merged; the 64 ms blip is dropped; 30 ms of padding on each side
    pad = 30 * R // 1000
    assert segs == [(0, 23 * F + pad), (85 * F - pad, 185 * F)]
    assert merge_vad_frames(probs, F, R, 0.5, 50, 250, 0, 0)[:2] == [(0, 10 * F), (13 * F, 23 * F)]
    assert merge_vad_frames(probs, F, R, 0.5, 300, 30, 0, 0)[1] == (53 * F, 55 * F)          # the blip kept
    cut = merge_vad_frames(probs, F, R, 0.5, 300, 250, 0, 1000)
    assert cut[-4:] == [(85 * F, 85 * F + 16000), (85 * F + 16000, 85 * F + 32000), (85 * F + 32000, 85 * F + 48000),
                        (85 * F + 48000, 185 * F)]
    assert merge_vad_frames([0.1] * 20, F, R) == [] and merge_vad_frames([], F, R) == []


def test_vad_chunking_finds_the_speech_spans_and_the_endpoint_uses_it():
    import base64

    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app
    from antfly_b200.pipelines.chunking import chunk_wav_vad

    spans = [(0.5, 1.5), (3.0, 4.2)]
    for rate in (16000, 22050):
        data = _tone_wav(rate, spans, 5.0)
        chunks = chunk_wav_vad(data)
        assert len(chunks) == 2
        for ch, (a, b) in zip(chunks, spans):
            assert abs(ch["start_time_ms"] - a * 1000) < 80 and abs(ch["end_time_ms"] - b * 1000) < 80
            assert ch["data"][:4] == b"RIFF"
    assert chunk_wav_vad(_tone_wav(16000, [], 2.0)) == []                      # silence: nothing to transcribe
    assert len(chunk_wav_vad(_tone_wav(16000, [(0.2, 3.8)], 4.0), {"max_segment_duration_ms": 1000})) == 4
    client = TestClient(create_app(ModelManager(models_dir="/nonexistent", device="cpu")))
    body = {"input": {"type": "media", "mime_type": "audio/wav",
                      "data": base64.b64encode(_tone_wav(16000, spans, 5.0)).decode()},
            "config": {"audio": {"vad": {"min_silence_duration_ms": 200}}}}
    r = client.post("/ai/v1/chunk", json=body)
    assert r.status_code == 200, r.text
    got = r.json()["data"][0]["chunks"] if "data" in r.json() and "chunks" in r.json()["data"][0] else r.json()["data"]
    assert len(got) == 2 and got[0]["mime_type"] == "audio/wav"
    body["config"]["audio"] = {"window_duration_ms": 2000}
    r = client.post("/ai/v1/chunk", json=body)
    fixed = r.json()["data"][0]["chunks"] if "chunks" in r.json()["data"][0] else r.json()["data"]
    assert len(fixed) == 3                                                     # fixed windows without the vad section
