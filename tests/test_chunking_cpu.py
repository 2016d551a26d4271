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
