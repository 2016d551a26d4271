"""Fixed-size text chunker (the reference's fixed chunker behind ``/chunk``: target tokens, overlap, separator
preference; zig/pkg/inference/src/pipelines/chunking.zig)."""
from __future__ import annotations

import re
from typing import List, Optional, Tuple


_TOKEN = re.compile(r"\w+|[^\w\s]", re.UNICODE)
DEFAULT_MAX_CHUNKS = 50


def _tokens(text: str) -> List[Tuple[int, int]]:
    """(start, end) character spans of the chunker's token model: words and single punctuation marks.  (The
    reference counts with an embedded subword tokenizer, zig/lib/chunker/src/fixed_text.zig:35; only the counts
    differ, not the structure of the result.)"""
    return [m.span() for m in _TOKEN.finditer(text)]


def _split(text: str, start: int, sep: str) -> List[Tuple[str, int]]:
    """Pieces of ``text`` between occurrences of ``sep`` with their absolute start; a ". " separator keeps the
    full stop with the sentence."""
    if not sep:
        return [(text, start)]
    out, at = [], 0
    while at <= len(text):
        nxt = text.find(sep, at)
        if nxt < 0:
            nxt = len(text)
        end = nxt + 1 if sep == ". " and nxt < len(text) else nxt
        out.append((text[at:end], start + at))
        if nxt == len(text):
            break
        at = nxt + len(sep)
    return out


def _flatten(sections: List[Tuple[str, int]], target: int) -> List[Tuple[str, int, int]]:
    """Sections above the target are split by ever finer separators (newline, sentence, space), at last into token
    windows: -> (text, start, tokens)."""
    out: List[Tuple[str, int, int]] = []
    for text, start in sections:
        spans = _tokens(text)
        if len(spans) <= target:
            out.append((text, start, len(spans)))
            continue
        for sep in ("\n", ". ", " "):
            finer = _split(text, start, sep)
            if len(finer) > 1:
                out.extend(_flatten(finer, target))
                break
        else:
            for i in range(0, len(spans), target):
                a, b = spans[i][0], spans[min(i + target, len(spans)) - 1][1]
                out.append((text[a:b], start + a, min(target, len(spans) - i)))
    return out


def chunk_text(text: str, target_tokens: int = 500, overlap_tokens: int = 50, max_chunks: int = 0,
               separator: str = "\n\n") -> List[dict]:
    """Fixed-size chunking the way the reference's ``fixed`` chunker does it (zig/lib/chunker/src/fixed_text.zig):
    the text is cut at the separator (falling back to newlines, then sentences, when it does not occur), sections
    are packed greedily up to ``target_tokens``, every chunk after the first starts with the last
    ``overlap_tokens`` tokens of its predecessor, and at most ``max_chunks`` (default 50) chunks are returned.
    Chunks are spans of the source: ``text[start_char:end_char]``."""
    if not text:
        return []
    target = target_tokens if target_tokens > 0 else 500
    limit = max_chunks if max_chunks > 0 else DEFAULT_MAX_CHUNKS
    sep = separator or "\n\n"
    if overlap_tokens >= target:
        raise ValueError("overlap_tokens must be smaller than target_tokens")
    sections = _split(text, 0, sep)
    if len(sections) <= 1 and sep != "\n":
        sections = _split(text, 0, "\n")
    if len(sections) <= 1:
        sections = _split(text, 0, ". ")
    chunks: List[dict] = []

    def emit(cur):
        a, b = cur[0][1], cur[-1][1] + len(cur[-1][0])
        chunks.append({"id": len(chunks), "text": text[a:b], "start_char": a, "end_char": b})

    cur: List[Tuple[str, int, int]] = []
    count = 0
    for sec in _flatten(sections, target):
        if count > 0 and count + sec[2] > target:
            emit(cur)
            if len(chunks) >= limit:
                return chunks
            prev = chunks[-1]
            cur, count = [], 0
            if overlap_tokens > 0:
                spans = _tokens(prev["text"])
                if len(spans) > overlap_tokens:
                    a = spans[len(spans) - overlap_tokens][0]
                    cur, count = [(prev["text"][a:], prev["start_char"] + a, overlap_tokens)], overlap_tokens
                elif spans:
                    cur, count = [(prev["text"], prev["start_char"], len(spans))], len(spans)
        cur.append(sec)
        count += sec[2]
    if cur and len(chunks) < limit:
        emit(cur)
    return chunks


def chunk_wav(data: bytes, window_ms: int = 30000, overlap_ms: int = 0, max_chunks: int = 0) -> List[dict]:
    """Fixed windows over a WAV file, each returned as a mono 16-bit WAV of its own with its time span
    (zig/lib/chunker/src/fixed_multimodal.zig chunkWav)."""
    import io
    import wave

    import numpy as np

    with wave.open(io.BytesIO(data), "rb") as w:
        rate, ch, width, n = w.getframerate(), w.getnchannels(), w.getsampwidth(), w.getnframes()
        raw = w.readframes(n)
    if width == 2:
        x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
    elif width == 1:
        x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    elif width == 4:
        x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
    else:
        raise ValueError(f"unsupported WAV sample width {width}")
    x = x.reshape(-1, ch).mean(1) if ch > 1 else x
    win = rate * (window_ms if window_ms > 0 else 30000) // 1000
    ovl = rate * max(overlap_ms, 0) // 1000
    if win == 0:
        raise ValueError("audio window is shorter than one sample")
    if ovl >= win:
        raise ValueError("audio overlap must be shorter than the window")
    out, off = [], 0
    while off < len(x):
        end = min(off + win, len(x))
        buf = io.BytesIO()
        with wave.open(buf, "wb") as w:
            w.setnchannels(1)
            w.setsampwidth(2)
            w.setframerate(rate)
            w.writeframes((np.clip(x[off:end], -1.0, 1.0) * 32767.0).round().astype("<i2").tobytes())
        out.append({"id": len(out), "mime_type": "audio/wav", "data": buf.getvalue(),
                    "start_time_ms": off * 1000.0 / rate, "end_time_ms": end * 1000.0 / rate})
        if max_chunks and len(out) >= max_chunks:
            break
        off += win - ovl
    return out


def chunk_gif(data: bytes, max_chunks: int = 0) -> List[dict]:
    """Frames of an animated GIF as PNG images with their display delay (fixed_multimodal.zig chunkGif)."""
    import io

    from PIL import Image, ImageSequence

    out = []
    with Image.open(io.BytesIO(data)) as im:
        for i, frame in enumerate(ImageSequence.Iterator(im)):
            buf = io.BytesIO()
            frame.convert("RGBA").save(buf, format="PNG")
            out.append({"id": i, "mime_type": "image/png", "data": buf.getvalue(), "frame_index": i,
                        "frame_delay_ms": int(frame.info.get("duration", 0))})
            if max_chunks and len(out) >= max_chunks:
                break
    return out


VAD_FRAME = 512                     # samples per frame at 16 kHz (32 ms), the frame of the reference's detector
VAD_DEFAULTS = {"threshold": 0.5, "min_silence_duration_ms": 300, "min_speech_duration_ms": 250, "speech_pad_ms": 30,
                "max_segment_duration_ms": 30000}


def vad_frame_probs(x16k) -> "np.ndarray":
    """Speech probability per 512-sample frame of 16 kHz mono audio, without a model: frame log-energy against a
    running noise floor (a low percentile of the recording's frame energies), squashed to (0, 1).  The reference
    runs a neural detector here (Silero, go/pkg/termite/lib/chunking/vad_audio_chunker.go:217-266); everything
    downstream of the probabilities follows its rules."""
    import numpy as np

    n = len(x16k) // VAD_FRAME
    if n == 0:
        return np.zeros(0, dtype=np.float32)
    frames = np.asarray(x16k[: n * VAD_FRAME], dtype=np.float32).reshape(n, VAD_FRAME)
    frames = frames - frames.mean(1, keepdims=True)
    db = 10.0 * np.log10((frames ** 2).mean(1) + 1e-10)
    k = max(3, n // 20)
    floor = max(float(np.sort(db)[:k].mean()), -80.0)            # the quietest twentieth of the recording
    # 0.5 at 9 dB above the floor, about 0.9 at 15 dB; the mid-point is kept between -50 and -35 dBFS, so a
    # recording that is quiet throughout has no speech and one that is loud throughout (no pauses to take a floor
    # from) is all speech
    mid = min(max(floor + 9.0, -50.0), -35.0)
    return (1.0 / (1.0 + np.exp(-(db - mid) / 2.7))).astype(np.float32)


def merge_vad_frames(probs, frame_samples: int, sample_rate: int, threshold: float = 0.5,
                     min_silence_duration_ms: int = 300, min_speech_duration_ms: int = 250, speech_pad_ms: int = 30,
                     max_segment_duration_ms: int = 30000) -> List[tuple]:
    """Per-frame speech probabilities -> [(start_sample, end_sample)]: threshold, runs of speech frames, runs shorter
    than the minimum speech length dropped, neighbours closer than the minimum silence merged, padding on both sides
    (clipped to the recording), segments longer than the maximum cut into pieces of the maximum length
    (go/pkg/termite/lib/chunking/vad_audio_chunker.go:272-375)."""
    raw, start = [], None
    for i, p in enumerate(probs):
        if p >= threshold and start is None:
            start = i
        elif p < threshold and start is not None:
            raw.append((start * frame_samples, i * frame_samples))
            start = None
    if start is not None:
        raw.append((start * frame_samples, len(probs) * frame_samples))
    min_speech = min_speech_duration_ms * sample_rate // 1000
    kept = [s for s in raw if s[1] - s[0] >= min_speech]
    if not kept:
        return []
    min_sil = min_silence_duration_ms * sample_rate // 1000
    merged = [list(kept[0])]
    for a, b in kept[1:]:
        if a - merged[-1][1] < min_sil:
            merged[-1][1] = b
        else:
            merged.append([a, b])
    pad, total = speech_pad_ms * sample_rate // 1000, len(probs) * frame_samples
    merged = [(max(a - pad, 0), min(b + pad, total)) for a, b in merged]
    if max_segment_duration_ms <= 0:
        return merged
    cap = max_segment_duration_ms * sample_rate // 1000
    out = []
    for a, b in merged:
        for s0 in range(a, b, cap):
            out.append((s0, min(s0 + cap, b)))
    return out


def chunk_wav_vad(data: bytes, vad: Optional[dict] = None, max_chunks: int = 0) -> List[dict]:
    """Speech segments of a WAV file as chunks (mono 16-bit WAV each, with their time span): voice-activity
    segmentation instead of fixed windows.  ``vad`` carries the request's overrides of :data:`VAD_DEFAULTS`."""
    import io
    import wave

    import numpy as np

    from ..ops.audio_ops import read_wav, resample

    cfg = dict(VAD_DEFAULTS)
    cfg.update({k: v for k, v in (vad or {}).items() if k in cfg and v})
    wave_t, rate = read_wav(data)
    x = wave_t.numpy()
    x16 = x if rate == 16000 else resample(wave_t, rate, 16000).numpy()
    segs = merge_vad_frames(vad_frame_probs(x16), VAD_FRAME, 16000, float(cfg["threshold"]),
                            int(cfg["min_silence_duration_ms"]), int(cfg["min_speech_duration_ms"]),
                            int(cfg["speech_pad_ms"]), int(cfg["max_segment_duration_ms"]))
    out = []
    for a, b in segs:
        lo, hi = a * rate // 16000, min(b * rate // 16000, len(x))
        buf = io.BytesIO()
        with wave.open(buf, "wb") as w:
            w.setnchannels(1)
            w.setsampwidth(2)
            w.setframerate(rate)
            w.writeframes((np.clip(x[lo:hi], -1.0, 1.0) * 32767.0).round().astype("<i2").tobytes())
        out.append({"id": len(out), "mime_type": "audio/wav", "data": buf.getvalue(),
                    "start_time_ms": a * 1000.0 / 16000, "end_time_ms": b * 1000.0 / 16000})
        if max_chunks and len(out) >= max_chunks:
            break
    return out


def chunk_binary(mime_type: str, data: bytes, window_ms: int = 30000, overlap_ms: int = 0,
                 max_chunks: int = 0, vad: Optional[dict] = None) -> List[dict]:
    """WAV audio in windows (or in speech segments when voice-activity options are given), GIF animations in frames,
    anything else as one chunk."""
    if mime_type == "audio/wav" and vad is not None:
        return chunk_wav_vad(data, vad, max_chunks)
    if mime_type == "audio/wav":
        return chunk_wav(data, window_ms, overlap_ms, max_chunks)
    if mime_type == "image/gif":
        return chunk_gif(data, max_chunks)
    return [{"id": 0, "mime_type": mime_type, "data": data}]


class NeuralChunker:
    """Semantic chunking with a token-classification model that marks the tokens after which a new chunk starts
    (checkpoints in the style of the reference's ``chunkers/`` models, go/pkg/termite/lib/pipelines/chunking.go: a
    binary ``separator`` label per token).  Long texts are tagged in windows of the model's context; boundaries that
    would make a chunk longer than ``max_tokens`` are supplemented by a hard cut, tiny chunks are merged forward."""

    def __init__(self, tagger, boundary_labels=("separator", "B", "B-SEP", "LABEL_1"), window_tokens: int = 510,
                 threshold: float = 0.5):
        self.tagger, self.labels, self.window, self.threshold = tagger, set(boundary_labels), window_tokens, threshold

    def _pieces(self, text: str):
        """(token id, start char, end char) for the whole text, without special tokens."""
        tk = self.tagger.tokenizer
        inner = getattr(tk, "tk", None)
        if inner is not None and hasattr(inner, "encode"):            # Hugging Face tokenizers: exact offsets
            enc = inner.encode(text, add_special_tokens=False)
            return [(i, a, b) for i, (a, b) in zip(enc.ids, enc.offsets)]
        ids = tk.encode(text)
        out, cursor = [], 0
        for i in ids:                                                   # fall back to decoding token by token
            piece = tk.decode([i])
            at = text.find(piece, cursor) if piece else -1
            if at < 0:
                at = cursor
            out.append((i, at, at + len(piece)))
            cursor = at + len(piece)
        return out

    def chunk(self, text: str, max_tokens: int = 500, min_tokens: int = 8, max_chunks: int = 0) -> List[dict]:
        pieces = self._pieces(text)
        if not pieces:
            return []
        tk = self.tagger.tokenizer
        cls_id, sep_id = tk.special.cls_id, tk.special.sep_id
        cut_after = [False] * len(pieces)
        for lo in range(0, len(pieces), self.window):
            win = pieces[lo:lo + self.window]
            seq = [cls_id] + [p[0] for p in win] + [sep_id]
            tags, scores = self.tagger.tag_ids([seq])[0]
            for j in range(len(win)):
                if tags[j + 1] in self.labels and scores[j + 1] >= self.threshold:
                    cut_after[lo + j] = True
        chunks, start = [], 0
        for i in range(len(pieces)):
            n = i - start + 1
            last = i == len(pieces) - 1
            if last or n >= max_tokens or (cut_after[i] and n >= min_tokens):
                a, b = pieces[start][1], pieces[i][2]
                chunks.append({"id": len(chunks), "text": text[a:b], "start_char": a, "end_char": b, "tokens": n})
                start = i + 1
                if max_chunks and len(chunks) >= max_chunks:
                    break
        return chunks
