"""Speech-to-text pipeline over the Whisper model: decode the audio container, resample to 16 kHz, cut into 30 s
windows, build log-mel features, and greedy-decode each window from the forced task prompt.

Prompt and suppression lists come from the checkpoint's ``generation_config.json`` when present
(``decoder_start_token_id``, ``lang_to_id``, ``task_to_id``, ``no_timestamps_token_id``, ``suppress_tokens``), as in
the reference's transcription pipeline (zig/pkg/inference/src/pipelines/transcription.zig, pipelines/audio.zig).
Only WAV containers are decoded here; compressed formats need to be converted by the caller.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Union

import torch

from ..models.whisper import WhisperModel
from ..ops import audio_ops as AO


@dataclass
class Transcription:
    text: str
    segments: List[dict]
    prompt_tokens: int
    completion_tokens: int
    timing_ms: Dict[str, float] = field(default_factory=dict)
    language: Optional[str] = None          # forced, or detected from the first window (multilingual checkpoints)


class Transcriber:
    def __init__(self, model: WhisperModel, tokenizer, generation_config: Optional[dict] = None,
                 chunk_seconds: int = 30):
        self.model, self.tokenizer, self.gen = model, tokenizer, generation_config or {}
        self.chunk = chunk_seconds * AO.SAMPLE_RATE
        self.frames = 2 * model.cfg.max_source_positions          # mel frames the encoder expects

    def prompt(self, language: Optional[str] = None, task: str = "transcribe") -> List[int]:
        g = self.gen
        ids = [int(g.get("decoder_start_token_id", self.model.cfg.decoder_start_token_id))]
        lang_ids = g.get("lang_to_id") or {}
        if language:
            key = language if language.startswith("<|") else f"<|{language}|>"
            if lang_ids and key not in lang_ids:
                raise ValueError(f"language {language!r} is not known to this model")
            if key in lang_ids:
                ids.append(int(lang_ids[key]))
        elif lang_ids and "<|en|>" in lang_ids and not g.get("is_multilingual", True):
            ids.append(int(lang_ids["<|en|>"]))
        task_ids = g.get("task_to_id") or {}
        if task in task_ids and len(ids) > 1:
            ids.append(int(task_ids[task]))
        if g.get("no_timestamps_token_id") is not None and len(ids) > 1:
            ids.append(int(g["no_timestamps_token_id"]))
        return ids

    def detect_language(self, mel: torch.Tensor) -> Optional[str]:
        """The language token the decoder finds most likely right after the start token (logits restricted to the
        checkpoint's language tokens); None for English-only checkpoints or ones without a language table."""
        lang_ids = self.gen.get("lang_to_id") or {}
        if not lang_ids or not self.gen.get("is_multilingual", True):
            return None
        start = int(self.gen.get("decoder_start_token_id", self.model.cfg.decoder_start_token_id))
        logits = self.model.decode(self.model.start_decoding(self.model.encode(mel)), [start])[-1].float()
        keys = list(lang_ids)
        ids = torch.tensor([int(lang_ids[k]) for k in keys], device=logits.device)
        return keys[int(logits[ids].argmax())].strip("<|>")

    def transcribe(self, audio: Union[bytes, str, torch.Tensor], sample_rate: Optional[int] = None,
                   language: Optional[str] = None, task: str = "transcribe",
                   max_new_tokens: int = 224, vad: Optional[dict] = None) -> Transcription:
        """``vad`` (voice-activity options, possibly empty): only the speech segments are decoded -- silence costs
        nothing and cannot be hallucinated over -- each as a window of its own (segments are cut at the model's
        30 s window by the segmenter)."""
        t0 = time.perf_counter()
        if isinstance(audio, torch.Tensor):
            wav, rate = audio.float().flatten(), sample_rate or AO.SAMPLE_RATE
        else:
            wav, rate = AO.read_wav(audio)
        wav = AO.resample(wav, rate)
        t1 = time.perf_counter()
        if not language:                                      # multilingual checkpoint, nothing forced: detect once
            first = AO.log_mel(wav[: self.chunk].to(self.model.device), self.model.cfg.num_mel_bins,
                               n_samples=self.frames * 160)
            language = self.detect_language(first)
        prompt = self.prompt(language, task)
        suppress = [int(t) for t in (self.gen.get("suppress_tokens") or []) if 0 <= int(t) < self.model.cfg.vocab_size]
        segments, n_prompt, n_out = [], 0, 0
        if vad is not None:
            from .chunking import VAD_DEFAULTS, VAD_FRAME, merge_vad_frames, vad_frame_probs

            cfg = dict(VAD_DEFAULTS)
            cfg.update({k: v for k, v in vad.items() if k in cfg and v})
            cfg["max_segment_duration_ms"] = min(int(cfg["max_segment_duration_ms"]), self.chunk * 1000 // AO.SAMPLE_RATE)
            spans = merge_vad_frames(vad_frame_probs(wav.cpu().numpy()), VAD_FRAME, AO.SAMPLE_RATE,
                                     float(cfg["threshold"]), int(cfg["min_silence_duration_ms"]),
                                     int(cfg["min_speech_duration_ms"]), int(cfg["speech_pad_ms"]),
                                     int(cfg["max_segment_duration_ms"]))
        else:
            spans = [(i, min(i + self.chunk, wav.numel())) for i in range(0, max(wav.numel(), 1), self.chunk)]
        for i, j in spans:
            piece = wav[i:j]
            mel = AO.log_mel(piece.to(self.model.device), self.model.cfg.num_mel_bins,
                             n_samples=self.frames * 160)
            ids = self.model.transcribe_ids(mel, prompt, max_new_tokens, suppress)
            text = self.tokenizer.decode(ids).strip() if self.tokenizer is not None else ""
            segments.append({"start": i / AO.SAMPLE_RATE, "end": j / AO.SAMPLE_RATE, "text": text, "tokens": ids})
            n_prompt += len(prompt)
            n_out += len(ids)
        t2 = time.perf_counter()
        return Transcription(" ".join(s["text"] for s in segments if s["text"]).strip(), segments, n_prompt, n_out,
                             {"decode_audio": (t1 - t0) * 1e3, "transcribe": (t2 - t1) * 1e3,
                              "total": (t2 - t0) * 1e3}, language=language.strip("<|>") if language else None)
