"""Reading text out of images (OCR) with a vision encoder-decoder: decode the image, resize and normalise it on the
device (the image kernel), encode with the ViT, greedy-decode the text.  One line / crop per image, which is what
TrOCR checkpoints are trained on; the reference's reader task (zig/pkg/inference/src/pipelines/ocr_multistage.zig,
go/pkg/termite/lib/pipelines/vision2seq.go) has the same single-image contract for this model family."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import torch

from ..models.trocr import TrOCRModel
from ..ops import image_ops as IM


@dataclass
class ReadResult:
    text: str
    token_ids: List[int]
    timing_ms: Dict[str, float] = field(default_factory=dict)


class Reader:
    def __init__(self, model: TrOCRModel, tokenizer, mean: Sequence[float] = (0.5, 0.5, 0.5),
                 std: Sequence[float] = (0.5, 0.5, 0.5), mode: str = "bilinear"):
        self.model, self.tokenizer, self.mean, self.std, self.mode = model, tokenizer, tuple(mean), tuple(std), mode

    def preprocess(self, image: torch.Tensor) -> torch.Tensor:
        """uint8 [H, W, 3 | 4] -> normalised [3, S, S] at the encoder's resolution (whole image, aspect not kept)."""
        s = self.model.cfg.encoder.image_size
        dev = self.model.device
        return IM.preprocess(image.to(dev) if dev.type == "cuda" else image, (s, s), self.mean, self.std, self.mode)[0]

    def read(self, images: Sequence[torch.Tensor], max_new_tokens: int = 256, prompt=None) -> List[ReadResult]:
        out = []                                            # (TrOCR is pure OCR: a task prompt has no effect)
        for img in images:
            t0 = time.perf_counter()
            px = self.preprocess(img)
            t1 = time.perf_counter()
            ids = self.model.read_ids(px, max_new_tokens)
            t2 = time.perf_counter()
            text = self.tokenizer.decode(ids).strip() if self.tokenizer is not None else ""
            out.append(ReadResult(text, ids, {"preprocess": (t1 - t0) * 1e3, "decode": (t2 - t1) * 1e3}))
        return out


class FlorenceReader:
    """Florence-2 as a reader: the task prompt (``<OCR>`` by default; ``<CAPTION>``, ``<OD>``, ... or free text) is
    rewritten to the sentence the model was trained on, wrapped in begin / end markers, and encoded behind the image
    tokens; decoding is greedy with the reference reader's no-repeat-n-gram guard and ``<s>`` / ``</s>`` are stripped
    from the text (zig/pkg/inference/src/pipelines/reading.zig:130-175, 358-410)."""

    def __init__(self, model, tokenizer, mean: Sequence[float] = (0.485, 0.456, 0.406),
                 std: Sequence[float] = (0.229, 0.224, 0.225), mode: str = "bicubic", image_size: int = 768,
                 no_repeat_ngram_size: int = 3):
        self.model, self.tokenizer = model, tokenizer
        self.mean, self.std, self.mode, self.image_size = tuple(mean), tuple(std), mode, image_size
        self.no_repeat_ngram_size = no_repeat_ngram_size

    def preprocess(self, image: torch.Tensor) -> torch.Tensor:
        dev = self.model.device
        s = self.image_size
        return IM.preprocess(image.to(dev) if dev.type == "cuda" else image, (s, s), self.mean, self.std, self.mode)[0]

    def prompt_ids(self, prompt: str) -> List[int]:
        from ..models.florence2 import FLORENCE_TASK_PROMPTS

        cfg = self.model.cfg
        text = FLORENCE_TASK_PROMPTS.get(prompt, prompt)
        return [cfg.bos_token_id] + list(self.tokenizer.encode(text)) + [cfg.eos_token_id]

    def read(self, images: Sequence[torch.Tensor], max_new_tokens: int = 256, prompt=None) -> List[ReadResult]:
        ids = self.prompt_ids(prompt or "<OCR>")
        out = []
        for img in images:
            t0 = time.perf_counter()
            px = self.preprocess(img)
            t1 = time.perf_counter()
            toks = self.model.generate(ids, px, max_new_tokens, self.no_repeat_ngram_size)
            t2 = time.perf_counter()
            text = self.tokenizer.decode(toks).replace("<s>", "").replace("</s>", "").strip()
            out.append(ReadResult(text, toks, {"preprocess": (t1 - t0) * 1e3, "decode": (t2 - t1) * 1e3}))
        return out
