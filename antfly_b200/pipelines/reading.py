"""Reading text out of images (OCR) with a vision encoder-decoder: decode the image, resize and normalise it on the
device (the image kernel), encode with the ViT, greedy-decode the text.  One line / crop per image, which is what
TrOCR checkpoints are trained on; the reference's reader task (zig/pkg/inference/src/pipelines/ocr_multistage.zig,
go/pkg/termite/lib/pipelines/vision2seq.go) has the same single-image contract for this model family."""
from __future__ import annotations

import re
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
    regions: List[dict] = field(default_factory=list)      # [{text, bbox [x1, y1, x2, y2] in pixels}] when the task has them


_LOC = re.compile(r"<loc_(\d+)>")


def parse_location_text(text: str, width: int, height: int, quads: bool = False) -> List[dict]:
    """Florence-2 region outputs -> regions.  The model writes a label (or a line of text) and its box as location
    tokens ``<loc_0>`` .. ``<loc_999>`` (thousandths of the image side): four per box for detection and region
    captions (several boxes may follow one label), eight per quadrilateral for OCR with regions (``quads``), in either order
    (text first or boxes first).  Boxes come back in pixels as [x1, y1, x2, y2] (quadrilaterals as their bounds)."""
    out: List[dict] = []
    pos, label = 0, ""
    for m in re.finditer(r"((?:<loc_\d+>)+)", text):
        before = text[pos:m.start()].replace("<s>", "").replace("</s>", "").replace("<pad>", "").strip()
        if before:
            label = before
        nums = [int(v) for v in _LOC.findall(m.group(1))]
        step = 8 if quads else 4
        for i in range(0, len(nums) - step + 1, step):
            xs = [nums[j] for j in range(i, i + step, 2)]
            ys = [nums[j] for j in range(i + 1, i + step, 2)]
            box = [min(xs), min(ys), max(xs), max(ys)]
            out.append({"text": label, "bbox": [round((box[0] + 0.5) / 1000 * width, 1),
                                                round((box[1] + 0.5) / 1000 * height, 1),
                                                round((box[2] + 0.5) / 1000 * width, 1),
                                                round((box[3] + 0.5) / 1000 * height, 1)]})
        pos = m.end()
    trailing = text[pos:].replace("<s>", "").replace("</s>", "").strip()
    if trailing and out and not out[-1]["text"]:      # boxes-first order: the text follows its box
        out[-1]["text"] = trailing
    return out


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
            raw = self.tokenizer.decode(toks)
            regions = parse_location_text(raw, int(img.shape[1]), int(img.shape[0]),
                                          quads=(prompt or "<OCR>") == "<OCR_WITH_REGION>") if "<loc_" in raw else []
            text = _LOC.sub(" ", raw).replace("<s>", "").replace("</s>", "").strip() if regions else \
                raw.replace("<s>", "").replace("</s>", "").strip()
            out.append(ReadResult(" ".join(text.split()) if regions else text, toks,
                                  {"preprocess": (t1 - t0) * 1e3, "decode": (t2 - t1) * 1e3}, regions))
        return out
