"""Layout-aware word labelling: words with their page boxes (from an OCR pass or a PDF text layer), optionally the
page image, through a LayoutLMv3 token classifier.

Every word is tokenised on its own; its sub-tokens share the word's box, ``<s>`` / ``</s>`` get the empty box, and
the word's label is the prediction at its first sub-token.  Pages longer than the model's window are processed in
consecutive windows of whole words.  ``group_entities`` joins B- / I- tagged words into fields with the union of
their boxes (the reference's layout extraction step, zig/pkg/inference/src/architectures/layoutlmv3.zig).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..models.layoutlmv3 import Document, LayoutLMv3Model

IMAGE_MEAN = IMAGE_STD = (0.5, 0.5, 0.5)


@dataclass
class WordLabel:
    word: str
    box: Tuple[int, int, int, int]
    label: str
    score: float


def normalize_box(box: Sequence[float], width: float, height: float) -> Tuple[int, int, int, int]:
    """Pixel box -> the 0..1000 page scale the model was trained on."""
    x0, y0, x1, y1 = box
    f = lambda v, s: max(0, min(1000, int(1000 * v / max(s, 1))))
    return f(x0, width), f(y0, height), f(x1, width), f(y1, height)


def page_pixels(image: torch.Tensor, size: int) -> torch.Tensor:
    """uint8 [H, W, 3] page -> [3, size, size] in [-1, 1] (plain bilinear resize: the whole page is kept, as the
    boxes refer to it)."""
    x = image.permute(2, 0, 1)[None].float() / 255.0
    x = torch.nn.functional.interpolate(x, size=(size, size), mode="bilinear", align_corners=False, antialias=True)[0]
    m, s = torch.tensor(IMAGE_MEAN)[:, None, None], torch.tensor(IMAGE_STD)[:, None, None]
    return (x - m) / s


class LayoutTokenClassifier:
    def __init__(self, model: LayoutLMv3Model, tokenizer, id2label: Dict[int, str], bos_id: int = 0, eos_id: int = 2):
        self.model, self.tok, self.id2label = model, tokenizer, id2label
        self.bos_id, self.eos_id = bos_id, eos_id
        self.window = model.cfg.max_position_embeddings - model.cfg.pad_token_id - 1

    def label_words(self, words: Sequence[str], boxes: Sequence[Sequence[int]],
                    image: Optional[torch.Tensor] = None) -> List[WordLabel]:
        """``boxes`` are on the 0..1000 scale (see :func:`normalize_box`); ``image`` is the uint8 page, if any."""
        if len(words) != len(boxes):
            raise ValueError("one box per word is required")
        px = page_pixels(image, self.model.cfg.input_size) if image is not None and self.model.cfg.visual_embed else None
        pieces = [list(self.tok.encode(w)) or [self.tok.special.unk_id or 3] for w in words]
        docs, spans = [], []
        i = 0
        while i < len(words):
            ids, bx, firsts, j = [self.bos_id], [(0, 0, 0, 0)], [], i
            while j < len(words) and len(ids) + len(pieces[j]) + 1 <= self.window:
                firsts.append(len(ids))
                ids += pieces[j]
                bx += [tuple(int(v) for v in boxes[j])] * len(pieces[j])
                j += 1
            if j == i:                               # a single word longer than the window: cut it
                firsts.append(1)
                ids += pieces[j][: self.window - 2]
                bx += [tuple(int(v) for v in boxes[j])] * (len(ids) - 1)
                j += 1
            ids.append(self.eos_id)
            bx.append((0, 0, 0, 0))
            docs.append(Document(ids, bx, px))
            spans.append((i, j, firsts))
            i = j
        out: List[WordLabel] = []
        for (a, b, firsts), lg in zip(spans, self.model.token_logits(docs)):
            pr = torch.softmax(lg.float().cpu(), -1)
            for w, f in zip(range(a, b), firsts):
                sc, k = pr[f].max(0)
                out.append(WordLabel(words[w], tuple(int(v) for v in boxes[w]), self.id2label.get(int(k), str(int(k))),
                                     float(sc)))
        return out


def group_entities(labels: Sequence[WordLabel]) -> List[dict]:
    """B- / I- (or bare) tags -> fields: consecutive words of one type become one entity whose box is the union of
    its words' boxes and whose score is their mean; ``O`` words are dropped."""
    out: List[dict] = []
    cur = None
    for wl in labels:
        tag = wl.label
        kind = tag[2:] if tag[:2] in ("B-", "I-", "S-", "E-") else tag
        if tag in ("O", "o") or not kind:
            cur = None
            continue
        if cur is not None and cur["label"] == kind and not tag.startswith(("B-", "S-")):
            cur["words"].append(wl.word)
            cur["scores"].append(wl.score)
            b = cur["box"]
            cur["box"] = (min(b[0], wl.box[0]), min(b[1], wl.box[1]), max(b[2], wl.box[2]), max(b[3], wl.box[3]))
        else:
            cur = {"label": kind, "words": [wl.word], "scores": [wl.score], "box": tuple(wl.box)}
            out.append(cur)
    return [{"label": e["label"], "text": " ".join(e["words"]), "box": list(e["box"]),
             "score": sum(e["scores"]) / len(e["scores"])} for e in out]


class DocumentClassifier:
    """Page-level labels (invoice / letter / form ...) from a LayoutLMv3 sequence-classification checkpoint: the
    first window of the page's words, their boxes and the page image decide."""

    def __init__(self, model: LayoutLMv3Model, tokenizer, id2label: Dict[int, str], bos_id: int = 0, eos_id: int = 2):
        self._tok = LayoutTokenClassifier(model, tokenizer, id2label, bos_id, eos_id)
        self.model, self.id2label = model, id2label

    def classify(self, words: Sequence[str], boxes: Sequence[Sequence[int]], image: Optional[torch.Tensor] = None,
                 top_k: int = 1) -> List[dict]:
        t = self._tok
        px = page_pixels(image, self.model.cfg.input_size) if image is not None and self.model.cfg.visual_embed else None
        ids, bx = [t.bos_id], [(0, 0, 0, 0)]
        for w, b in zip(words, boxes):
            sub = list(t.tok.encode(w))
            if len(ids) + len(sub) + 1 > t.window:
                break
            ids += sub
            bx += [tuple(int(v) for v in b)] * len(sub)
        doc = Document(ids + [t.eos_id], bx + [(0, 0, 0, 0)], px)
        pr = torch.softmax(self.model.sequence_logits([doc])[0].cpu(), -1)
        top = torch.topk(pr, min(max(top_k, 1), pr.numel()))
        return [{"label": self.id2label.get(int(i), str(int(i))), "score": float(s)}
                for s, i in zip(top.values.tolist(), top.indices.tolist())]
