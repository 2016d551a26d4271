"""Multi-stage OCR: find text regions on a page, read each region with a recogniser, put the results in reading
order, and optionally attach layout labels.

Stages and rules follow the reference (zig/pkg/inference/src/pipelines/multistage_ocr.zig:86-135 region
post-processing, :558-590 reading order and text assembly, :592 overlap; ctc_decode.zig:28 greedy CTC):

* detection gives a per-pixel text probability map; pixels above ``threshold`` are grouped into 8-connected
  components, a component survives if the mean probability inside its bounding rectangle reaches ``box_threshold``,
  and its box is grown by ``area * unclip_ratio / perimeter`` (the shrink the detectors are trained with) and scaled
  back to the page;
* regions are ordered top to bottom, left to right within a line (two regions share a line when their vertical
  centres differ by less than half the mean region height); texts on one line are joined by a space, lines by a
  newline;
* a layout region's label goes to the text regions it overlaps most (intersection over union).

The detector is any callable returning a probability map.  ``InkDensityDetector`` is a model-free one for clean
scans: dark pixels, smeared along the line with a max-pool so that words of a line merge, computed on the device
the page is on.  Recognisers: anything with ``read(images)`` (the ViT + TrOCR reader) or a CTC model through
:func:`ctc_greedy`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class TextRegion:
    bbox: Tuple[float, float, float, float]
    confidence: float = 0.0
    text: str = ""
    rec_confidence: float = 0.0
    label: Optional[str] = None


@dataclass
class LayoutRegion:
    bbox: Tuple[float, float, float, float]
    label: str
    confidence: float = 0.0
    order_idx: int = 0


@dataclass
class OcrResult:
    full_text: str
    regions: List[TextRegion]
    layout: List[LayoutRegion] = field(default_factory=list)


def connected_components(mask: np.ndarray, min_area: int = 1) -> List[Tuple[int, int, int, int, int]]:
    """8-connected components of a boolean image -> (min_x, min_y, max_x, max_y, area), in scan order of their first
    pixel.  Two-pass labelling with union-find over row runs."""
    h, w = mask.shape
    parent: List[int] = []

    def find(a: int) -> int:
        while parent[a] != a:
            parent[a] = parent[parent[a]]
            a = parent[a]
        return a

    runs: List[Tuple[int, int, int, int]] = []          # (row, x0, x1 inclusive, label)
    prev: List[Tuple[int, int, int]] = []
    for y in range(h):
        row = mask[y]
        edges = np.flatnonzero(np.diff(np.concatenate(([0], row.astype(np.int8), [0]))))
        cur: List[Tuple[int, int, int]] = []
        for x0, x1 in zip(edges[0::2].tolist(), (edges[1::2] - 1).tolist()):
            lab = -1
            for px0, px1, pl in prev:
                if px0 <= x1 + 1 and px1 >= x0 - 1:      # touches, diagonals included
                    r = find(pl)
                    if lab < 0:
                        lab = r
                    elif r != lab:
                        parent[max(r, lab)] = min(r, lab)
                        lab = min(r, lab)
            if lab < 0:
                lab = len(parent)
                parent.append(lab)
            cur.append((x0, x1, lab))
            runs.append((y, x0, x1, lab))
        prev = cur
    boxes = {}
    order = []
    for y, x0, x1, lab in runs:
        r = find(lab)
        if r not in boxes:
            boxes[r] = [x0, y, x1, y, 0]
            order.append(r)
        b = boxes[r]
        b[0], b[2], b[3], b[4] = min(b[0], x0), max(b[2], x1), max(b[3], y), b[4] + (x1 - x0 + 1)
    return [tuple(boxes[r]) for r in order if boxes[r][4] >= min_area]


@dataclass
class RegionPostProcessor:
    threshold: float = 0.3
    box_threshold: float = 0.6
    unclip_ratio: float = 1.5
    min_box_area: int = 10
    max_candidates: int = 1000

    def process(self, prob: torch.Tensor, page_width: int, page_height: int) -> List[TextRegion]:
        """Probability map [h, w] (any device) -> text regions in page coordinates."""
        p = prob.detach().float().cpu().numpy()
        h, w = p.shape
        sx, sy = page_width / w, page_height / h
        out: List[TextRegion] = []
        for i, (x0, y0, x1, y1, _) in enumerate(connected_components(p > self.threshold, self.min_box_area)):
            if i >= self.max_candidates:
                break
            score = float(p[y0:y1 + 1, x0:x1 + 1].mean())
            if score < self.box_threshold:
                continue
            bw, bh = (x1 - x0 + 1) * sx, (y1 - y0 + 1) * sy
            d = bw * bh * self.unclip_ratio / (2 * (bw + bh)) if bw + bh > 0 else 0.0
            clamp = lambda v, hi: float(min(max(v, 0.0), hi))
            out.append(TextRegion((clamp(x0 * sx - d, page_width), clamp(y0 * sy - d, page_height),
                                   clamp((x1 + 1) * sx + d, page_width), clamp((y1 + 1) * sy + d, page_height)), score))
        return out


def _tolerance(regions: Sequence) -> float:
    return 0.5 * sum(r.bbox[3] - r.bbox[1] for r in regions) / len(regions) if regions else 0.0


def sort_reading_order(regions: List) -> List:
    """Top to bottom; regions whose vertical centres are closer than half the mean height count as one line and go
    left to right.  (Lines are formed greedily from the top so that the order is a proper total order.)"""
    if len(regions) <= 1:
        return list(regions)
    tol = _tolerance(regions)
    yc = lambda r: (r.bbox[1] + r.bbox[3]) / 2
    rest = sorted(regions, key=yc)
    out: List = []
    while rest:
        top = yc(rest[0])
        line = [r for r in rest if abs(yc(r) - top) < tol]
        ids = {id(r) for r in line}
        out += sorted(line, key=lambda r: r.bbox[0])
        rest = [r for r in rest if id(r) not in ids]
    return out


def assemble_text(regions: Sequence[TextRegion]) -> str:
    if not regions:
        return ""
    tol = _tolerance(regions)
    yc = lambda r: (r.bbox[1] + r.bbox[3]) / 2
    parts = [regions[0].text]
    for prev, cur in zip(regions, regions[1:]):
        parts.append(" " if abs(yc(cur) - yc(prev)) < tol else "\n")
        parts.append(cur.text)
    return "".join(parts)


def overlap(a: Sequence[float], b: Sequence[float]) -> float:
    """Intersection over union of two boxes."""
    x1, y1, x2, y2 = max(a[0], b[0]), max(a[1], b[1]), min(a[2], b[2]), min(a[3], b[3])
    if x2 <= x1 or y2 <= y1:
        return 0.0
    inter = (x2 - x1) * (y2 - y1)
    union = (a[2] - a[0]) * (a[3] - a[1]) + (b[2] - b[0]) * (b[3] - b[1]) - inter
    return inter / union if union > 0 else 0.0


def attach_layout_labels(regions: Sequence[TextRegion], layout: Sequence[LayoutRegion], min_overlap: float = 0.0) -> None:
    """Each text region takes the label of the layout region that covers most of it (judged by the share of the
    text region's own area that lies inside)."""
    for r in regions:
        best, best_v = None, min_overlap
        area = max((r.bbox[2] - r.bbox[0]) * (r.bbox[3] - r.bbox[1]), 1e-9)
        for l in layout:
            w = min(r.bbox[2], l.bbox[2]) - max(r.bbox[0], l.bbox[0])
            h = min(r.bbox[3], l.bbox[3]) - max(r.bbox[1], l.bbox[1])
            v = w * h / area if w > 0 and h > 0 else 0.0
            if v > best_v:
                best, best_v = l, v
        if best is not None:
            r.label = best.label


def ctc_greedy(logits: torch.Tensor, charset: Sequence[str]) -> Tuple[str, float]:
    """[time, vocab] scores -> (text, confidence): arg-max per step, repeats collapsed, class 0 is the blank,
    class ``i`` is ``charset[i - 1]``; the confidence is the mean winning score of the kept steps."""
    if logits.numel() == 0:
        return "", 0.0
    val, idx = logits.float().max(-1)
    keep = (idx != 0) & (idx != torch.cat([idx.new_full((1,), -1), idx[:-1]]))
    if not bool(keep.any()):
        return "", 0.0
    chars = [charset[i - 1] for i in idx[keep].tolist() if i - 1 < len(charset)]
    return "".join(chars), float(val[keep].mean())


class InkDensityDetector:
    """Text probability without a model: darkness relative to the page background, spread sideways so that the
    letters and words of one line form one blob while lines stay apart.  For clean, upright scans."""

    def __init__(self, max_side: int = 1024, smear: float = 0.9, lift: float = 0.18):
        self.max_side, self.smear, self.lift = max_side, smear, lift

    def __call__(self, page: torch.Tensor) -> torch.Tensor:
        x = page.float().mean(-1)[None, None]                       # [1, 1, H, W] grey
        H, W = x.shape[-2:]
        s = min(1.0, self.max_side / max(H, W))
        if s < 1.0:
            x = torch.nn.functional.interpolate(x, size=(max(1, int(H * s)), max(1, int(W * s))), mode="area")
        bg = torch.quantile(x.flatten()[:: max(1, x.numel() // 65536)], 0.9)
        ink = ((bg - x) / bg.clamp(min=1.0)).clamp(0, 1)
        ink = (ink > self.lift).float()
        h = x.shape[-2]
        rows = ink.amax(-1).flatten()                               # rows that contain ink
        line_h = max(3, int(_median_run(rows)))                     # typical text height in pixels
        kw = max(3, int(line_h * self.smear * 2) | 1)
        kh = max(1, (line_h // 6) | 1)
        prob = torch.nn.functional.max_pool2d(ink, (kh, kw), stride=1, padding=(kh // 2, kw // 2))
        return prob[0, 0, :h]


def _median_run(flags: torch.Tensor) -> float:
    f = flags.cpu().numpy() > 0
    if not f.any():
        return 3.0
    e = np.flatnonzero(np.diff(np.concatenate(([0], f.astype(np.int8), [0]))))
    return float(np.median(e[1::2] - e[0::2]))


class MultiStageOCR:
    def __init__(self, recognizer, detector: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
                 post: Optional[RegionPostProcessor] = None,
                 layout: Optional[Callable[[torch.Tensor], List[LayoutRegion]]] = None, batch_size: int = 32):
        self.recognizer, self.detector = recognizer, detector or InkDensityDetector()
        self.post, self.layout, self.batch_size = post or RegionPostProcessor(), layout, batch_size

    def run(self, page: torch.Tensor, max_new_tokens: int = 64) -> OcrResult:
        """uint8 [H, W, 3] page -> regions with text in reading order, and the page text."""
        H, W = page.shape[0], page.shape[1]
        regions = sort_reading_order(self.post.process(self.detector(page), W, H))
        crops = []
        for r in regions:
            x0, y0, x1, y1 = (int(round(v)) for v in r.bbox)
            crops.append(page[max(0, y0):max(y0 + 1, y1), max(0, x0):max(x0 + 1, x1)])
        for lo in range(0, len(crops), self.batch_size):
            for r, res in zip(regions[lo:lo + self.batch_size], self.recognizer.read(crops[lo:lo + self.batch_size],
                                                                                     max_new_tokens)):
                r.text, r.rec_confidence = res.text.strip(), float(getattr(res, "confidence", 0.0) or 0.0)
        layout = self.layout(page) if self.layout is not None else []
        if layout:
            attach_layout_labels(regions, layout)
        kept = [r for r in regions if r.text]
        return OcrResult(assemble_text(kept), kept, layout)
