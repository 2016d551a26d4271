"""Image inputs for generation: the adapter between a chat prompt with image parts and the decoder engine.

A prompt reaches the adapter tokenised, with ONE placeholder token per image (what the chat template writes between
the vision start / end markers).  The adapter decodes and patches each image, runs the vision tower, widens every
placeholder to as many tokens as the image has merged patches, and describes the result to the engine: which prompt
positions take a given embedding instead of a table row, and the three rotary position streams of the prompt.  The
reference's adapter does the same around its Qwen2-VL session (zig/pkg/inference/src/pipelines/vlm_qwen2vl.zig); as
there, prompts with images do not use speculative decoding or the prefix cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..models import qwen2vl as QV
from .multimodal import ImageLike, load_image


@dataclass
class VlmTokens:
    image: int                       # <|image_pad|>
    vision_start: Optional[int] = None
    vision_end: Optional[int] = None


class Qwen2VLAdapter:
    placeholder = "<|vision_start|><|image_pad|><|vision_end|>"

    def __init__(self, vision: QV.Qwen2VLVisionModel, tokens: VlmTokens, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280):
        self.vision, self.tokens = vision, tokens
        self.min_pixels, self.max_pixels = min_pixels, max_pixels

    def encode_images(self, images: Sequence[ImageLike]):
        """-> (soft tokens [sum of merged patches, hidden], patch grid of each image)."""
        patches, grids = [], []
        for src in images:
            p, g = QV.image_to_patches(load_image(src).cpu(), self.vision.cfg, self.min_pixels, self.max_pixels)
            patches.append(p)
            grids.append(g)
        soft = self.vision.forward(torch.cat(patches, 0), grids)
        return soft, grids

    def expand(self, ids: Sequence[int], images: Sequence[ImageLike]) -> Tuple[List[int], Optional[dict]]:
        """Prompt ids with one placeholder per image -> (ids with each placeholder repeated once per merged patch,
        the engine's description of the soft tokens).  Without images the prompt is returned unchanged."""
        n_ph = sum(1 for t in ids if t == self.tokens.image)
        if not images:
            if n_ph:
                raise ValueError("the prompt has image placeholders but no images were given")
            return list(ids), None
        if n_ph != len(images):
            raise ValueError(f"{len(images)} image(s) for {n_ph} placeholder(s) in the prompt")
        soft, grids = self.encode_images(images)
        m = self.vision.cfg.spatial_merge_size
        out: List[int] = []
        g = 0
        for t in ids:
            if t == self.tokens.image:
                tt, h, w = grids[g]
                out += [t] * (tt * (h // m) * (w // m))
                g += 1
            else:
                out.append(t)
        rows = [i for i, t in enumerate(out) if t == self.tokens.image]
        pos3, delta = QV.rope_index(out, grids, self.tokens.image, m)
        return out, {"rows": rows, "vals": soft, "pos3": pos3, "delta": delta}


def split_content(messages: Sequence[dict]) -> List[ImageLike]:
    """The images of a chat request, in reading order: content parts of type ``image_url`` (``{"url": data-URL}`` or a
    bare string) and ``image`` (a data URL, a path, or a decoded array)."""
    from .multimodal import decode_data_url

    found: List[ImageLike] = []
    for m in messages:
        c = m.get("content")
        if not isinstance(c, list):
            continue
        for p in c:
            if not isinstance(p, dict) or p.get("type") not in ("image_url", "image"):
                continue
            v = p.get("image_url") if p.get("type") == "image_url" else p.get("image", p.get("url"))
            if isinstance(v, dict):
                v = v.get("url")
            found.append(decode_data_url(v) if isinstance(v, str) and v.startswith("data:") else v)
    return found


class Gemma3Adapter:
    """Gemma-3 images: every ``<start_of_image>`` in the prompt becomes a blank line, the begin marker, 256 soft
    tokens, the end marker and another blank line; the soft tokens of one image attend to one another in both
    directions, so the engine prefills such a prompt in one piece (zig/pkg/inference/src/pipelines/vlm_gemma3.zig)."""

    placeholder = "<start_of_image>"

    def __init__(self, vision, image_token: int, boi_token: int, eoi_token: int, newline_ids: Sequence[int] = ()):
        self.vision, self.image, self.boi, self.eoi = vision, image_token, boi_token, eoi_token
        self.newline_ids = list(newline_ids)

    def expand(self, ids: Sequence[int], images: Sequence[ImageLike]) -> Tuple[List[int], Optional[dict]]:
        from ..models.gemma3v import gemma3_pixels

        n_ph = sum(1 for t in ids if t == self.boi)
        if not images:
            if n_ph:
                raise ValueError("the prompt has image placeholders but no images were given")
            return list(ids), None
        if n_ph != len(images):
            raise ValueError(f"{len(images)} image(s) for {n_ph} placeholder(s) in the prompt")
        size = self.vision.cfg.image_size
        px = torch.stack([gemma3_pixels(load_image(s).cpu(), size) for s in images])
        soft = self.vision.soft_tokens(px)                                   # [images, tokens, hidden]
        n_tok = soft.shape[1]
        out: List[int] = []
        spans = []
        for t in ids:
            if t == self.boi:
                out += self.newline_ids + [self.boi]
                spans.append((len(out), len(out) + n_tok))
                out += [self.image] * n_tok + [self.eoi] + self.newline_ids
            else:
                out.append(t)
        rows = [i for a, b in spans for i in range(a, b)]
        return out, {"rows": rows, "vals": soft.reshape(-1, soft.shape[-1]), "bidir": spans}


class ColQwenEmbedder:
    """Late-interaction retrieval over page images (ColQwen2): a query or an image is run through the Qwen2-VL
    decoder, every token's final hidden state is projected to a small vector and L2-normalised, and a query is
    scored against a page by summing, over the query's tokens, the best dot product with any of the page's tokens
    (the MaxSim kernel).  The reference's multimodal reranker does the same
    (zig/pkg/inference/src/pipelines/multimodal_reranker_colqwen_impl.zig)."""

    def __init__(self, model, adapter: Qwen2VLAdapter, proj_w: torch.Tensor, proj_b: Optional[torch.Tensor],
                 tokenizer=None, page: int = 16):
        self.model, self.adapter, self.tokenizer, self.page = model, adapter, tokenizer, page
        self.proj_w, self.proj_b = proj_w, proj_b

    @property
    def dim(self) -> int:
        return self.proj_w.shape[0]

    def _hidden(self, ids: Sequence[int], soft: Optional[dict]) -> torch.Tensor:
        from ..models.llama import StepBatch

        m, dev, page = self.model, self.model.device, self.page
        n = len(ids)
        nblk = (n + page - 1) // page
        kc = torch.zeros((m.n_layers, nblk, page, m.Hkv, m.D), dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        idx = torch.arange(n, dtype=torch.int32, device=dev)
        b = StepBatch(i32(list(ids)), idx, idx.clone(), i32([0]), i32([n]), i32([n]),
                      torch.arange(nblk, dtype=torch.int32, device=dev)[None], idx.clone(), n, 1)
        if soft is not None:
            b.embed_rows = torch.tensor(soft["rows"], dtype=torch.int64, device=dev)
            b.embed_vals, b.pos3 = soft["vals"].to(dev), soft["pos3"].to(dev)
        prev, m.return_hidden = m.return_hidden, True
        try:
            return m.forward(b, kc, vc)
        finally:
            m.return_hidden = prev

    def _project(self, h: torch.Tensor) -> torch.Tensor:
        from ..ops import dense as Dn

        e = Dn.gemm_bf16(h.to(self.proj_w.dtype).contiguous(), self.proj_w, bias=self.proj_b,
                         out_dtype=torch.float32).float()
        return torch.nn.functional.normalize(e, dim=-1)

    def embed_ids(self, ids: Sequence[int], images: Sequence[ImageLike] = ()) -> torch.Tensor:
        """Prompt ids (one image placeholder per image) -> [tokens, dim] unit vectors."""
        full, soft = self.adapter.expand(ids, list(images))
        return self._project(self._hidden(full, soft))

    def score(self, query: torch.Tensor, pages: Sequence[torch.Tensor]) -> List[float]:
        """MaxSim of one query's token vectors against each page's."""
        from ..ops import dense as Dn

        if not pages:
            return []
        lens = torch.tensor([p.shape[0] for p in pages], dtype=torch.int32)
        starts = (torch.cumsum(lens, 0) - lens).to(torch.int32)
        dev = query.device
        d = torch.cat(list(pages), 0).to(dev)
        return Dn.maxsim(query.to(torch.bfloat16).contiguous(), d.to(torch.bfloat16).contiguous(), starts.to(dev),
                         lens.to(dev)).float().cpu().tolist()

    # query / page prompts as the retrieval checkpoints were trained: the page is one image followed by a fixed
    # instruction, the query is the text followed by a few padding-like suffix tokens
    page_prompt = "<|im_start|>user\n<|vision_start|><|image_pad|><|vision_end|>Describe the image.<|im_end|><|endoftext|>"
    query_prefix, query_suffix = "Query: ", "<|endoftext|>" * 10

    def rerank_pages(self, query: str, docs: Sequence[Tuple[Sequence[str], Sequence[ImageLike]]]):
        """``docs`` = (texts, images) per document -> (one score per document: the best MaxSim over its parts,
        prompt tokens spent)."""
        if self.tokenizer is None:
            raise RuntimeError("this model has no tokenizer")
        enc = lambda t: list(self.tokenizer.encode_prompt(t, add_bos=False))
        q_ids = enc(self.query_prefix + query + self.query_suffix)
        qv = self.embed_ids(q_ids)
        ntok, parts, owner = len(q_ids), [], []
        for i, (texts, images) in enumerate(docs):
            for t in texts:
                ids = enc(self.query_prefix + t + self.query_suffix)
                ntok += len(ids)
                parts.append(self.embed_ids(ids)); owner.append(i)
            for im in images:
                v = self.embed_ids(enc(self.page_prompt), [im])
                ntok += v.shape[0]
                parts.append(v); owner.append(i)
        raw = self.score(qv, parts)
        scores = [float("-inf")] * len(docs)
        for s_, i in zip(raw, owner):
            scores[i] = max(scores[i], s_)
        return [0.0 if s_ == float("-inf") else s_ for s_ in scores], ntok
