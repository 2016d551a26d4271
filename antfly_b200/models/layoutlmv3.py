"""LayoutLMv3: a document encoder over word tokens with their page boxes and the page image's patches.

A document is the concatenation of its text tokens (word + RoBERTa position + token type + box embeddings, where a
box contributes x0 / y0 / x1 / y1 / height / width lookups laid side by side) and the image tokens (a class token
plus 16 x 16 patches with learned positions); one post-LayerNorm transformer runs over both.  Attention scores get
two learned biases: one over bucketed token distance, one over bucketed distance between the boxes' left edges and
between their bottom edges (patches carry the box of their grid cell).  Heads: token classification over the text
tokens (linear, or dense-tanh-linear for ten or more labels), sequence classification on the first token.

The reference runs the same model for layout-aware extraction (zig/pkg/inference/src/architectures/layoutlmv3.zig,
zig/pkg/inference/src/models/layoutlmv3.zig).  Projections and MLPs run on the bf16 GEMM with bias / GELU /
residual epilogues and LayerNorms on the norm kernel, over all documents of a batch packed together; the attention
with its per-document additive bias is batched tensor arithmetic.  Weight names are the Hugging Face ones.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import dense as Dn


@dataclass
class LayoutLMv3Config:
    vocab_size: int = 50265
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 514
    type_vocab_size: int = 1
    layer_norm_eps: float = 1e-5
    pad_token_id: int = 1
    max_2d_position_embeddings: int = 1024
    coordinate_size: int = 128
    shape_size: int = 128
    has_relative_attention_bias: bool = True
    rel_pos_bins: int = 32
    max_rel_pos: int = 128
    has_spatial_attention_bias: bool = True
    rel_2d_pos_bins: int = 64
    max_rel_2d_pos: int = 256
    visual_embed: bool = True
    input_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    hidden_act: str = "gelu"
    num_labels: int = 0

    @classmethod
    def from_hf(cls, d: dict) -> "LayoutLMv3Config":
        c = cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None})
        if "id2label" in d and not d.get("num_labels"):
            c.num_labels = len(d["id2label"])
        return c


def distance_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Signed distance -> bucket: half of the buckets per direction; within a direction the first half is one
    bucket per unit, the rest grow logarithmically up to ``max_distance``."""
    nb = num_buckets // 2
    ret = (rel > 0).long() * nb
    n = rel.abs()
    exact = nb // 2
    large = exact + (torch.log(n.float().clamp(min=1) / exact) / math.log(max_distance / exact) * (nb - exact)).long()
    large = large.clamp(max=nb - 1)
    return ret + torch.where(n < exact, n, large)


@dataclass
class Document:
    ids: Sequence[int]                          # text tokens, with <s> ... </s>
    boxes: Sequence[Sequence[int]]              # one (x0, y0, x1, y1) per token, page coordinates scaled to 0..1000
    pixels: Optional[torch.Tensor] = None       # [3, S, S] normalised page image, or None for text + layout only


class LayoutLMv3Model:
    def __init__(self, cfg: LayoutLMv3Config, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["emb.word"].device

    @classmethod
    def from_state_dict(cls, cfg: LayoutLMv3Config, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "LayoutLMv3Model":
        pre = "layoutlmv3." if any(k.startswith("layoutlmv3.") for k in sd) else ""
        t = lambda x: x.to(dtype).to(device).contiguous()
        f32 = lambda x: x.float().to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}
        e = pre + "embeddings."
        for dst, src in (("word", "word_embeddings"), ("pos", "position_embeddings"), ("type", "token_type_embeddings"),
                         ("x", "x_position_embeddings"), ("y", "y_position_embeddings"),
                         ("h", "h_position_embeddings"), ("w", "w_position_embeddings")):
            w["emb." + dst] = f32(sd[e + src + ".weight"])
        w["emb.ln.g"], w["emb.ln.b"] = t(sd[e + "LayerNorm.weight"]), t(sd[e + "LayerNorm.bias"])
        if cfg.visual_embed:
            w["vis.patch.w"] = t(sd[pre + "patch_embed.proj.weight"].flatten(1))
            w["vis.patch.b"] = t(sd[pre + "patch_embed.proj.bias"])
            w["vis.cls"], w["vis.pos"] = f32(sd[pre + "cls_token"][0]), f32(sd[pre + "pos_embed"][0])
            w["vis.norm.g"], w["vis.norm.b"] = t(sd[pre + "norm.weight"]), t(sd[pre + "norm.bias"])
            w["vis.ln.g"], w["vis.ln.b"] = t(sd[pre + "LayerNorm.weight"]), t(sd[pre + "LayerNorm.bias"])
        if cfg.has_relative_attention_bias:
            w["rel.pos"] = f32(sd[pre + "encoder.rel_pos_bias.weight"])           # [heads, bins]
        if cfg.has_spatial_attention_bias:
            w["rel.x"], w["rel.y"] = f32(sd[pre + "encoder.rel_pos_x_bias.weight"]), f32(
                sd[pre + "encoder.rel_pos_y_bias.weight"])
        for l in range(cfg.num_hidden_layers):
            s, p = pre + f"encoder.layer.{l}.", f"l{l}."
            w[p + "qkv.w"] = t(torch.cat([sd[s + f"attention.self.{n}.weight"] for n in ("query", "key", "value")], 0))
            w[p + "qkv.b"] = t(torch.cat([sd[s + f"attention.self.{n}.bias"] for n in ("query", "key", "value")], 0))
            w[p + "o.w"], w[p + "o.b"] = t(sd[s + "attention.output.dense.weight"]), t(sd[s + "attention.output.dense.bias"])
            w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "attention.output.LayerNorm.weight"]), t(
                sd[s + "attention.output.LayerNorm.bias"])
            w[p + "ff1.w"], w[p + "ff1.b"] = t(sd[s + "intermediate.dense.weight"]), t(sd[s + "intermediate.dense.bias"])
            w[p + "ff2.w"], w[p + "ff2.b"] = t(sd[s + "output.dense.weight"]), t(sd[s + "output.dense.bias"])
            w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "output.LayerNorm.weight"]), t(sd[s + "output.LayerNorm.bias"])
        if "classifier.weight" in sd:
            w["cls.w"], w["cls.b"] = t(sd["classifier.weight"]), t(sd["classifier.bias"])
            cfg.num_labels = w["cls.w"].shape[0]
        elif "classifier.out_proj.weight" in sd:
            w["cls.dense.w"], w["cls.dense.b"] = t(sd["classifier.dense.weight"]), t(sd["classifier.dense.bias"])
            w["cls.w"], w["cls.b"] = t(sd["classifier.out_proj.weight"]), t(sd["classifier.out_proj.bias"])
            cfg.num_labels = w["cls.w"].shape[0]
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def _patch_boxes(self, g: int) -> torch.Tensor:
        """Boxes of the class token and of the g x g patch cells on the 0..1000 page scale."""
        edge = torch.div(torch.arange(0, 1000 * (g + 1), 1000), g, rounding_mode="trunc")
        x0, x1 = edge[:-1].repeat(g, 1), edge[1:].repeat(g, 1)
        y0, y1 = edge[:-1].repeat(g, 1).T, edge[1:].repeat(g, 1).T
        cells = torch.stack([x0, y0, x1, y1], -1).view(-1, 4)
        return torch.cat([torch.tensor([[1, 1, 999, 999]]), cells], 0)

    def _embed(self, doc: Document) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """One document -> (token states [L, H] fp32 before the encoder, boxes [L, 4], positions [L])."""
        c, w, dev = self.cfg, self.w, self.device
        ids = torch.tensor(list(doc.ids), dtype=torch.long, device=dev)
        box = torch.tensor([list(b) for b in doc.boxes], dtype=torch.long, device=dev).view(-1, 4)
        if box.shape[0] != ids.numel():
            raise ValueError("one box per token is required")
        if int(box.min()) < 0 or int(box.max()) >= c.max_2d_position_embeddings:
            raise ValueError("box coordinates must lie in 0..1000")
        keep = (ids != c.pad_token_id).long()
        pos = torch.cumsum(keep, 0) * keep + c.pad_token_id
        x = w["emb.word"][ids] + w["emb.type"][torch.zeros_like(ids)] + w["emb.pos"][pos]
        hh = (box[:, 3] - box[:, 1]).clamp(0, 1023)
        ww = (box[:, 2] - box[:, 0]).clamp(0, 1023)
        x = x + torch.cat([w["emb.x"][box[:, 0]], w["emb.y"][box[:, 1]], w["emb.x"][box[:, 2]], w["emb.y"][box[:, 3]],
                           w["emb.h"][hh], w["emb.w"][ww]], -1)
        x = Dn.norm(x.to(w["emb.ln.g"].dtype), w["emb.ln.g"], w["emb.ln.b"], eps=c.layer_norm_eps).float()
        positions = torch.arange(ids.numel(), device=dev)
        if doc.pixels is not None and c.visual_embed:
            P = c.patch_size
            px = doc.pixels.to(dev)
            C, S, _ = px.shape
            g = S // P
            if g * g + 1 != w["vis.pos"].shape[0]:
                raise ValueError(f"page image must be {c.input_size} x {c.input_size}")
            dt = w["vis.patch.w"].dtype
            cols = px.to(dt).view(C, g, P, g, P).permute(1, 3, 0, 2, 4).reshape(g * g, C * P * P).contiguous()
            v = Dn.gemm_bf16(cols, w["vis.patch.w"], bias=w["vis.patch.b"]).float()
            v = torch.cat([w["vis.cls"], v], 0) + w["vis.pos"]
            v = Dn.norm(v.to(dt), w["vis.norm.g"], w["vis.norm.b"], eps=1e-6).float()
            x = torch.cat([x, v], 0)
            x = Dn.norm(x.to(dt), w["vis.ln.g"], w["vis.ln.b"], eps=c.layer_norm_eps).float()
            box = torch.cat([box, self._patch_boxes(g).to(dev)], 0)
            positions = torch.cat([positions, torch.arange(g * g + 1, device=dev)])
        return x, box, positions

    def _bias(self, box: torch.Tensor, positions: torch.Tensor) -> Optional[torch.Tensor]:
        """[heads, L, L] additive attention bias of one document (already divided by sqrt(head_dim))."""
        c, w = self.cfg, self.w
        out = None
        if c.has_relative_attention_bias:
            b = distance_bucket(positions[None, :] - positions[:, None], c.rel_pos_bins, c.max_rel_pos)
            out = w["rel.pos"].T[b].permute(2, 0, 1)
        if c.has_spatial_attention_bias:
            bx = distance_bucket(box[None, :, 0] - box[:, None, 0], c.rel_2d_pos_bins, c.max_rel_2d_pos)
            by = distance_bucket(box[None, :, 3] - box[:, None, 3], c.rel_2d_pos_bins, c.max_rel_2d_pos)
            sp = w["rel.x"].T[bx].permute(2, 0, 1) + w["rel.y"].T[by].permute(2, 0, 1)
            out = sp if out is None else out + sp
        if out is None:
            return None
        return out / math.sqrt(c.hidden_size // c.num_attention_heads)

    def encode(self, docs: Sequence[Document]) -> List[torch.Tensor]:
        """Final hidden states of every document: one [L_i, H] tensor each (text tokens first, then the image's)."""
        c, w = self.cfg, self.w
        H, nh = c.hidden_size, c.num_attention_heads
        D = H // nh
        parts = [self._embed(d) for d in docs]
        lens = [p[0].shape[0] for p in parts]
        biases = [self._bias(p[1], p[2]) for p in parts]
        dt = w["l0.qkv.w"].dtype
        x = torch.cat([p[0] for p in parts], 0).to(dt).contiguous()
        T = x.shape[0]
        for l in range(c.num_hidden_layers):
            p = f"l{l}."
            qkv = Dn.gemm_bf16(x, w[p + "qkv.w"], bias=w[p + "qkv.b"]).float().view(T, 3, nh, D)
            ctx = torch.empty((T, nh, D), dtype=torch.float32, device=x.device)
            o = 0
            for n, bias in zip(lens, biases):
                q, k, v = (qkv[o:o + n, i].transpose(0, 1) for i in range(3))          # [nh, n, D]
                s = (q / math.sqrt(D)) @ k.transpose(-1, -2)
                if bias is not None:
                    s = s + bias
                ctx[o:o + n] = (torch.softmax(s, -1) @ v).transpose(0, 1)
                o += n
            h = Dn.gemm_bf16(ctx.view(T, H).to(dt), w[p + "o.w"], bias=w[p + "o.b"], residual=x)
            x = Dn.norm(h, w[p + "ln1.g"], w[p + "ln1.b"], eps=c.layer_norm_eps)
            f = Dn.gemm_bf16(x, w[p + "ff1.w"], bias=w[p + "ff1.b"], act=c.hidden_act)
            h = Dn.gemm_bf16(f, w[p + "ff2.w"], bias=w[p + "ff2.b"], residual=x)
            x = Dn.norm(h, w[p + "ln2.g"], w[p + "ln2.b"], eps=c.layer_norm_eps)
        return list(torch.split(x, lens, 0))

    def token_logits(self, docs: Sequence[Document]) -> List[torch.Tensor]:
        """Per document, fp32 [text tokens, num_labels]."""
        w = self.w
        if "cls.w" not in w:
            raise ValueError("this checkpoint has no classification head")
        out = []
        for d, h in zip(docs, self.encode(docs)):
            t = h[: len(d.ids)].contiguous()
            if "cls.dense.w" in w:
                t = torch.tanh(Dn.gemm_bf16(t, w["cls.dense.w"], bias=w["cls.dense.b"], out_dtype=torch.float32).float())
                t = t.to(w["cls.w"].dtype).contiguous()
            out.append(Dn.gemm_bf16(t, w["cls.w"], bias=w["cls.b"], out_dtype=torch.float32).float())
        return out

    def sequence_logits(self, docs: Sequence[Document]) -> torch.Tensor:
        """Document-level classification: the head (dense, tanh, projection) on each document's first token ->
        fp32 [documents, num_labels] (zig/pkg/inference/src/pipelines/document_classification.zig)."""
        w = self.w
        if "cls.dense.w" not in w:
            raise ValueError("this checkpoint has no document classification head")
        first = torch.stack([h[0] for h in self.encode(docs)]).contiguous()
        t = torch.tanh(Dn.gemm_bf16(first, w["cls.dense.w"], bias=w["cls.dense.b"], out_dtype=torch.float32).float())
        return Dn.gemm_bf16(t.to(w["cls.w"].dtype).contiguous(), w["cls.w"], bias=w["cls.b"],
                            out_dtype=torch.float32).float()
