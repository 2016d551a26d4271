"""Florence-2: DaViT vision tower + image projector + BART encoder-decoder (OCR, captioning, detection prompts).

The reference runs this family natively from the original safetensors layout (``vision_tower.*``,
``image_projection``, ``image_proj_norm``, ``language_model.model.*``):
zig/pkg/inference/src/architectures/florence.zig:48-104 (encoder over image + prompt), :225-303 (vision tower),
:309-553 (DaViT blocks), :982-1030 (2-D and temporal position terms), :1037-1081 (feature sources);
config in zig/pkg/inference/src/models/florence.zig.  This module reads both that layout and the transformers
port's (``model.vision_tower.*``, ``model.multi_modal_projector.*``, ``model.language_model.*``).

DaViT stage = strided patch convolution (+ LayerNorm before or after), then blocks of
  spatial block: depthwise 3x3 (+x) -> LN -> attention inside 12 x 12 windows (+x) -> depthwise 3x3 (+x) -> LN -> MLP (+x)
  channel block: depthwise 3x3 (+x) -> LN -> attention between channel groups (+x) -> depthwise 3x3 (+x) -> LN -> MLP (+x)
Execution split: every token-wise linear / MLP is the shared bf16 GEMM with bias + GELU + residual epilogues, the
norms are the shared LayerNorm kernel, window attention runs every window as one sequence of the packed flash kernel,
the convolutions are cuDNN calls on channels-last views, channel-group attention (a [C/g, C/g] score per group) is
two batched matmuls.  The text half is :class:`antfly_b200.models.bart.BartModel`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops import attention as A
from ..ops import dense as Dn
from ..ops import reference as R
from .bart import BartConfig, BartModel


@dataclass
class DaViTConfig:
    in_channels: int = 3
    depths: Tuple[int, ...] = (1, 1, 9, 1)
    patch_size: Tuple[int, ...] = (7, 3, 3, 3)
    patch_stride: Tuple[int, ...] = (4, 2, 2, 2)
    patch_padding: Tuple[int, ...] = (3, 1, 1, 1)
    patch_prenorm: Tuple[bool, ...] = (False, True, True, True)
    embed_dim: Tuple[int, ...] = (128, 256, 512, 1024)
    num_heads: Tuple[int, ...] = (4, 8, 16, 32)
    num_groups: Tuple[int, ...] = (4, 8, 16, 32)
    window_size: int = 12
    mlp_ratio: float = 4.0
    projection_dim: int = 1024
    max_temporal_embeddings: int = 100
    max_position_embeddings: int = 50
    image_size: int = 768
    feature_sources: Tuple[str, ...] = ("spatial_avg_pool", "temporal_avg_pool")

    @classmethod
    def from_hf(cls, d: dict) -> "DaViTConfig":
        kw = {}
        alias = {"dim_embed": "embed_dim"}                 # the original checkpoints' name
        for k, v in d.items():
            k = alias.get(k, k)
            if k in cls.__dataclass_fields__:
                kw[k] = tuple(v) if isinstance(v, list) else v
        if "image_pos_embed" in d:
            kw["max_position_embeddings"] = int(d["image_pos_embed"].get("max_pos_embeddings", 50))
        if "visual_temporal_embedding" in d:
            kw["max_temporal_embeddings"] = int(d["visual_temporal_embedding"].get("max_temporal_embeddings", 100))
        if "image_feature_source" in d:
            kw["feature_sources"] = tuple(d["image_feature_source"])
        return cls(**kw)


def hf_names(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Tensor names of the original checkpoint layout -> the transformers port's names (a dict already in the
    port's layout is returned unchanged)."""
    if any(k.startswith("model.vision_tower.") for k in sd):
        return sd
    out: Dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        if k.startswith("vision_tower."):
            n = k.replace(".proj.", ".conv.") if ".convs." in k else k
            n = n.replace(".conv1.fn.dw.", ".conv1.").replace(".conv2.fn.dw.", ".conv2.")
            n = n.replace(".window_attn.norm.", ".norm1.").replace(".channel_attn.norm.", ".norm1.")
            n = n.replace(".window_attn.fn.", ".window_attn.").replace(".channel_attn.fn.", ".channel_attn.")
            n = n.replace(".ffn.norm.", ".norm2.").replace(".ffn.fn.net.", ".ffn.")
            out["model." + n] = v
        elif k == "image_projection":
            out["model.multi_modal_projector.image_projection.weight"] = v.t().contiguous()
        elif k.startswith("image_proj_norm."):
            out["model.multi_modal_projector." + k] = v
        elif k.startswith("image_pos_embed."):
            out["model.multi_modal_projector.image_position_embed." + k[len("image_pos_embed."):]] = v
        elif k.startswith("visual_temporal_embed."):
            out["model.multi_modal_projector." + k] = v
        elif k.startswith("language_model.model."):
            out["model.language_model." + k[len("language_model.model."):]] = v
        elif k == "language_model.final_logits_bias":
            out["final_logits_bias"] = v
        elif k == "language_model.lm_head.weight":
            out["lm_head.weight"] = v
        else:
            out[k] = v
    return out


def _sinusoid_table(n: int, dim: int) -> torch.Tensor:
    half = dim // 2
    freq = torch.exp(torch.arange(half).float() * -(math.log(10000) / half))
    ang = torch.arange(n).float()[:, None] * freq[None]
    t = torch.empty((n, dim))
    t[:, 0::2], t[:, 1::2] = torch.sin(ang), torch.cos(ang)
    return t


class DaViT:
    def __init__(self, cfg: DaViTConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device, self.dtype = weights["s0.conv.w"].device, weights["s0.conv.w"].dtype

    @classmethod
    def from_state_dict(cls, cfg: DaViTConfig, sd: Dict[str, torch.Tensor], prefix: str = "model.vision_tower.",
                        device="cuda", dtype=torch.bfloat16) -> "DaViT":
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}
        for s in range(len(cfg.embed_dim)):
            c = f"{prefix}convs.{s}."
            w[f"s{s}.conv.w"], w[f"s{s}.conv.b"] = t(sd[c + "conv.weight"]), t(sd[c + "conv.bias"])
            w[f"s{s}.norm.g"], w[f"s{s}.norm.b"] = t(sd[c + "norm.weight"]), t(sd[c + "norm.bias"])
            for b in range(cfg.depths[s]):
                for blk, attn in (("spatial_block", "window_attn"), ("channel_block", "channel_attn")):
                    src, dst = f"{prefix}blocks.{s}.{b}.{blk}.", f"s{s}.b{b}.{blk[0]}."
                    for n in ("conv1", "conv2"):
                        w[dst + n + ".w"], w[dst + n + ".b"] = t(sd[src + n + ".weight"]), t(sd[src + n + ".bias"])
                    for n in ("norm1", "norm2"):
                        w[dst + n + ".g"], w[dst + n + ".b"] = t(sd[src + n + ".weight"]), t(sd[src + n + ".bias"])
                    for n, key in (("qkv", attn + ".qkv"), ("proj", attn + ".proj"), ("fc1", "ffn.fc1"),
                                   ("fc2", "ffn.fc2")):
                        w[dst + n + ".w"], w[dst + n + ".b"] = t(sd[src + key + ".weight"]), t(sd[src + key + ".bias"])
        return cls(cfg, w)

    # -- pieces: activations are [B, H, W, C] ------------------------------------------------------------------
    def _conv(self, x: torch.Tensor, wt: torch.Tensor, b: torch.Tensor, stride: int, pad: int, groups: int = 1):
        y = F.conv2d(x.permute(0, 3, 1, 2), wt, b, stride=stride, padding=pad, groups=groups)
        return y.permute(0, 2, 3, 1).contiguous()

    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        shp = x.shape
        if not x.is_cuda:        # plain fp32 on the host (the shared op's host path rounds to bf16 like the kernel)
            return F.layer_norm(x, (shp[-1],), self.w[name + ".g"], self.w[name + ".b"], 1e-5)
        return Dn.norm(x.reshape(-1, shp[-1]).contiguous(), self.w[name + ".g"], self.w[name + ".b"], eps=1e-5).view(shp)

    def _lin(self, x: torch.Tensor, name: str, act: Optional[str] = None, residual: Optional[torch.Tensor] = None):
        shp = x.shape
        r = residual.reshape(-1, residual.shape[-1]).contiguous() if residual is not None else None
        y = Dn.gemm_bf16(x.reshape(-1, shp[-1]).contiguous(), self.w[name + ".w"], bias=self.w[name + ".b"], act=act,
                         residual=r, out_dtype=self.dtype)
        return y.view(*shp[:-1], -1)

    def _mlp(self, x: torch.Tensor, p: str) -> torch.Tensor:
        x = x + self._conv(x, self.w[p + "conv2.w"], self.w[p + "conv2.b"], 1, 1, groups=x.shape[-1])
        h = self._lin(self._ln(x, p + "norm2"), p + "fc1", act="gelu")
        return self._lin(h, p + "fc2", residual=x)

    def _window_attention(self, x: torch.Tensor, p: str, heads: int) -> torch.Tensor:
        """Attention inside non-overlapping ws x ws windows.  The map is zero-padded on the right / bottom to whole
        windows *after* the norm, so padded positions carry the bias of the qkv projection as keys, as in the
        original model."""
        B, H, W, C = x.shape
        ws = self.cfg.window_size
        ph, pw = (ws - H % ws) % ws, (ws - W % ws) % ws
        xp = F.pad(x, (0, 0, 0, pw, 0, ph))
        Hp, Wp = H + ph, W + pw
        win = xp.view(B, Hp // ws, ws, Wp // ws, ws, C).permute(0, 1, 3, 2, 4, 5).reshape(-1, ws * ws, C)
        nwin, L = win.shape[0], ws * ws
        D = C // heads
        qkv = self._lin(win, p + "qkv").view(nwin * L, 3, heads, D)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        starts = torch.arange(nwin, dtype=torch.int32, device=x.device) * L
        lens = torch.full((nwin,), L, dtype=torch.int32, device=x.device)
        if x.is_cuda:
            ctx = A.varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), starts, lens, L, causal=False)
        else:
            cu = torch.arange(nwin + 1, dtype=torch.int64) * L
            ctx = R.varlen_attention(q.float(), k.float(), v.float(), cu, D ** -0.5, False, 0).to(x.dtype)
        out = self._lin(ctx.reshape(nwin, L, C), p + "proj")
        out = out.view(B, Hp // ws, Wp // ws, ws, ws, C).permute(0, 1, 3, 2, 4, 5).reshape(B, Hp, Wp, C)
        return out[:, :H, :W, :]

    def _channel_attention(self, x: torch.Tensor, p: str, groups: int) -> torch.Tensor:
        """Every group of C/g channels attends over channels: scores are [C/g, C/g] contractions over the N tokens
        (scaled by N^-1/2), and the values are the channels' own token columns."""
        B, H, W, C = x.shape
        N, Cg = H * W, C // groups
        qkv = self._lin(x.view(B, N, C), p + "qkv").view(B, N, 3, groups, Cg).permute(2, 0, 3, 4, 1).float()
        q, k, v = qkv[0], qkv[1], qkv[2]                                         # [B, g, Cg, N]
        att = torch.softmax((q @ k.transpose(-1, -2)) * N ** -0.5, dim=-1)
        out = (att @ v).permute(0, 3, 1, 2).reshape(B, N, C).to(x.dtype)         # [B, N, g * Cg]
        return self._lin(out, p + "proj").view(B, H, W, C)

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """[B, 3, H, W] normalised pixels -> feature map [B, H', W', C_last]."""
        c, w = self.cfg, self.w
        x = pixel_values.to(self.device).to(self.dtype).permute(0, 2, 3, 1).contiguous()
        for s in range(len(c.embed_dim)):
            if c.patch_prenorm[s]:
                x = self._ln(x, f"s{s}.norm")
            x = self._conv(x, w[f"s{s}.conv.w"], w[f"s{s}.conv.b"], c.patch_stride[s], c.patch_padding[s])
            if not c.patch_prenorm[s]:
                x = self._ln(x, f"s{s}.norm")
            for b in range(c.depths[s]):
                p = f"s{s}.b{b}.s."
                x = x + self._conv(x, w[p + "conv1.w"], w[p + "conv1.b"], 1, 1, groups=x.shape[-1])
                x = x + self._window_attention(self._ln(x, p + "norm1"), p, c.num_heads[s])
                x = self._mlp(x, p)
                p = f"s{s}.b{b}.c."
                x = x + self._conv(x, w[p + "conv1.w"], w[p + "conv1.b"], 1, 1, groups=x.shape[-1])
                x = x + self._channel_attention(self._ln(x, p + "norm1"), p, c.num_groups[s])
                x = self._mlp(x, p)
        return x


class Florence2Model:
    """``encode(ids, pixel_values)`` / ``start_decoding`` / ``decode`` / ``generate``: the encoder-decoder interface
    of :class:`BartModel`, with image tokens in front of the prompt."""

    def __init__(self, vision_cfg: DaViTConfig, tower: DaViT, proj: Dict[str, torch.Tensor], text: BartModel,
                 image_token_id: int = 51289):
        self.vcfg, self.tower, self.p, self.text = vision_cfg, tower, proj, text
        self.cfg, self.device, self.image_token_id = text.cfg, text.device, image_token_id

    @classmethod
    def from_state_dict(cls, hf_config: dict, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "Florence2Model":
        sd = hf_names(sd)
        vcfg = DaViTConfig.from_hf(hf_config.get("vision_config") or {})
        tower = DaViT.from_state_dict(vcfg, sd, device=device, dtype=dtype)
        t = lambda x: x.to(dtype).to(device).contiguous()
        mp = "model.multi_modal_projector."
        proj = {"w": t(sd[mp + "image_projection.weight"]), "g": t(sd[mp + "image_proj_norm.weight"]),
                "b": t(sd[mp + "image_proj_norm.bias"]),
                "row": sd[mp + "image_position_embed.row_embeddings.weight"].float().to(device),
                "col": sd[mp + "image_position_embed.column_embeddings.weight"].float().to(device)}
        key = mp + "visual_temporal_embed.pos_idx_to_embed"
        proj["time"] = (sd[key].float() if key in sd else
                        _sinusoid_table(vcfg.max_temporal_embeddings, vcfg.embed_dim[-1])).to(device)
        tcfg = BartConfig.from_hf(hf_config.get("text_config") or {})
        text_sd = {"model." + k[len("model.language_model."):]: v for k, v in sd.items()
                   if k.startswith("model.language_model.")}
        if "final_logits_bias" in sd:
            text_sd["final_logits_bias"] = sd["final_logits_bias"]
        text = BartModel.from_state_dict(tcfg, text_sd, device=device, dtype=dtype)
        return cls(vcfg, tower, proj, text, int(hf_config.get("image_token_id", 51289)))

    def image_tokens(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """[B, 3, H, W] -> [B, n, d_model]: the feature map plus a learned (column | row) position term and the first
        temporal term, then the configured feature sources (mean over positions, the positions themselves) in
        sequence, projected and normalised."""
        p = self.p
        f = self.tower.forward(pixel_values).float()                               # [B, H, W, C]
        B, H, W, C = f.shape
        pos = torch.cat([p["col"][:W][None].expand(H, W, -1), p["row"][:H][:, None].expand(H, W, -1)], -1)
        tok = (f + pos[None]).view(B, H * W, C) + p["time"][0]
        parts = []
        for src in self.vcfg.feature_sources:
            if src == "spatial_avg_pool":
                parts.append(tok.mean(1, keepdim=True))
            elif src in ("temporal_avg_pool", "last_frame"):          # one frame: both are the frame's own tokens
                parts.append(tok)
            else:
                raise ValueError(f"unknown image feature source {src!r}")
        x = torch.cat(parts, 1)
        n = x.shape[1]
        dt = p["w"].dtype
        y = Dn.gemm_bf16(x.reshape(B * n, C).to(dt).contiguous(), p["w"], out_dtype=dt)
        if not y.is_cuda:
            return F.layer_norm(y, (y.shape[-1],), p["g"], p["b"], 1e-5).view(B, n, -1)
        return Dn.norm(y, p["g"], p["b"], eps=1e-5).view(B, n, -1)

    def encode(self, ids: Sequence[int], pixel_values: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Prompt ids (image placeholder tokens, if any, are dropped: the image tokens always lead) + one image
        [3, H, W] -> encoder states [n_image + n_prompt, d_model]."""
        text = self.text
        ids = [t for t in ids if t != self.image_token_id]
        tok = text.w["shared"].index_select(0, torch.tensor(ids, device=self.device)).float() * text.scale
        if pixel_values is not None:
            px = pixel_values if pixel_values.dim() == 4 else pixel_values[None]
            tok = torch.cat([self.image_tokens(px)[0].float(), tok], 0)
        return text.encode(None, token_embeds=tok)

    def start_decoding(self, enc: torch.Tensor) -> dict:
        return self.text.start_decoding(enc)

    def decode(self, state: dict, ids: Sequence[int]) -> torch.Tensor:
        return self.text.decode(state, ids)

    def generate(self, ids: Sequence[int], pixel_values: Optional[torch.Tensor] = None, max_new_tokens: int = 64,
                 no_repeat_ngram_size: int = 0) -> List[int]:
        """Greedy decoding; ``no_repeat_ngram_size`` > 0 masks every token that would complete an n-gram already in
        the output (the reference reader's guard against OCR loops: pipelines/reading.zig selectGreedyToken)."""
        cfg = self.cfg
        state = self.start_decoding(self.encode(ids, pixel_values))
        prefix = [cfg.decoder_start_token_id] + ([cfg.forced_bos_token_id] if cfg.forced_bos_token_id >= 0 else [])
        logits = self.decode(state, prefix)[-1]
        out: List[int] = []
        hist = list(prefix)
        for _ in range(max_new_tokens):
            if no_repeat_ngram_size > 0:
                logits = logits.clone()
                for t in banned_next_tokens(hist, no_repeat_ngram_size):
                    logits[t] = float("-inf")
            tok = int(logits.argmax())
            if tok == cfg.eos_token_id:
                break
            out.append(tok)
            hist.append(tok)
            logits = self.decode(state, [tok])[-1]
        return out


def banned_next_tokens(history: Sequence[int], n: int) -> List[int]:
    """Tokens that would repeat an n-gram of ``history`` if appended to it."""
    if n <= 0 or len(history) + 1 < n:
        return []
    tail = tuple(history[len(history) - (n - 1):]) if n > 1 else ()
    out = []
    for i in range(len(history) - n + 1):
        if tuple(history[i:i + n - 1]) == tail:
            out.append(history[i + n - 1])
    return out


FLORENCE_TASK_PROMPTS = {
    "<OCR>": "What is the text in the image?",
    "<OCR_WITH_REGION>": "What is the text in the image, with regions?",
    "<CAPTION>": "What does the image describe?",
    "<DETAILED_CAPTION>": "Describe in detail what is shown in the image.",
    "<MORE_DETAILED_CAPTION>": "Describe with a paragraph what is shown in the image.",
    "<OD>": "Locate the objects with category name in the image.",
    "<DENSE_REGION_CAPTION>": "Locate the objects in the image, with their descriptions.",
    "<REGION_PROPOSAL>": "Locate the region proposals in the image.",
}
