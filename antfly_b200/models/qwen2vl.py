"""Qwen2-VL: a vision transformer that turns image patches into soft tokens of the Qwen2 decoder, and the
three-stream rotary positions (time, row, column) those tokens carry inside the decoder.

Vision tower (zig/pkg/inference/src/architectures/qwen2vl_vision.zig): patches of ``2 x 14 x 14`` pixels (a still
image is repeated along time) are embedded by one GEMM; every block is pre-LayerNorm attention + MLP where
attention is bidirectional within one frame and rotates Q / K by the patch's row and column (half of the rotary
pairs each); a merger LayerNorms the patch states, concatenates each ``2 x 2`` neighbourhood (patches arrive
grouped that way) and projects it to the decoder width with a two-layer GELU MLP.  GEMMs, LayerNorms and the packed
variable-length attention are the same kernels the text encoders use; the 2-D rotation is elementwise tensor
arithmetic on the fused QKV buffer.

Decoder side: an image occupies ``rows / 2 * cols / 2`` placeholder tokens whose rotary position is (t, row, col)
offset by the position of the text before it; text after the image continues from the largest position used so
far, so rotary positions run behind the cache index by a per-request delta.  ``rope_index`` computes the three
streams for a prompt; :func:`mrope_rotate` applies them (sections of the rotary pairs take their angle from the
time, row or column stream).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import attention as A
from ..ops import dense as Dn


@dataclass
class Qwen2VLVisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584           # decoder width (output of the merger)
    num_heads: int = 16
    mlp_ratio: float = 4.0
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    hidden_act: str = "quick_gelu"

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen2VLVisionConfig":
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None})


def _act(x: torch.Tensor, name: str) -> torch.Tensor:
    xf = x.float()
    if name == "quick_gelu":
        return (xf * torch.sigmoid(1.702 * xf)).to(x.dtype)
    if name in ("gelu", "gelu_pytorch_tanh"):
        return torch.nn.functional.gelu(xf, approximate="tanh" if name.endswith("tanh") else "none").to(x.dtype)
    if name == "silu":
        return torch.nn.functional.silu(xf).to(x.dtype)
    raise ValueError(name)


class Qwen2VLVisionModel:
    def __init__(self, cfg: Qwen2VLVisionConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["patch.w"].device

    @classmethod
    def from_state_dict(cls, cfg: Qwen2VLVisionConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16, prefix: Optional[str] = None) -> "Qwen2VLVisionModel":
        if prefix is None:
            prefix = next((p for p in ("model.visual.", "visual.", "") if p + "patch_embed.proj.weight" in sd), None)
            if prefix is None:
                raise KeyError("patch_embed.proj.weight")
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {"patch.w": t(sd[prefix + "patch_embed.proj.weight"].flatten(1))}
        for l in range(cfg.depth):
            s, p = prefix + f"blocks.{l}.", f"l{l}."
            for n in ("norm1", "norm2"):
                w[p + n + ".g"], w[p + n + ".b"] = t(sd[s + n + ".weight"]), t(sd[s + n + ".bias"])
            w[p + "qkv.w"], w[p + "qkv.b"] = t(sd[s + "attn.qkv.weight"]), t(sd[s + "attn.qkv.bias"])
            w[p + "o.w"], w[p + "o.b"] = t(sd[s + "attn.proj.weight"]), t(sd[s + "attn.proj.bias"])
            w[p + "fc1.w"], w[p + "fc1.b"] = t(sd[s + "mlp.fc1.weight"]), t(sd[s + "mlp.fc1.bias"])
            w[p + "fc2.w"], w[p + "fc2.b"] = t(sd[s + "mlp.fc2.weight"]), t(sd[s + "mlp.fc2.bias"])
        m = prefix + "merger."
        w["merge.ln.g"], w["merge.ln.b"] = t(sd[m + "ln_q.weight"]), t(sd[m + "ln_q.bias"])
        w["merge.fc1.w"], w["merge.fc1.b"] = t(sd[m + "mlp.0.weight"]), t(sd[m + "mlp.0.bias"])
        w["merge.fc2.w"], w["merge.fc2.b"] = t(sd[m + "mlp.2.weight"]), t(sd[m + "mlp.2.bias"])
        return cls(cfg, w)

    def _angles(self, grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
        """[patches, head_dim / 2] rotation angles: the first half of the pairs turns with the patch row, the second
        with its column.  Patches are ordered frame by frame, inside a frame by 2x2 merge cell."""
        c = self.cfg
        D = c.embed_dim // c.num_heads
        m = c.spatial_merge_size
        inv = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2, dtype=torch.float32) / (D // 2)))
        out = []
        for t, h, w_ in grids:
            r = torch.arange(h)[:, None].expand(h, w_).reshape(h // m, m, w_ // m, m).permute(0, 2, 1, 3).flatten()
            cc = torch.arange(w_)[None, :].expand(h, w_).reshape(h // m, m, w_ // m, m).permute(0, 2, 1, 3).flatten()
            ang = torch.cat([r[:, None].float() * inv, cc[:, None].float() * inv], -1)
            out.append(ang.repeat(t, 1))
        return torch.cat(out, 0)

    def forward(self, patches: torch.Tensor, grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
        """``patches`` [N, channels * 2 * patch * patch] (see :func:`image_to_patches`), ``grids`` the (frames, rows,
        cols) of each image -> soft tokens [N / 4, hidden_size] in the weights' dtype."""
        c, w, dev = self.cfg, self.w, self.device
        H, nh = c.embed_dim, c.num_heads
        D = H // nh
        dt = w["patch.w"].dtype
        x = Dn.gemm_bf16(patches.to(dev).to(dt).contiguous(), w["patch.w"])
        T = x.shape[0]
        ang = self._angles(grids).to(dev)
        cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :]                  # [T, 1, D]
        sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
        lens_l = [h * w_ for t, h, w_ in grids for _ in range(t)]
        lens = torch.tensor(lens_l, dtype=torch.int32)
        starts = (torch.cumsum(lens, 0) - lens).to(torch.int32).to(dev)
        lens = lens.to(dev)
        for l in range(c.depth):
            p = f"l{l}."
            h = Dn.norm(x, w[p + "norm1.g"], w[p + "norm1.b"], eps=1e-6)
            qkv = Dn.gemm_bf16(h, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            qk = qkv[:, : 2 * H].view(T, 2 * nh, D).float()
            rot = torch.cat([-qk[..., D // 2:], qk[..., : D // 2]], -1)
            qkv[:, : 2 * H] = (qk * cos + rot * sin).to(dt).view(T, 2 * H)
            ctx = A.varlen_attention(qkv[:, :H].view(T, nh, D), qkv[:, H:2 * H].view(T, nh, D),
                                     qkv[:, 2 * H:].view(T, nh, D), starts, lens, max(lens_l), causal=False).view(T, H)
            x = Dn.gemm_bf16(ctx.to(dt), w[p + "o.w"], bias=w[p + "o.b"], residual=x)
            h = Dn.norm(x, w[p + "norm2.g"], w[p + "norm2.b"], eps=1e-6)
            if c.hidden_act in Dn.ACT:                       # the activation rides in the GEMM's epilogue
                m = Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=c.hidden_act)
            else:
                m = _act(Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"]), c.hidden_act)
            x = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
        k = c.spatial_merge_size ** 2
        x = Dn.norm(x, w["merge.ln.g"], w["merge.ln.b"], eps=1e-6).view(T // k, k * H)
        m = Dn.gemm_bf16(x.contiguous(), w["merge.fc1.w"], bias=w["merge.fc1.b"], act="gelu")
        return Dn.gemm_bf16(m, w["merge.fc2.w"], bias=w["merge.fc2.b"])


# -- image -> patches ------------------------------------------------------------------------------------------
CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    """Target size: both sides multiples of ``factor`` (patch x merge), area within [min_pixels, max_pixels],
    aspect ratio kept as closely as that allows."""
    import math

    if max(height, width) / max(min(height, width), 1) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def image_to_patches(image: torch.Tensor, cfg: Qwen2VLVisionConfig, min_pixels: int = 56 * 56,
                     max_pixels: int = 14 * 14 * 4 * 1280, size: Optional[Tuple[int, int]] = None):
    """uint8 [H, W, 3] image -> (patches [rows * cols, 3 * 2 * patch * patch] fp32, (1, rows, cols)).

    The image is resized (bicubic, antialiased) to the :func:`smart_resize` size, scaled to [0, 1], normalised with
    the CLIP statistics and repeated along time to fill one temporal patch.  Patches are emitted merge cell by
    merge cell (the four patches of a 2x2 cell are consecutive), each flattened as (channel, time, y, x)."""
    P, m, tp = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    H0, W0 = image.shape[0], image.shape[1]
    h, w = size or smart_resize(H0, W0, P * m, min_pixels, max_pixels)
    x = image.permute(2, 0, 1)[None].float()
    if (h, w) != (H0, W0):
        x = torch.nn.functional.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True)
        x = x.round().clamp(0, 255)                       # the resized image goes back to 8-bit pixels
    x = x[0] / 255.0
    x = (x - torch.tensor(CLIP_MEAN)[:, None, None]) / torch.tensor(CLIP_STD)[:, None, None]
    gh, gw = h // P, w // P
    v = x[None].expand(tp, -1, -1, -1)                    # [time, C, h, w]
    v = v.reshape(tp, 3, gh // m, m, P, gw // m, m, P).permute(2, 5, 3, 6, 1, 0, 4, 7)
    return v.reshape(gh * gw, 3 * tp * P * P).contiguous(), (1, gh, gw)


# -- rotary positions in the decoder -----------------------------------------------------------------------------
def rope_index(ids: Sequence[int], grids: Sequence[Tuple[int, int, int]], image_token_id: int,
               merge: int = 2) -> Tuple[torch.Tensor, int]:
    """Prompt token ids + the (frames, rows, cols) patch grid of each image, in order -> (positions [3, T] int64,
    delta).  Text tokens advance all three streams together; an image's placeholder run takes (frame, row, col) of
    each merged cell, offset by the position where the image starts; whatever follows continues from the largest
    position so far.  ``delta`` is what must be added to a cache index beyond the prompt to get its position."""
    T = len(ids)
    pos = torch.zeros((3, T), dtype=torch.int64)
    i, nxt, g = 0, 0, 0
    while i < T:
        if ids[i] == image_token_id and g < len(grids):
            t, h, w = grids[g]
            lh, lw = h // merge, w // merge
            n = t * lh * lw
            if i + n > T or any(x != image_token_id for x in ids[i:i + n]):
                raise ValueError("image placeholder run does not match the image's patch grid")
            tt = torch.arange(t).repeat_interleave(lh * lw)
            hh = torch.arange(lh).repeat_interleave(lw).repeat(t)
            ww = torch.arange(lw).repeat(lh * t)
            pos[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
            nxt += max(t, lh, lw)
            i += n
            g += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    if g != len(grids):
        raise ValueError("fewer image placeholders than images")
    return pos, nxt - T


def mrope_rotate(x: torch.Tensor, pos3: torch.Tensor, theta: float, sections: Sequence[int]) -> torch.Tensor:
    """Rotate x [T, heads, D] by three position streams: rotary pair ``j`` (dimensions j and j + D/2) turns by
    ``pos[s(j)] * theta^(-2j/D)`` where ``s(j)`` is 0 / 1 / 2 for the pairs in the first / second / third section."""
    T, Hh, D = x.shape
    assert sum(sections) == D // 2
    inv = theta ** (-torch.arange(0, D, 2, dtype=torch.float32, device=x.device) / D)          # [D/2]
    which = torch.repeat_interleave(torch.arange(3, device=x.device), torch.tensor(list(sections), device=x.device))
    p = pos3.to(x.device).float()[which]                                                      # [D/2, T]
    ang = (p.T * inv)[:, None, :]                                                              # [T, 1, D/2]
    cos, sin = torch.cat([ang.cos()] * 2, -1), torch.cat([ang.sin()] * 2, -1)
    xf = x.float()
    rot = torch.cat([-xf[..., D // 2:], xf[..., : D // 2]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


def text_state_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The decoder's tensors under the names a text-only Qwen2 checkpoint uses (``model.layers.*``, ``lm_head.*``),
    whichever of the two published layouts (``model.language_model.*`` or ``model.*`` beside ``visual.*``) the
    checkpoint has."""
    out: Dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        if k.startswith("model.language_model."):
            out["model." + k[len("model.language_model."):]] = v
        elif k.startswith("language_model."):               # retrieval checkpoints: the bare backbone
            out["model." + k[len("language_model."):]] = v
        elif k.startswith(("model.visual.", "visual.")):
            continue
        else:
            out[k] = v
    return out
