"""Gemma-4 vision tower and projector: patches with 2-D positions -> soft tokens in the language model's space.

* Patch embedder: a linear map of the flattened 16 x 16 x 3 patch (pixels rescaled to [-1, 1]) plus the sum of two
  learned position rows, one for the patch's x and one for its y coordinate; padding patches (position (-1, -1))
  get no position row and are masked out of attention.
* Encoder layers: the text decoder's layer without the causal mask -- four RMS norms, per-head RMS norms on Q / K, a
  weight-free norm on V, softmax scale 1, gated-GELU MLP -- with a two-dimensional rotary embedding: the first half
  of every head rotates by the x coordinate, the second half by y (each half-split, base 100).  Linear layers may
  clamp their inputs and outputs to stored ranges (``use_clipped_linears``).
* Pooler: k x k average pooling by patch position down to ``patches / pooling_kernel_size^2`` soft tokens, scaled by
  sqrt(hidden); optional standardisation with stored bias and scale; padding removed.
* Projector: weight-free RMS norm and a linear map into the text model's hidden size.

The reference's counterpart is architectures/gemma4_projector.zig + gemma4_runtime.zig.  Attention runs on the
packed (varlen) attention op, projections on the bf16 GEMM.  Checked against ``transformers`` on CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..ops import attention as A
from ..ops import dense as Dn
from ..ops import reference as R
from .gemma4 import _gelu_tanh, _rms, _rope_half


@dataclass
class Gemma4VisionConfig:
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 16
    num_attention_heads: int = 12
    num_key_value_heads: int = 12
    head_dim: int = 64
    rms_norm_eps: float = 1e-6
    pooling_kernel_size: int = 3
    patch_size: int = 16
    position_embedding_size: int = 10240
    use_clipped_linears: bool = False
    standardize: bool = False
    rope_theta: float = 100.0

    @classmethod
    def from_hf(cls, d: dict) -> "Gemma4VisionConfig":
        d = dict(d.get("vision_config") or d)
        kw = {k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None}
        kw["rope_theta"] = (d.get("rope_parameters") or {}).get("rope_theta", 100.0)
        return cls(**kw)


class Gemma4VisionTower:
    def __init__(self, cfg: Gemma4VisionConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device, self.dtype = weights["patch.w"].device, weights["patch.w"].dtype
        half = cfg.head_dim // 2          # channels rotated by one coordinate
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, 2, device=self.device).float() / half))

    @classmethod
    def from_state_dict(cls, cfg: Gemma4VisionConfig, sd: Dict[str, torch.Tensor], prefix: str = "", device="cuda",
                        dtype=torch.bfloat16) -> "Gemma4VisionTower":
        t = lambda x: x.to(dtype).to(device).contiguous()
        f = lambda x: x.float().to(device).contiguous()
        w: Dict[str, torch.Tensor] = {"patch.w": t(sd[prefix + "patch_embedder.input_proj.weight"]),
                                      "patch.pos": f(sd[prefix + "patch_embedder.position_embedding_table"])}
        if cfg.standardize:
            w["std.bias"], w["std.scale"] = f(sd[prefix + "std_bias"]), f(sd[prefix + "std_scale"])

        def lin(dst: str, src: str):
            w[dst] = t(sd[src + ".linear.weight"])
            if cfg.use_clipped_linears:
                w[dst + ".clip"] = torch.stack([sd[src + "." + n].float() for n in
                                                ("input_min", "input_max", "output_min", "output_max")]).to(device)

        for l in range(cfg.num_hidden_layers):
            s, p = f"{prefix}encoder.layers.{l}.", f"l{l}."
            for n in ("q", "k", "v", "o"):
                lin(p + n, s + f"self_attn.{n}_proj")
            w[p + "qn"], w[p + "kn"] = f(sd[s + "self_attn.q_norm.weight"]), f(sd[s + "self_attn.k_norm.weight"])
            for n, key in (("ln1", "input_layernorm"), ("ln2", "post_attention_layernorm"),
                           ("ln3", "pre_feedforward_layernorm"), ("ln4", "post_feedforward_layernorm")):
                w[p + n] = f(sd[s + key + ".weight"])
            for n in ("gate", "up", "down"):
                lin(p + n, s + f"mlp.{n}_proj")
        return cls(cfg, w)

    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        clip = self.w.get(name + ".clip")
        if clip is not None:
            x = x.clamp(clip[0], clip[1])
        y = Dn.gemm_bf16(x.to(self.dtype).contiguous(), self.w[name], out_dtype=torch.float32).float()
        return y.clamp(clip[2], clip[3]) if clip is not None else y

    def forward(self, pixel_values: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """pixel_values [B, P, 3 * patch^2] in [0, 1]; position_ids [B, P, 2] (x, y), (-1, -1) = padding.
        Returns the soft tokens of all images, padding removed: [n_tokens, hidden] fp32."""
        c, w = self.cfg, self.w
        B, P, _ = pixel_values.shape
        H, nh, nkv, D = c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim
        pad = (position_ids == -1).all(-1)                                    # [B, P]
        pos = position_ids.clamp_min(0).long()
        x = self._plain(2.0 * (pixel_values.float() - 0.5), "patch.w")
        posemb = w["patch.pos"][0][pos[..., 0]] + w["patch.pos"][1][pos[..., 1]]
        x = x + torch.where(pad[..., None], torch.zeros_like(posemb), posemb)
        # attention only among an image's real patches: pack them (padding rows are dropped and restored as zeros)
        keep = ~pad
        lens = keep.sum(1).int()
        starts = (torch.cumsum(lens, 0) - lens).int()
        xs = x[keep]                                                          # [T, H]
        px, py = pos[..., 0][keep], pos[..., 1][keep]
        T = xs.shape[0]
        max_len = int(lens.max()) if B else 0
        for l in range(c.num_hidden_layers):
            p = f"l{l}."
            h = _rms(xs, w[p + "ln1"], c.rms_norm_eps)
            q = self._rope2d(_rms(self._lin(h, p + "q").view(T, nh, D), w[p + "qn"], c.rms_norm_eps), px, py)
            k = self._rope2d(_rms(self._lin(h, p + "k").view(T, nkv, D), w[p + "kn"], c.rms_norm_eps), px, py)
            v = _rms(self._lin(h, p + "v").view(T, nkv, D), None, c.rms_norm_eps)
            if xs.is_cuda:
                ctx = A.varlen_attention(q.to(torch.bfloat16).contiguous(), k.to(torch.bfloat16).contiguous(),
                                         v.to(torch.bfloat16).contiguous(), starts.to(xs.device), lens.to(xs.device),
                                         max_len, causal=False, scale=1.0)
            else:   # the fp32 oracle, without the bf16 rounding of the op's CPU wrapper
                cu = torch.cat([starts.long(), (starts[-1:] + lens[-1:]).long()])
                ctx = R.varlen_attention(q, k, v, cu, 1.0, False, 0)
            a = self._lin(ctx.float().reshape(T, nh * D), p + "o")
            xs = xs + _rms(a, w[p + "ln2"], c.rms_norm_eps)
            h = _rms(xs, w[p + "ln3"], c.rms_norm_eps)
            m = self._lin(_gelu_tanh(self._lin(h, p + "gate")) * self._lin(h, p + "up"), p + "down")
            xs = xs + _rms(m, w[p + "ln4"], c.rms_norm_eps)
        full = torch.zeros((B, P, H), dtype=torch.float32, device=xs.device)
        full[keep] = xs
        # pool k x k patches by position
        kk = c.pooling_kernel_size
        out_len = P // (kk * kk)
        if out_len != P:
            k = int((P // out_len) ** 0.5)
            max_x = pos[..., 0].max(-1, keepdim=True).values + 1
            cell = (pos[..., 0] // k) + (max_x // k) * (pos[..., 1] // k)
            wts = torch.nn.functional.one_hot(cell, out_len).float() / (k * k)          # [B, P, out]
            wts = wts * keep[..., None]
            # (padding rows are zero, so whether they are counted in a cell does not change the sum)
            pooled = wts.transpose(1, 2) @ full
            valid = ~(torch.nn.functional.one_hot(cell, out_len).float() == 0).all(1)
        else:
            pooled, valid = full, keep
        pooled = pooled * H ** 0.5
        tokens = pooled[valid]
        if c.standardize:
            tokens = (tokens - w["std.bias"]) * w["std.scale"]
        return tokens

    def _plain(self, x: torch.Tensor, name: str) -> torch.Tensor:
        shp = x.shape
        y = Dn.gemm_bf16(x.reshape(-1, shp[-1]).to(self.dtype).contiguous(), self.w[name], out_dtype=torch.float32)
        return y.float().view(*shp[:-1], -1)

    def _rope2d(self, x: torch.Tensor, px: torch.Tensor, py: torch.Tensor) -> torch.Tensor:
        half = x.shape[-1] // 2
        return torch.cat([_rope_half(x[..., :half], px, self.inv_freq), _rope_half(x[..., half:], py, self.inv_freq)], -1)


class Gemma4Projector:
    """Soft tokens -> text hidden size: weight-free RMS norm, then a linear map."""

    def __init__(self, weight: torch.Tensor, eps: float = 1e-6):
        self.w, self.eps = weight, eps

    @classmethod
    def from_state_dict(cls, sd: Dict[str, torch.Tensor], prefix: str = "model.embed_vision.", eps: float = 1e-6,
                        device="cuda", dtype=torch.bfloat16) -> "Gemma4Projector":
        return cls(sd[prefix + "embedding_projection.weight"].to(dtype).to(device).contiguous(), eps)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        x = _rms(tokens, None, self.eps)
        return Dn.gemm_bf16(x.to(self.w.dtype).contiguous(), self.w, out_dtype=torch.float32).float()


def gemma4_target_size(height: int, width: int, patch: int, max_patches: int, pool: int) -> Tuple[int, int]:
    """The largest (height, width) with the image's aspect ratio whose sides are multiples of ``pool * patch`` and
    that hold at most ``max_patches`` patches; a side that would round to nothing becomes one pooling cell."""
    import math

    factor = math.sqrt(max_patches * patch * patch / (height * width))
    side = pool * patch
    th, tw = int(factor * height // side) * side, int(factor * width // side) * side
    longest = (max_patches // (pool * pool)) * side
    if th == 0 and tw == 0:
        raise ValueError(f"a {height} x {width} image cannot be resized to whole {side}-pixel cells")
    if th == 0:
        th, tw = side, min(int(width // height) * side, longest)
    elif tw == 0:
        tw, th = side, min(int(height // width) * side, longest)
    return th, tw


def gemma4_patches(image: torch.Tensor, patch: int = 16, max_soft_tokens: int = 280, pool: int = 3):
    """uint8 [H, W, 3] -> (patches [max_patches, 3 patch^2] in [0, 1] (zero rows after the image's own),
    positions [max_patches, 2] as (x, y), -1 on padding rows, number of soft tokens).  Bicubic resize with
    antialiasing to the aspect-preserving target size, rounded back to 8 bits before the 1/255 rescale; a patch
    row is laid out pixel-major, channel-minor."""
    max_patches = max_soft_tokens * pool * pool
    h, w = image.shape[0], image.shape[1]
    th, tw = gemma4_target_size(h, w, patch, max_patches, pool)
    x = image[..., :3].permute(2, 0, 1)[None].float()
    if (th, tw) != (h, w):
        x = torch.nn.functional.interpolate(x, size=(th, tw), mode="bicubic", align_corners=False, antialias=True)
        x = x.round().clamp(0, 255)
    x = x[0] / 255.0
    ph, pw = th // patch, tw // patch
    rows = x.reshape(3, ph, patch, pw, patch).permute(1, 3, 2, 4, 0).reshape(ph * pw, -1)
    ys, xs = torch.meshgrid(torch.arange(ph), torch.arange(pw), indexing="ij")
    pos = torch.stack([xs.flatten(), ys.flatten()], -1)
    pad = max_patches - ph * pw
    rows = torch.nn.functional.pad(rows, (0, 0, 0, pad))
    pos = torch.nn.functional.pad(pos, (0, 0, 0, pad), value=-1)
    return rows, pos, ph * pw // (pool * pool)


class Gemma4Multimodal:
    """Text decoder + vision tower + projector as one model: image placeholder tokens in the prompt take the
    projected soft tokens of their image, in order (the reference's Gemma-4 vision path:
    go-termite pkg/termite/lib/pipelines image-text generation; transformers Gemma4Model.forward)."""

    def __init__(self, text, tower: Gemma4VisionTower, projector: Gemma4Projector, image_token_id: int,
                 pad_token_id: int = 0, bidirectional_vision: bool = False, boi_token_id: Optional[int] = None,
                 eoi_token_id: Optional[int] = None, max_soft_tokens: int = 280):
        self.text, self.tower, self.projector = text, tower, projector
        self.image_token_id, self.pad_token_id = image_token_id, pad_token_id
        self.boi_token_id, self.eoi_token_id = boi_token_id, eoi_token_id
        self.bidirectional_vision = bidirectional_vision
        self.max_soft_tokens = max_soft_tokens
        self.device, self.dtype, self.cfg = text.device, text.dtype, text.cfg

    def new_state(self):
        return self.text.new_state()

    def prepare_images(self, ids, images, bos_id: Optional[int] = None):
        """Prompt ids with one placeholder token per image + the images -> (ids with every placeholder replaced by
        begin marker, that image's soft-token placeholders, end marker; keyword inputs of ``forward``)."""
        from ..pipelines.multimodal import load_image

        ids = list(ids)
        n_ph = sum(1 for t in ids if t == self.image_token_id)
        if n_ph == 0 and images:             # a prompt format without image slots: the images lead the prompt
            at = 1 if ids and bos_id is not None and ids[0] == bos_id else 0
            ids[at:at] = [self.image_token_id] * len(images)
            n_ph = len(images)
        if n_ph != len(images):
            raise ValueError(f"{len(images)} image(s) for {n_ph} placeholder(s) in the prompt")
        vc = self.tower.cfg
        prep = [gemma4_patches(load_image(s).cpu(), vc.patch_size, self.max_soft_tokens, vc.pooling_kernel_size)
                for s in images]
        out, it = [], iter(prep)
        for t in ids:
            if t != self.image_token_id:
                out.append(t)
                continue
            n = next(it)[2]
            out += ([self.boi_token_id] if self.boi_token_id is not None else []) + [self.image_token_id] * n + \
                   ([self.eoi_token_id] if self.eoi_token_id is not None else [])
        return out, {"pixel_values": torch.stack([p[0] for p in prep]).to(self.device),
                     "position_ids": torch.stack([p[1] for p in prep]).to(self.device)}

    @classmethod
    def from_state_dict(cls, hf_config: dict, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "Gemma4Multimodal":
        from .gemma4 import Gemma4Config, Gemma4TextModel

        tc = hf_config["text_config"]
        text = Gemma4TextModel.from_state_dict(Gemma4Config.from_hf(tc), sd, device=device, dtype=dtype)
        vcfg = Gemma4VisionConfig.from_hf(hf_config["vision_config"])
        tower = Gemma4VisionTower.from_state_dict(vcfg, sd, prefix="model.vision_tower.", device=device, dtype=dtype)
        proj = Gemma4Projector.from_state_dict(sd, eps=hf_config["vision_config"].get("rms_norm_eps", 1e-6),
                                               device=device, dtype=dtype)
        return cls(text, tower, proj, int(hf_config.get("image_token_id", 258880)), int(tc.get("pad_token_id") or 0),
                   tc.get("use_bidirectional_attention") == "vision", hf_config.get("boi_token_id"),
                   hf_config.get("eoi_token_id"))

    def encode_images(self, pixel_values: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """Patches [B, P, 3 p^2] + their (x, y) grid positions [B, P, 2] (-1 = padding) -> soft tokens
        [n, text hidden], image after image."""
        return self.projector.forward(self.tower.forward(pixel_values, position_ids))

    def vision_groups(self, ids: torch.Tensor) -> torch.Tensor:
        """Image number of every prompt position (a run of placeholder tokens is one image), -1 for text."""
        is_img = ids == self.image_token_id
        prev = torch.cat([torch.zeros(1, dtype=torch.bool, device=ids.device), is_img[:-1]])
        starts = is_img & ~prev
        grp = torch.cumsum(starts.int(), 0) - 1
        return torch.where(is_img, grp, torch.full_like(grp, -1))

    def forward(self, ids: torch.Tensor, state=None, pixel_values: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None):
        ids = ids.long()
        if pixel_values is None:
            return self.text.forward(ids, state)
        rows = torch.nonzero(ids == self.image_token_id).flatten()
        soft = self.encode_images(pixel_values, position_ids)
        if soft.shape[0] != rows.numel():
            raise ValueError(f"{rows.numel()} image placeholder tokens but {soft.shape[0]} soft tokens")
        groups = self.vision_groups(ids) if self.bidirectional_vision else None
        return self.text.forward(ids, state, soft_rows=rows, soft_vals=soft, pad_token_id=self.pad_token_id,
                                 vision_groups=groups)

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, max_new_tokens: int, pixel_values=None, position_ids=None, eos=()):
        logits, st = self.forward(ids, None, pixel_values, position_ids)
        out = []
        for _ in range(max_new_tokens):
            nxt = int(logits[-1].argmax())
            out.append(nxt)
            if nxt in eos:
                break
            logits, st = self.text.forward(torch.tensor([nxt], device=ids.device), st)
        return out
