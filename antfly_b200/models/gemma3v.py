"""Gemma-3 image inputs: a SigLIP vision transformer and the projector that turns its patch states into 256 soft
tokens of the Gemma-3 decoder.

Vision tower (zig/pkg/inference/src/architectures/gemma3_vision.zig): patch convolution as one GEMM, learned
positions (no class token), pre-LayerNorm blocks with biased projections and tanh-GELU MLPs, a final LayerNorm.
Heads are 72 wide in the released towers; the attention wrapper runs them zero-padded to the next built width.
Projector (zig/pkg/inference/src/architectures/gemma3_projector.zig): the patch grid is average-pooled down to
16 x 16 cells, RMS-normalised with a (1 + gamma) gain and multiplied by the projection matrix.  In the decoder the
soft tokens of one image attend to one another in both directions.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import attention as A
from ..ops import dense as Dn


@dataclass
class SiglipVisionConfig:
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_hidden_layers: int = 27
    num_attention_heads: int = 16
    image_size: int = 896
    patch_size: int = 14
    num_channels: int = 3
    layer_norm_eps: float = 1e-6
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_hf(cls, d: dict) -> "SiglipVisionConfig":
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None})


class Gemma3VisionModel:
    def __init__(self, cfg: SiglipVisionConfig, weights: Dict[str, torch.Tensor], tokens_per_image: int = 256,
                 norm_eps: float = 1e-6):
        self.cfg, self.w, self.tokens_per_image, self.norm_eps = cfg, weights, tokens_per_image, norm_eps
        self.device = weights["patch.w"].device

    @classmethod
    def from_state_dict(cls, cfg: SiglipVisionConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16, tokens_per_image: int = 256, norm_eps: float = 1e-6
                        ) -> "Gemma3VisionModel":
        pre = next((p for p in ("model.vision_tower.vision_model.", "vision_tower.vision_model.", "vision_model.")
                    if p + "embeddings.patch_embedding.weight" in sd), None)
        if pre is None:
            raise KeyError("embeddings.patch_embedding.weight")
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {
            "patch.w": t(sd[pre + "embeddings.patch_embedding.weight"].flatten(1)),
            "patch.b": t(sd[pre + "embeddings.patch_embedding.bias"]),
            "pos": sd[pre + "embeddings.position_embedding.weight"].float().to(device),
            "post.g": t(sd[pre + "post_layernorm.weight"]), "post.b": t(sd[pre + "post_layernorm.bias"]),
        }
        for l in range(cfg.num_hidden_layers):
            s, p = pre + f"encoder.layers.{l}.", f"l{l}."
            for n in ("layer_norm1", "layer_norm2"):
                w[p + n + ".g"], w[p + n + ".b"] = t(sd[s + n + ".weight"]), t(sd[s + n + ".bias"])
            w[p + "qkv.w"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0))
            w[p + "qkv.b"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.bias"] for n in "qkv"], 0))
            w[p + "o.w"], w[p + "o.b"] = t(sd[s + "self_attn.out_proj.weight"]), t(sd[s + "self_attn.out_proj.bias"])
            w[p + "fc1.w"], w[p + "fc1.b"] = t(sd[s + "mlp.fc1.weight"]), t(sd[s + "mlp.fc1.bias"])
            w[p + "fc2.w"], w[p + "fc2.b"] = t(sd[s + "mlp.fc2.weight"]), t(sd[s + "mlp.fc2.bias"])
        mp = next((p for p in ("model.multi_modal_projector.", "multi_modal_projector.")
                   if p + "mm_input_projection_weight" in sd), None)
        if mp is not None:
            w["proj.w"] = t(sd[mp + "mm_input_projection_weight"].T)        # stored [vision, text]: use as a Linear
            w["proj.norm"] = t(sd[mp + "mm_soft_emb_norm.weight"])
        return cls(cfg, w, tokens_per_image, norm_eps)

    def patch_states(self, pixels: torch.Tensor) -> torch.Tensor:
        """Normalised images [B, 3, S, S] -> final patch states [B, (S / patch)^2, hidden]."""
        c, w, dev = self.cfg, self.w, self.device
        B, C, S, _ = pixels.shape
        P = c.patch_size
        g = S // P
        H, nh = c.hidden_size, c.num_attention_heads
        D = H // nh
        dt = w["patch.w"].dtype
        cols = pixels.to(dev).to(dt).view(B, C, g, P, g, P).permute(0, 2, 4, 1, 3, 5).reshape(B * g * g, C * P * P)
        x = Dn.gemm_bf16(cols.contiguous(), w["patch.w"], bias=w["patch.b"]).float().view(B, g * g, H)
        x = (x + w["pos"][: g * g][None]).to(dt).reshape(B * g * g, H).contiguous()
        T, n = B * g * g, g * g
        lens = torch.full((B,), n, dtype=torch.int32, device=dev)
        starts = (torch.arange(B, dtype=torch.int32, device=dev) * n).to(torch.int32)
        fused = c.hidden_act if c.hidden_act in ("gelu", "relu") else None
        for l in range(c.num_hidden_layers):
            p = f"l{l}."
            h = Dn.norm(x, w[p + "layer_norm1.g"], w[p + "layer_norm1.b"], eps=c.layer_norm_eps)
            qkv = Dn.gemm_bf16(h, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            ctx = A.varlen_attention(qkv[:, :H].view(T, nh, D), qkv[:, H:2 * H].view(T, nh, D),
                                     qkv[:, 2 * H:].view(T, nh, D), starts, lens, n, causal=False).view(T, H)
            x = Dn.gemm_bf16(ctx.to(dt), w[p + "o.w"], bias=w[p + "o.b"], residual=x)
            h = Dn.norm(x, w[p + "layer_norm2.g"], w[p + "layer_norm2.b"], eps=c.layer_norm_eps)
            m = Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=fused)
            if fused is None:
                m = torch.nn.functional.gelu(m.float(), approximate="tanh").to(m.dtype)
            x = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
        x = Dn.norm(x, w["post.g"], w["post.b"], eps=c.layer_norm_eps)
        return x.view(B, n, H)

    def soft_tokens(self, pixels: torch.Tensor) -> torch.Tensor:
        """Images -> [B, tokens_per_image, decoder width] soft tokens."""
        w = self.w
        if "proj.w" not in w:
            raise ValueError("this checkpoint has no multimodal projector")
        x = self.patch_states(pixels)
        B, n, H = x.shape
        g = int(round(n ** 0.5))
        side = int(round(self.tokens_per_image ** 0.5))
        k = g // side
        pooled = x.float().view(B, side, k, side, k, H).mean((2, 4)).reshape(B * side * side, H)
        normed = Dn.norm(pooled.to(x.dtype).contiguous(), w["proj.norm"], eps=self.norm_eps, rms=True,
                         gamma_plus_one=True)
        return Dn.gemm_bf16(normed, w["proj.w"]).view(B, side * side, -1)


def gemma3_pixels(image: torch.Tensor, size: int) -> torch.Tensor:
    """uint8 [H, W, 3] -> [3, size, size] in [-1, 1]: bilinear resize of the whole image (no crop), mean / std 0.5."""
    x = image.permute(2, 0, 1)[None].float()
    x = torch.nn.functional.interpolate(x, size=(size, size), mode="bilinear", align_corners=False, antialias=True)
    return (x[0].round().clamp(0, 255) / 255.0 - 0.5) / 0.5
