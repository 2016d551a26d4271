"""CLIP: a text tower and a vision tower (ViT) that embed captions and images into one space.

Both towers are pre-LayerNorm transformers (``x + attn(ln1 x)``, ``x + mlp(ln2 x)``) on the same kernels as the
BERT encoder: the LayerNorm kernel, the tcgen05 bf16 GEMM with bias / residual epilogues and the packed
variable-length flash attention (causal for text, bidirectional for image patches).  What is specific:

* text: learned positions, causal mask, the hidden state of the end-of-text token (the highest token id of a
  sequence, as in the original model, or the configured eos id) goes through ``text_projection``;
* vision: the patch embedding is a stride-``patch`` convolution, done as a GEMM over unfolded patches; a class
  token is prepended, positions are learned, a pre-LayerNorm precedes the stack, and the post-LayerNorm class token
  goes through ``visual_projection``; pixels come from :func:`antfly_b200.ops.image_ops.clip_preprocess`;
* the MLP activation is quick-GELU (``x * sigmoid(1.702 x)``) for the original checkpoints, applied between the
  two GEMMs, or GELU (a GEMM epilogue) for later ones.

The reference embeds images and text through the same two towers (zig/pkg/inference/src/architectures/clip.zig,
zig/pkg/inference/src/pipelines/embedding.zig:432 ``embedImages``).  Weight names are the Hugging Face ones
(``text_model.*`` / ``vision_model.*``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import attention as A
from ..ops import dense as Dn


@dataclass
class ClipTowerConfig:
    hidden_size: int = 512
    num_hidden_layers: int = 12
    num_attention_heads: int = 8
    intermediate_size: int = 2048
    layer_norm_eps: float = 1e-5
    hidden_act: str = "quick_gelu"
    # text
    vocab_size: int = 49408
    max_position_embeddings: int = 77
    eos_token_id: int = 2
    # vision
    image_size: int = 224
    patch_size: int = 32


@dataclass
class ClipConfig:
    text: ClipTowerConfig
    vision: ClipTowerConfig
    projection_dim: int = 512

    @classmethod
    def from_hf(cls, d: dict) -> "ClipConfig":
        def tower(t: dict) -> ClipTowerConfig:
            keys = ClipTowerConfig.__dataclass_fields__
            return ClipTowerConfig(**{k: v for k, v in t.items() if k in keys and v is not None})

        return cls(tower(d.get("text_config", {})), tower(d.get("vision_config", {})), d.get("projection_dim", 512))


def _act(x: torch.Tensor, name: str) -> torch.Tensor:
    if name == "quick_gelu":
        xf = x.float()
        return (xf * torch.sigmoid(1.702 * xf)).to(x.dtype)
    raise ValueError(name)


class ClipModel:
    def __init__(self, cfg: ClipConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["text.emb.tok"].device

    # ------------------------------------------------------------------------------------------------------
    @classmethod
    def from_state_dict(cls, cfg: ClipConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "ClipModel":
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}

        def stack(prefix_hf: str, prefix: str, n_layers: int):
            for l in range(n_layers):
                s, p = f"{prefix_hf}.encoder.layers.{l}.", f"{prefix}.l{l}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "layer_norm1.weight"]), t(sd[s + "layer_norm1.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "layer_norm2.weight"]), t(sd[s + "layer_norm2.bias"])
                w[p + "qkv.w"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.weight"] for n in ("q", "k", "v")], 0))
                w[p + "qkv.b"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.bias"] for n in ("q", "k", "v")], 0))
                w[p + "o.w"], w[p + "o.b"] = t(sd[s + "self_attn.out_proj.weight"]), t(sd[s + "self_attn.out_proj.bias"])
                w[p + "fc1.w"], w[p + "fc1.b"] = t(sd[s + "mlp.fc1.weight"]), t(sd[s + "mlp.fc1.bias"])
                w[p + "fc2.w"], w[p + "fc2.b"] = t(sd[s + "mlp.fc2.weight"]), t(sd[s + "mlp.fc2.bias"])

        w["text.emb.tok"] = t(sd["text_model.embeddings.token_embedding.weight"])
        w["text.emb.pos"] = t(sd["text_model.embeddings.position_embedding.weight"])
        stack("text_model", "text", cfg.text.num_hidden_layers)
        w["text.lnf.g"], w["text.lnf.b"] = t(sd["text_model.final_layer_norm.weight"]), t(
            sd["text_model.final_layer_norm.bias"])
        w["text.proj"] = t(sd["text_projection.weight"])
        v = cfg.vision
        w["vis.patch.w"] = t(sd["vision_model.embeddings.patch_embedding.weight"].reshape(v.hidden_size, -1))
        if "vision_model.embeddings.patch_embedding.bias" in sd:
            w["vis.patch.b"] = t(sd["vision_model.embeddings.patch_embedding.bias"])
        w["vis.cls"] = t(sd["vision_model.embeddings.class_embedding"].reshape(1, -1))
        w["vis.emb.pos"] = t(sd["vision_model.embeddings.position_embedding.weight"])
        w["vis.pre.g"], w["vis.pre.b"] = t(sd["vision_model.pre_layrnorm.weight"]), t(
            sd["vision_model.pre_layrnorm.bias"])
        stack("vision_model", "vis", v.num_hidden_layers)
        w["vis.post.g"], w["vis.post.b"] = t(sd["vision_model.post_layernorm.weight"]), t(
            sd["vision_model.post_layernorm.bias"])
        w["vis.proj"] = t(sd["visual_projection.weight"])
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def _stack(self, x: torch.Tensor, prefix: str, tc: ClipTowerConfig, starts, lens, max_len: int,
               causal: bool) -> torch.Tensor:
        w = self.w
        H, nh = tc.hidden_size, tc.num_attention_heads
        D = H // nh
        T = x.shape[0]
        fused_act = tc.hidden_act if tc.hidden_act in Dn.ACT else None
        for l in range(tc.num_hidden_layers):
            p = f"{prefix}.l{l}."
            h = Dn.norm(x, w[p + "ln1.g"], w[p + "ln1.b"], eps=tc.layer_norm_eps)
            qkv = Dn.gemm_bf16(h, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            ctx = A.varlen_attention(qkv[:, :H].view(T, nh, D), qkv[:, H:2 * H].view(T, nh, D),
                                     qkv[:, 2 * H:].view(T, nh, D), starts, lens, max_len, causal=causal).view(T, H)
            x = Dn.gemm_bf16(ctx, w[p + "o.w"], bias=w[p + "o.b"], residual=x)
            h = Dn.norm(x, w[p + "ln2.g"], w[p + "ln2.b"], eps=tc.layer_norm_eps)
            m = Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=fused_act)
            if fused_act is None:
                m = _act(m, tc.hidden_act)
            x = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
        return x

    def embed_text(self, seqs: Sequence[Sequence[int]], normalize: bool = True) -> torch.Tensor:
        """Token id sequences (with their begin / end tokens) -> fp32 [B, projection_dim]."""
        tc, w, dev = self.cfg.text, self.w, self.device
        lens_l = [len(s) for s in seqs]
        lens = torch.tensor(lens_l, dtype=torch.int32)
        starts = (torch.cumsum(lens, 0) - lens).to(torch.int32)
        ids = torch.tensor([t for s in seqs for t in s], dtype=torch.int64, device=dev)
        pos = torch.cat([torch.arange(n) for n in lens_l]).to(dev)
        x = (w["text.emb.tok"].index_select(0, ids).float() + w["text.emb.pos"].index_select(0, pos).float()).to(
            w["text.emb.tok"].dtype)
        x = self._stack(x, "text", tc, starts.to(dev), lens.to(dev), max(lens_l), causal=True)
        x = Dn.norm(x, w["text.lnf.g"], w["text.lnf.b"], eps=tc.layer_norm_eps)
        # pooled token: the end-of-text token -- the highest id for the original vocabulary (eos id 2 in its
        # config is a placeholder), the first eos occurrence otherwise
        rows: List[int] = []
        for s, st in zip(seqs, starts.tolist()):
            if tc.eos_token_id == 2:
                rows.append(st + max(range(len(s)), key=lambda i: s[i]))
            else:
                rows.append(st + (list(s).index(tc.eos_token_id) if tc.eos_token_id in s else len(s) - 1))
        pooled = x.index_select(0, torch.tensor(rows, device=dev))
        e = Dn.gemm_bf16(pooled, w["text.proj"], out_dtype=torch.float32).float()
        return torch.nn.functional.normalize(e, dim=-1) if normalize else e

    def embed_images(self, pixels: torch.Tensor, normalize: bool = True) -> torch.Tensor:
        """Preprocessed pixels [B, 3, S, S] (see ops.image_ops.clip_preprocess) -> fp32 [B, projection_dim]."""
        vc, w, dev = self.cfg.vision, self.w, self.device
        B, C, S, _ = pixels.shape
        P = vc.patch_size
        g = S // P
        dt = w["vis.patch.w"].dtype
        # non-overlapping patches, each flattened in (channel, row, column) order = the convolution's weight layout
        patches = pixels.to(dev).to(dt).view(B, C, g, P, g, P).permute(0, 2, 4, 1, 3, 5).reshape(B * g * g, C * P * P)
        pe = Dn.gemm_bf16(patches.contiguous(), w["vis.patch.w"], bias=w.get("vis.patch.b"))
        H = vc.hidden_size
        x = torch.cat([w["vis.cls"].expand(B, 1, H), pe.view(B, g * g, H)], 1)
        x = (x.float() + w["vis.emb.pos"][: g * g + 1].float()[None]).to(dt).reshape(B * (g * g + 1), H).contiguous()
        n = g * g + 1
        lens = torch.full((B,), n, dtype=torch.int32, device=dev)
        starts = (torch.arange(B, dtype=torch.int32, device=dev) * n).to(torch.int32)
        x = Dn.norm(x, w["vis.pre.g"], w["vis.pre.b"], eps=vc.layer_norm_eps)
        x = self._stack(x, "vis", vc, starts, lens, n, causal=False)
        cls = x.view(B, n, H)[:, 0].contiguous()
        cls = Dn.norm(cls, w["vis.post.g"], w["vis.post.b"], eps=vc.layer_norm_eps)
        e = Dn.gemm_bf16(cls, w["vis.proj"], out_dtype=torch.float32).float()
        return torch.nn.functional.normalize(e, dim=-1) if normalize else e
