"""Differentiable networks for fine-tuning: the Llama-family decoder and the BERT-family encoder as plain torch
modules built from the same checkpoints and configurations the serving models read.

Serving runs hand-written kernels over packed, quantised weights and has no backward pass; training wants autograd
over the original weights.  These modules restate the two architectures with module names equal to the checkpoint's
tensor names (``model.layers.3.self_attn.q_proj``, ``encoder.layer.0.attention.self.query``), so that an adapter
trained here carries the names :mod:`antfly_b200.formats.lora` resolves when it merges the adapter for serving.
The reference trains through its own graph IR and autodiff (zig/lib/ml/src/graph/autodiff.zig, trainers under
zig/pkg/inference/src/finetune/); here torch's autograd plays that part.

Decoder features: grouped-query attention, rotary positions (half-split, frequency scale or table), optional QKV
bias (Qwen2), per-head Q / K norms (Qwen3), sliding window (Mistral), Gemma's 1 + gamma norms / scaled embeddings /
GeGLU; sequence packing through per-token document ids (attention stays inside a document, positions restart);
activation checkpointing per layer.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..models.bert import BertConfig
from ..models.llama import LlamaConfig


class RMSNorm(nn.Module):
    def __init__(self, weight: torch.Tensor, eps: float, plus_one: bool):
        super().__init__()
        self.weight, self.eps, self.plus_one = nn.Parameter(weight.clone()), eps, plus_one

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        w = self.weight.float() + 1.0 if self.plus_one else self.weight.float()
        return (y * w).to(x.dtype)


def _linear(w: torch.Tensor, b: Optional[torch.Tensor]) -> nn.Linear:
    lin = nn.Linear(w.shape[1], w.shape[0], bias=b is not None)
    lin.weight = nn.Parameter(w.clone())
    if b is not None:
        lin.bias = nn.Parameter(b.clone())
    return lin


def _rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rope_dim: int, half_split: bool,
          mscale: float) -> torch.Tensor:
    """x [B, S, H, D]; positions [B, S]."""
    ang = positions[..., None].float() * inv_freq                       # [B, S, rd / 2]
    c, s = (ang.cos() * mscale)[:, :, None, :], (ang.sin() * mscale)[:, :, None, :]
    xf = x.float()
    rot, rest = xf[..., :rope_dim], xf[..., rope_dim:]
    if half_split:
        a, b = rot[..., : rope_dim // 2], rot[..., rope_dim // 2:]
        out = torch.cat([a * c - b * s, a * s + b * c], -1)
    else:
        a, b = rot[..., 0::2], rot[..., 1::2]
        out = torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)
    return torch.cat([out, rest], -1).to(x.dtype)


class DecoderAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig, sd: Dict[str, torch.Tensor], pre: str):
        super().__init__()
        g = lambda n: sd.get(pre + n)
        self.q_proj = _linear(sd[pre + "q_proj.weight"], g("q_proj.bias"))
        self.k_proj = _linear(sd[pre + "k_proj.weight"], g("k_proj.bias"))
        self.v_proj = _linear(sd[pre + "v_proj.weight"], g("v_proj.bias"))
        self.o_proj = _linear(sd[pre + "o_proj.weight"], g("o_proj.bias"))
        self.q_norm = RMSNorm(sd[pre + "q_norm.weight"], cfg.rms_norm_eps, cfg.norm_plus_one) if cfg.qk_norm else None
        self.k_norm = RMSNorm(sd[pre + "k_norm.weight"], cfg.rms_norm_eps, cfg.norm_plus_one) if cfg.qk_norm else None
        self.cfg = cfg

    def forward(self, x, positions, mask, inv_freq):
        c = self.cfg
        B, S, _ = x.shape
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        q = self.q_proj(x).view(B, S, Hq, D)
        k = self.k_proj(x).view(B, S, Hkv, D)
        v = self.v_proj(x).view(B, S, Hkv, D)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        q = _rope(q, positions, inv_freq, c.rope_dim, c.rope_half_split, c.rope_mscale)
        k = _rope(k, positions, inv_freq, c.rope_dim, c.rope_half_split, c.rope_mscale)
        rep = Hq // Hkv
        k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
        scale = c.attn_scale if c.attn_scale else D ** -0.5
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                             scale=scale)
        return self.o_proj(out.transpose(1, 2).reshape(B, S, Hq * D))


class DecoderMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, sd, pre: str):
        super().__init__()
        self.gate_proj = _linear(sd[pre + "gate_proj.weight"], None)
        self.up_proj = _linear(sd[pre + "up_proj.weight"], None)
        self.down_proj = _linear(sd[pre + "down_proj.weight"], None)
        self.act = {"silu": F.silu, "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "gelu": F.gelu}[cfg.gate_act]

    def forward(self, x):
        return self.down_proj(self.act(self.gate_proj(x)) * self.up_proj(x))


class DecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, sd, pre: str):
        super().__init__()
        self.input_layernorm = RMSNorm(sd[pre + "input_layernorm.weight"], cfg.rms_norm_eps, cfg.norm_plus_one)
        self.post_attention_layernorm = RMSNorm(sd[pre + "post_attention_layernorm.weight"], cfg.rms_norm_eps,
                                                cfg.norm_plus_one)
        self.self_attn = DecoderAttention(cfg, sd, pre + "self_attn.")
        self.mlp = DecoderMLP(cfg, sd, pre + "mlp.")

    def forward(self, x, positions, mask, inv_freq):
        x = x + self.self_attn(self.input_layernorm(x), positions, mask, inv_freq)
        return x + self.mlp(self.post_attention_layernorm(x))


class _DecoderBody(nn.Module):
    def __init__(self, cfg: LlamaConfig, sd, dtype):
        super().__init__()
        self.embed_tokens = nn.Embedding.from_pretrained(sd["model.embed_tokens.weight"].to(dtype), freeze=True)
        self.layers = nn.ModuleList([DecoderLayer(cfg, sd, f"model.layers.{l}.") for l in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(sd["model.norm.weight"], cfg.rms_norm_eps, cfg.norm_plus_one)


class DecoderNet(nn.Module):
    """Llama / Mistral / Qwen2 / Qwen3 / Gemma decoder.  ``forward`` returns final-norm hidden states; the vocabulary
    projection is a separate call (:meth:`logits`) so that the loss can run it over chunks of tokens."""

    def __init__(self, cfg: LlamaConfig, sd: Dict[str, torch.Tensor], dtype=torch.float32, checkpointing: bool = False):
        super().__init__()
        if cfg.num_experts or cfg.bitnet or cfg.post_norms or cfg.mrope_sections or cfg.layer_rope:
            raise NotImplementedError("fine-tuning covers the dense Llama / Mistral / Qwen2 / Qwen3 / Gemma decoders")
        if "model.layers.0.self_attn.q_proj.weight" not in sd:
            raise NotImplementedError("checkpoints with fused projections (Phi-3) are not trainable here")
        sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
        self.cfg, self.checkpointing = cfg, checkpointing
        self.neftune_alpha = 0.0          # > 0: uniform noise of magnitude alpha / sqrt(S * H) on the embeddings while training
        self.model = _DecoderBody(cfg, sd, dtype)
        head = sd.get("lm_head.weight")
        self.lm_head = _linear(head if head is not None and not cfg.tie_word_embeddings
                               else sd["model.embed_tokens.weight"], None)
        if cfg.rope_inv_freq:
            inv = torch.tensor(cfg.rope_inv_freq, dtype=torch.float32)
        else:
            inv = cfg.rope_freq_scale * cfg.rope_theta ** (-2.0 * torch.arange(cfg.rope_dim // 2).float() / cfg.rope_dim)
        self.register_buffer("inv_freq", inv, persistent=False)

    def forward(self, ids: torch.Tensor, doc_ids: Optional[torch.Tensor] = None,
                pad_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids [B, S].  ``doc_ids`` [B, S] (packed rows: tokens attend within their document and positions restart
        at each document); ``pad_mask`` [B, S] True on real tokens (right- or left-padded rows)."""
        B, S = ids.shape
        c = self.cfg
        idx = torch.arange(S, device=ids.device)
        causal = idx[None, :] <= idx[:, None]                                        # [S, S] key <= query
        if c.sliding_window:
            causal = causal & (idx[None, :] > idx[:, None] - c.sliding_window)
        mask = causal[None].expand(B, S, S)
        if doc_ids is not None:
            mask = mask & (doc_ids[:, :, None] == doc_ids[:, None, :])
            first = (doc_ids != torch.nn.functional.pad(doc_ids, (1, 0), value=-1)[:, :-1])
            start = torch.where(first, idx[None].expand(B, S), torch.zeros_like(doc_ids)).cummax(1).values
            positions = idx[None] - start
        elif pad_mask is not None:
            mask = mask & pad_mask[:, None, :]
            positions = (pad_mask.long().cumsum(1) - 1).clamp_min(0)
        else:
            positions = idx[None].expand(B, S)
        mask = mask | torch.eye(S, dtype=torch.bool, device=ids.device)[None]        # no empty rows (padding queries)
        x = self.model.embed_tokens(ids) * c.embed_scale
        if self.training and self.neftune_alpha > 0:
            x = x + (torch.rand_like(x) * 2 - 1) * (self.neftune_alpha / (S * x.shape[-1]) ** 0.5)
        for layer in self.model.layers:
            if self.checkpointing and self.training:
                x = checkpoint(layer, x, positions, mask[:, None], self.inv_freq, use_reentrant=False)
            else:
                x = layer(x, positions, mask[:, None], self.inv_freq)
        return self.model.norm(x)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        y = self.lm_head(hidden).float()
        cap = self.cfg.final_logit_softcapping
        return cap * torch.tanh(y / cap) if cap else y


# ----------------------------------------------------------------------------------------------------------
class _BertSelfAttention(nn.Module):
    def __init__(self, sd, pre):
        super().__init__()
        for n in ("query", "key", "value"):
            setattr(self, n, _linear(sd[pre + n + ".weight"], sd[pre + n + ".bias"]))


class _BertAttnOutput(nn.Module):
    def __init__(self, sd, pre, eps):
        super().__init__()
        self.dense = _linear(sd[pre + "dense.weight"], sd[pre + "dense.bias"])
        self.LayerNorm = nn.LayerNorm(self.dense.out_features, eps=eps)
        self.LayerNorm.weight, self.LayerNorm.bias = nn.Parameter(sd[pre + "LayerNorm.weight"].clone()), nn.Parameter(
            sd[pre + "LayerNorm.bias"].clone())


class _BertAttention(nn.Module):
    def __init__(self, sd, pre, eps):
        super().__init__()
        self.self = _BertSelfAttention(sd, pre + "self.")
        self.output = _BertAttnOutput(sd, pre + "output.", eps)


class _BertIntermediate(nn.Module):
    def __init__(self, sd, pre):
        super().__init__()
        self.dense = _linear(sd[pre + "dense.weight"], sd[pre + "dense.bias"])


class BertLayer(nn.Module):
    def __init__(self, cfg: BertConfig, sd, pre):
        super().__init__()
        self.nh = cfg.num_attention_heads
        self.attention = _BertAttention(sd, pre + "attention.", cfg.layer_norm_eps)
        self.intermediate = _BertIntermediate(sd, pre + "intermediate.")
        self.output = _BertAttnOutput(sd, pre + "output.", cfg.layer_norm_eps)
        self.act = {"gelu": F.gelu, "relu": F.relu, "gelu_new": lambda t: F.gelu(t, approximate="tanh")}[cfg.hidden_act]

    def forward(self, x, mask):
        B, S, H = x.shape
        a = self.attention
        split = lambda t: t.view(B, S, self.nh, H // self.nh).transpose(1, 2)
        ctx = F.scaled_dot_product_attention(split(a.self.query(x)), split(a.self.key(x)), split(a.self.value(x)),
                                             attn_mask=mask)
        x = a.output.LayerNorm(x + a.output.dense(ctx.transpose(1, 2).reshape(B, S, H)))
        return self.output.LayerNorm(x + self.output.dense(self.act(self.intermediate.dense(x))))


class _BertEmbeddings(nn.Module):
    def __init__(self, cfg, sd, pre):
        super().__init__()
        emb = lambda n: nn.Embedding.from_pretrained(sd[pre + n + ".weight"].clone(), freeze=True)
        self.word_embeddings, self.position_embeddings = emb("word_embeddings"), emb("position_embeddings")
        self.token_type_embeddings = emb("token_type_embeddings")
        self.LayerNorm = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.LayerNorm.weight = nn.Parameter(sd[pre + "LayerNorm.weight"].clone())
        self.LayerNorm.bias = nn.Parameter(sd[pre + "LayerNorm.bias"].clone())


class _BertEncoder(nn.Module):
    def __init__(self, cfg, sd, pre):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(cfg, sd, f"{pre}layer.{l}.") for l in range(cfg.num_hidden_layers)])


class EncoderNet(nn.Module):
    """BERT / RoBERTa encoder with an optional sequence-classification head (cross-encoder rerankers).  ``forward``
    returns token states [B, S, H]; :meth:`pool` and :meth:`score` give sentence vectors and head logits."""

    def __init__(self, cfg: BertConfig, sd: Dict[str, torch.Tensor], checkpointing: bool = False):
        super().__init__()
        pre = next((p for p in ("", "bert.", "roberta.", "model.", "xlm_roberta.")
                    if p + "embeddings.word_embeddings.weight" in sd), None)
        if pre is None:
            raise KeyError("checkpoint has no embeddings.word_embeddings.weight")
        sd = {k: (v.float() if v.is_floating_point() else v) for k, v in sd.items()}
        self.cfg, self.checkpointing, self.prefix = cfg, checkpointing, pre
        self.embeddings = _BertEmbeddings(cfg, sd, pre + "embeddings.")
        self.encoder = _BertEncoder(cfg, sd, pre + "encoder.")
        self.classifier = None
        if cfg.num_labels and "classifier.weight" in sd:
            self.classifier = _linear(sd["classifier.weight"], sd["classifier.bias"])
        self.pooler_dense = _linear(sd[pre + "pooler.dense.weight"], sd[pre + "pooler.dense.bias"]) \
            if cfg.use_pooler and pre + "pooler.dense.weight" in sd else None

    def forward(self, ids, mask, type_ids=None):
        B, S = ids.shape
        pos = torch.arange(S, device=ids.device)[None] + self.cfg.position_offset
        if self.cfg.position_offset:
            pos = (mask.long().cumsum(1) * mask.long()) + self.cfg.position_offset - 1 + (1 - mask.long())
        e = self.embeddings
        tt = type_ids if type_ids is not None else torch.zeros_like(ids)
        x = e.LayerNorm(e.word_embeddings(ids) + e.position_embeddings(pos) + e.token_type_embeddings(tt))
        am = mask.bool()[:, None, None, :]
        for layer in self.encoder.layer:
            x = checkpoint(layer, x, am, use_reentrant=False) if self.checkpointing and self.training else layer(x, am)
        return x

    def pool(self, states, mask, mode: Optional[str] = None, normalize: bool = True):
        mode = mode or self.cfg.pooling
        m = mask.float()[..., None]
        if mode == "cls":
            v = states[:, 0]
        elif mode == "max":
            v = states.masked_fill(m == 0, float("-inf")).amax(1)
        elif mode == "last":
            v = states[torch.arange(states.shape[0]), mask.long().sum(1) - 1]
        else:
            v = (states * m).sum(1) / m.sum(1).clamp_min(1.0)
        return F.normalize(v, dim=-1) if normalize else v

    def score(self, states):
        if self.classifier is None:
            raise ValueError("this checkpoint has no classification head")
        cls = states[:, 0]
        if self.pooler_dense is not None:
            cls = torch.tanh(self.pooler_dense(cls))
        return self.classifier(cls)
