"""ModernBERT encoder: rotary positions, pre-LayerNorm blocks, gated-GELU MLP, alternating global / local attention.

What differs from the BERT encoder and how it maps to the kernels:

* no position / type embeddings: the token embedding goes through a LayerNorm; Q and K are rotated in place inside
  the fused QKV buffer by the strided RoPE kernel, with one base for the global layers and another for the local
  ones;
* every ``global_attn_every_n_layers``-th layer attends to the whole sequence, the others to a two-sided window of
  ``local_attention`` tokens (``|key - query| <= local_attention / 2``), which is the windowed mode of the packed
  varlen flash kernel;
* blocks are pre-norm (``x + attn(ln x)``, ``x + mlp(ln x)``; the first block's attention norm is the identity
  because the embedding norm precedes it), LayerNorms and linears have no bias by default;
* the MLP is ``Wo(act(a) * g)`` with ``a, g`` the two halves of one GEMM's output.

The reference runs this family in zig/pkg/inference/src/architectures/modern_bert.zig (encoder) with the
classification / embedding heads wired in architectures/session_factory.zig.  Weight names are the Hugging Face
ones (``model.embeddings.tok_embeddings`` / ``model.layers.N.{attn_norm,attn.Wqkv,attn.Wo,mlp_norm,mlp.Wi,mlp.Wo}``
/ ``model.final_norm`` / ``head.{dense,norm}`` / ``classifier``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..ops import attention as A
from ..ops import dense as Dn
from ..ops import reference as R
from .bert import PackedBatch


@dataclass
class ModernBertConfig:
    vocab_size: int = 50368
    hidden_size: int = 768
    num_hidden_layers: int = 22
    num_attention_heads: int = 12
    intermediate_size: int = 1152
    max_position_embeddings: int = 8192
    norm_eps: float = 1e-5
    hidden_activation: str = "gelu"
    global_attn_every_n_layers: int = 3
    local_attention: int = 128
    global_rope_theta: float = 160000.0
    local_rope_theta: float = 10000.0
    classifier_pooling: str = "cls"
    classifier_activation: str = "gelu"
    num_labels: int = 0
    pooling: str = "mean"
    layer_types: Optional[List[str]] = None
    position_offset: int = 0     # positions start at 0 (field shared with the BERT-family pipelines)

    @classmethod
    def from_hf(cls, d: dict) -> "ModernBertConfig":
        keys = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in keys and v is not None}
        rp = d.get("rope_parameters") or {}
        if isinstance(rp.get("full_attention"), dict):
            kw["global_rope_theta"] = float(rp["full_attention"].get("rope_theta", 160000.0))
        if isinstance(rp.get("sliding_attention"), dict):
            kw["local_rope_theta"] = float(rp["sliding_attention"].get("rope_theta", 10000.0))
        if "num_labels" not in kw and d.get("id2label") and (d.get("architectures") or [""])[0].endswith(
                "Classification"):
            kw["num_labels"] = len(d["id2label"])
        return cls(**kw)

    def is_global(self, layer: int) -> bool:
        if self.layer_types:
            return self.layer_types[layer] == "full_attention"
        return layer % self.global_attn_every_n_layers == 0


class ModernBertModel:
    """Packed-batch ModernBERT with the interface of :class:`antfly_b200.models.bert.BertModel` (``encode``, ``embed``,
    ``classify``, ``token_logits``)."""

    def __init__(self, cfg: ModernBertConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["emb.tok"].device

    @classmethod
    def from_state_dict(cls, cfg: ModernBertConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "ModernBertModel":
        pre = "model." if any(k.startswith("model.") for k in sd) else ""
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}

        def put(dst: str, src: str, required: bool = True) -> None:
            if src in sd:
                w[dst] = t(sd[src])
            elif required:
                raise KeyError(src)

        put("emb.tok", pre + "embeddings.tok_embeddings.weight")
        put("emb.ln.g", pre + "embeddings.norm.weight")
        put("emb.ln.b", pre + "embeddings.norm.bias", False)
        for l in range(cfg.num_hidden_layers):
            s, p = f"{pre}layers.{l}.", f"l{l}."
            put(p + "ln1.g", s + "attn_norm.weight", required=l > 0)
            put(p + "ln1.b", s + "attn_norm.bias", False)
            put(p + "qkv.w", s + "attn.Wqkv.weight")
            put(p + "qkv.b", s + "attn.Wqkv.bias", False)
            put(p + "o.w", s + "attn.Wo.weight")
            put(p + "o.b", s + "attn.Wo.bias", False)
            put(p + "ln2.g", s + "mlp_norm.weight")
            put(p + "ln2.b", s + "mlp_norm.bias", False)
            put(p + "wi.w", s + "mlp.Wi.weight")
            put(p + "wi.b", s + "mlp.Wi.bias", False)
            put(p + "wo.w", s + "mlp.Wo.weight")
            put(p + "wo.b", s + "mlp.Wo.bias", False)
        put("lnf.g", pre + "final_norm.weight")
        put("lnf.b", pre + "final_norm.bias", False)
        put("head.w", "head.dense.weight", False)
        put("head.b", "head.dense.bias", False)
        put("head.ln.g", "head.norm.weight", False)
        put("head.ln.b", "head.norm.bias", False)
        put("cls.w", "classifier.weight", False)
        put("cls.b", "classifier.bias", False)
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def encode(self, b: PackedBatch) -> torch.Tensor:
        """Hidden states after the final norm, packed: [T, H] bf16."""
        cfg, w = self.cfg, self.w
        H, nh = cfg.hidden_size, cfg.num_attention_heads
        D = H // nh
        x = Dn.embed_gather(b.ids, w["emb.tok"])
        x = Dn.norm(x, w["emb.ln.g"], w.get("emb.ln.b"), eps=cfg.norm_eps)
        T = x.shape[0]
        half = cfg.local_attention // 2
        for l in range(cfg.num_hidden_layers):
            p = f"l{l}."
            h = Dn.norm(x, w[p + "ln1.g"], w.get(p + "ln1.b"), eps=cfg.norm_eps) if p + "ln1.g" in w else x
            qkv = Dn.gemm_bf16(h, w[p + "qkv.w"], bias=w.get(p + "qkv.b"))
            glob = cfg.is_global(l)
            A.rope_(qkv[:, :2 * H].view(T, 2 * nh, D), b.positions,
                    cfg.global_rope_theta if glob else cfg.local_rope_theta)
            ctx = A.varlen_attention(qkv[:, :H].view(T, nh, D), qkv[:, H:2 * H].view(T, nh, D),
                                     qkv[:, 2 * H:].view(T, nh, D), b.starts, b.lens, b.max_len, causal=False,
                                     window=0 if glob else half + 1).view(T, H)
            x = Dn.gemm_bf16(ctx, w[p + "o.w"], bias=w.get(p + "o.b"), residual=x)
            h = Dn.norm(x, w[p + "ln2.g"], w.get(p + "ln2.b"), eps=cfg.norm_eps)
            ag = Dn.gemm_bf16(h, w[p + "wi.w"], bias=w.get(p + "wi.b"))
            I = ag.shape[1] // 2
            m = Dn.gated_act(ag, cfg.hidden_activation)
            x = Dn.gemm_bf16(m, w[p + "wo.w"], bias=w.get(p + "wo.b"), residual=x)
        return Dn.norm(x, w["lnf.g"], w.get("lnf.b"), eps=cfg.norm_eps)

    def embed(self, b: PackedBatch, pooling: Optional[str] = None, normalize: bool = True) -> torch.Tensor:
        """Sentence embeddings, fp32 [B, H]."""
        return Dn.pool(self.encode(b), b.starts, b.lens, mode=pooling or self.cfg.pooling, normalize=normalize)

    def _head(self, h: torch.Tensor) -> torch.Tensor:
        w, cfg = self.w, self.cfg
        act = cfg.classifier_activation if cfg.classifier_activation in Dn.ACT else None
        y = Dn.gemm_bf16(h, w["head.w"], bias=w.get("head.b"), act=act)
        if act is None:
            y = R.act_fn(y.float(), cfg.classifier_activation).to(h.dtype)
        return Dn.norm(y, w["head.ln.g"], w.get("head.ln.b"), eps=cfg.norm_eps)

    def classify(self, b: PackedBatch) -> torch.Tensor:
        """Sequence-classification logits, fp32 [B, num_labels]: pool (class token or mean), prediction head
        (dense, activation, LayerNorm), classifier."""
        assert "cls.w" in self.w, "model has no classification head"
        h = self.encode(b)
        mode = "cls" if self.cfg.classifier_pooling == "cls" else "mean"
        pooled = Dn.pool(h, b.starts, b.lens, mode=mode, normalize=False).to(h.dtype)
        return Dn.gemm_bf16(self._head(pooled), self.w["cls.w"], bias=self.w.get("cls.b"), out_dtype=torch.float32)

    def token_logits(self, b: PackedBatch) -> torch.Tensor:
        """Token-classification logits, fp32 [T, num_labels] (prediction head then classifier on every token)."""
        assert "cls.w" in self.w, "model has no classification head"
        h = self.encode(b)
        return Dn.gemm_bf16(self._head(h), self.w["cls.w"], bias=self.w.get("cls.b"), out_dtype=torch.float32)

    def param_count(self) -> int:
        return sum(t.numel() for t in self.w.values())
