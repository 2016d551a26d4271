"""DeBERTa-v2 / v3 encoder: BERT-style post-LayerNorm blocks with *disentangled* attention.

The score of query i against key j is ``(Qc_i . Kc_j + Qc_i . Kr[d(i, j)] + Kc_j . Qr[d(j, i)]) / sqrt(3 D)``: a
content-to-content term plus content-to-position and position-to-content terms, where ``Kr`` / ``Qr`` project a
table of relative-position embeddings (shared with the content projections in v3, ``share_att_key``) and ``d`` is
the log-bucketed relative distance.  The reference implements this in
zig/pkg/inference/src/architectures/deberta.zig and as its ``termite_deberta_attention_f32`` CUDA kernel
(zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:1471, one thread per output element).

Execution here: projections, output and FFN GEMMs (bias / GELU / residual epilogues) and the LayerNorms are the
same kernels as the BERT encoder; the two position terms are small GEMMs against the 2 x span position table
followed by an index gather, added to the content scores before the softmax.  That attention core is written with
tensor ops per sequence (no fused kernel yet), so this family runs correctly on either device but is not a tuned
path.  Weight names are the Hugging Face ones (``deberta.embeddings.*``, ``deberta.encoder.layer.N.*``,
``deberta.encoder.rel_embeddings``, ``pooler.dense``, ``classifier``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..ops import dense as Dn
from ..ops import reference as R
from .bert import PackedBatch


@dataclass
class DebertaConfig:
    vocab_size: int = 128100
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 0
    layer_norm_eps: float = 1e-7
    hidden_act: str = "gelu"
    relative_attention: bool = True
    max_relative_positions: int = -1
    position_buckets: int = 256
    pos_att_type: Optional[List[str]] = None
    share_att_key: bool = True
    norm_rel_ebd: str = "layer_norm"
    position_biased_input: bool = False
    pooler_hidden_act: str = "gelu"
    num_labels: int = 0
    pooling: str = "mean"
    position_offset: int = 0

    @classmethod
    def from_hf(cls, d: dict) -> "DebertaConfig":
        keys = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in keys and v is not None}
        if isinstance(kw.get("pos_att_type"), str):
            kw["pos_att_type"] = [s for s in kw["pos_att_type"].split("|") if s]
        if "num_labels" not in kw and d.get("id2label") and (d.get("architectures") or [""])[0].endswith(
                "Classification"):
            kw["num_labels"] = len(d["id2label"])
        if d.get("conv_kernel_size", 0):
            raise ValueError("DeBERTa checkpoints with the convolution branch are not supported")
        return cls(**kw)

    @property
    def span(self) -> int:
        if self.position_buckets > 0:
            return self.position_buckets
        return self.max_relative_positions if self.max_relative_positions > 0 else self.max_position_embeddings


def relative_buckets(L: int, bucket_size: int, max_position: int, device) -> torch.Tensor:
    """[L, L] of query - key distances, log-bucketed beyond bucket_size / 2 (exact below)."""
    i = torch.arange(L, device=device)
    rel = i[:, None] - i[None, :]
    if bucket_size <= 0 or max_position <= 0:
        return rel
    mid = bucket_size // 2
    sign = torch.sign(rel)
    a = torch.where((rel < mid) & (rel > -mid), torch.full_like(rel, mid - 1), rel.abs()).float()
    logp = torch.ceil(torch.log(a / mid) / math.log((max_position - 1) / mid) * (mid - 1)) + mid
    return torch.where(a <= mid, rel.float(), logp * sign).long()


class DebertaModel:
    """Packed-batch DeBERTa-v2 / v3 with the interface of :class:`antfly_b200.models.bert.BertModel`."""

    def __init__(self, cfg: DebertaConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["emb.word"].device
        self._rel_cache: Dict[int, torch.Tensor] = {}

    @classmethod
    def from_state_dict(cls, cfg: DebertaConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "DebertaModel":
        pre = "deberta." if any(k.startswith("deberta.") for k in sd) else ""
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}

        def put(dst: str, src: str, required: bool = True) -> None:
            if src in sd:
                w[dst] = t(sd[src])
            elif required:
                raise KeyError(src)

        e = pre + "embeddings."
        put("emb.word", e + "word_embeddings.weight")
        put("emb.pos", e + "position_embeddings.weight", cfg.position_biased_input)
        put("emb.type", e + "token_type_embeddings.weight", cfg.type_vocab_size > 0)
        put("emb.proj", e + "embed_proj.weight", False)
        put("emb.ln.g", e + "LayerNorm.weight")
        put("emb.ln.b", e + "LayerNorm.bias")
        enc = pre + "encoder."
        put("rel.emb", enc + "rel_embeddings.weight", cfg.relative_attention)
        put("rel.ln.g", enc + "LayerNorm.weight", False)
        put("rel.ln.b", enc + "LayerNorm.bias", False)
        for l in range(cfg.num_hidden_layers):
            s, p = f"{enc}layer.{l}.", f"l{l}."
            a = s + "attention.self."
            w[p + "qkv.w"] = t(torch.cat([sd[a + f"{n}_proj.weight"] for n in ("query", "key", "value")], 0))
            w[p + "qkv.b"] = t(torch.cat([sd[a + f"{n}_proj.bias"] for n in ("query", "key", "value")], 0))
            put(p + "posk.w", a + "pos_key_proj.weight", False)
            put(p + "posk.b", a + "pos_key_proj.bias", False)
            put(p + "posq.w", a + "pos_query_proj.weight", False)
            put(p + "posq.b", a + "pos_query_proj.bias", False)
            put(p + "o.w", s + "attention.output.dense.weight")
            put(p + "o.b", s + "attention.output.dense.bias")
            put(p + "ln1.g", s + "attention.output.LayerNorm.weight")
            put(p + "ln1.b", s + "attention.output.LayerNorm.bias")
            put(p + "ff1.w", s + "intermediate.dense.weight")
            put(p + "ff1.b", s + "intermediate.dense.bias")
            put(p + "ff2.w", s + "output.dense.weight")
            put(p + "ff2.b", s + "output.dense.bias")
            put(p + "ln2.g", s + "output.LayerNorm.weight")
            put(p + "ln2.b", s + "output.LayerNorm.bias")
        put("pooler.w", "pooler.dense.weight", False)
        put("pooler.b", "pooler.dense.bias", False)
        put("cls.w", "classifier.weight", False)
        put("cls.b", "classifier.bias", False)
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def _rel_index(self, L: int) -> torch.Tensor:
        if L not in self._rel_cache:
            cfg = self.cfg
            maxp = cfg.max_relative_positions if cfg.max_relative_positions > 0 else cfg.max_position_embeddings
            rel = relative_buckets(L, cfg.position_buckets, maxp, self.device)
            self._rel_cache[L] = rel
        return self._rel_cache[L]

    def _attention(self, q, k, v, starts: List[int], lens: List[int], pos_k, pos_q) -> torch.Tensor:
        """q / k / v [T, nh, D]; pos_k / pos_q [2 span, nh, D] or None.  Returns [T, nh * D]."""
        cfg = self.cfg
        T, nh, D = q.shape
        span = cfg.span
        factor = 1 + (pos_k is not None) + (pos_q is not None)
        inv = 1.0 / math.sqrt(D * factor)
        out = torch.empty((T, nh, D), dtype=q.dtype, device=q.device)
        for s, L in zip(starts, lens):
            qq, kk, vv = (x[s:s + L].float().transpose(0, 1) for x in (q, k, v))        # [nh, L, D]
            sc = qq @ kk.transpose(1, 2)
            if pos_k is not None or pos_q is not None:
                rel = self._rel_index(L)
            if pos_k is not None:
                c2p = qq @ pos_k.float().permute(1, 2, 0)                                   # [nh, L, 2 span]
                idx = (rel + span).clamp(0, 2 * span - 1)
                sc = sc + torch.gather(c2p, 2, idx[None].expand(nh, L, L))
            if pos_q is not None:
                p2c = kk @ pos_q.float().permute(1, 2, 0)                                   # [nh, L(key), 2 span]
                idx = (-rel + span).clamp(0, 2 * span - 1)
                sc = sc + torch.gather(p2c, 2, idx[None].expand(nh, L, L)).transpose(1, 2)
            out[s:s + L] = ((sc * inv).softmax(-1) @ vv).transpose(0, 1).to(q.dtype)
        return out.view(T, nh * D)

    def encode(self, b: PackedBatch) -> torch.Tensor:
        """Hidden states of every token, packed: [T, H]."""
        cfg, w = self.cfg, self.w
        H, nh = cfg.hidden_size, cfg.num_attention_heads
        D = H // nh
        x = w["emb.word"].index_select(0, b.ids.long()).float()
        if "emb.pos" in w:
            x = x + w["emb.pos"].index_select(0, b.positions.long()).float()
        if "emb.type" in w:
            ty = b.type_ids.long() if b.type_ids is not None else torch.zeros_like(b.ids, dtype=torch.long)
            x = x + w["emb.type"].index_select(0, ty).float()
        x = x.to(w["emb.word"].dtype)
        if "emb.proj" in w:
            x = Dn.gemm_bf16(x, w["emb.proj"])
        x = Dn.norm(x, w["emb.ln.g"], w["emb.ln.b"], eps=cfg.layer_norm_eps)
        T = x.shape[0]
        starts, lens = b.starts.tolist(), b.lens.tolist()
        rel = None
        if cfg.relative_attention:
            rel = w["rel.emb"][: 2 * cfg.span]
            if "layer_norm" in cfg.norm_rel_ebd and "rel.ln.g" in w:
                rel = Dn.norm(rel, w["rel.ln.g"], w["rel.ln.b"], eps=cfg.layer_norm_eps)
        types = cfg.pos_att_type or []
        for l in range(cfg.num_hidden_layers):
            p = f"l{l}."
            qkv = Dn.gemm_bf16(x, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            pos_k = pos_q = None
            if rel is not None:
                if cfg.share_att_key:
                    pqk = Dn.gemm_bf16(rel, w[p + "qkv.w"][: 2 * H], bias=w[p + "qkv.b"][: 2 * H])
                    pos_q, pos_k = pqk[:, :H], pqk[:, H:]
                else:
                    if "c2p" in types:
                        pos_k = Dn.gemm_bf16(rel, w[p + "posk.w"], bias=w.get(p + "posk.b"))
                    if "p2c" in types:
                        pos_q = Dn.gemm_bf16(rel, w[p + "posq.w"], bias=w.get(p + "posq.b"))
                pos_k = pos_k.reshape(-1, nh, D) if "c2p" in types else None
                pos_q = pos_q.reshape(-1, nh, D) if "p2c" in types else None
            ctx = self._attention(qkv[:, :H].reshape(T, nh, D), qkv[:, H:2 * H].reshape(T, nh, D),
                                  qkv[:, 2 * H:].reshape(T, nh, D), starts, lens, pos_k, pos_q)
            h = Dn.gemm_bf16(ctx, w[p + "o.w"], bias=w[p + "o.b"], residual=x)
            x = Dn.norm(h, w[p + "ln1.g"], w[p + "ln1.b"], eps=cfg.layer_norm_eps)
            f = Dn.gemm_bf16(x, w[p + "ff1.w"], bias=w[p + "ff1.b"], act=cfg.hidden_act)
            h = Dn.gemm_bf16(f, w[p + "ff2.w"], bias=w[p + "ff2.b"], residual=x)
            x = Dn.norm(h, w[p + "ln2.g"], w[p + "ln2.b"], eps=cfg.layer_norm_eps)
        return x

    def embed(self, b: PackedBatch, pooling: Optional[str] = None, normalize: bool = True) -> torch.Tensor:
        return Dn.pool(self.encode(b), b.starts, b.lens, mode=pooling or self.cfg.pooling, normalize=normalize)

    def classify(self, b: PackedBatch) -> torch.Tensor:
        """Sequence-classification logits, fp32 [B, num_labels]: first token -> pooler dense + activation ->
        classifier."""
        assert "cls.w" in self.w, "model has no classification head"
        h = self.encode(b)
        cls = Dn.pool(h, b.starts, b.lens, mode="cls", normalize=False).to(h.dtype)
        if "pooler.w" in self.w:
            act = self.cfg.pooler_hidden_act if self.cfg.pooler_hidden_act in Dn.ACT else None
            cls = Dn.gemm_bf16(cls, self.w["pooler.w"], bias=self.w["pooler.b"], act=act)
            if act is None:
                cls = R.act_fn(cls.float(), self.cfg.pooler_hidden_act).to(h.dtype)
        return Dn.gemm_bf16(cls, self.w["cls.w"], bias=self.w["cls.b"], out_dtype=torch.float32)

    def token_logits(self, b: PackedBatch) -> torch.Tensor:
        assert "cls.w" in self.w, "model has no classification head"
        return Dn.gemm_bf16(self.encode(b), self.w["cls.w"], bias=self.w["cls.b"], out_dtype=torch.float32)

    def param_count(self) -> int:
        return sum(t.numel() for t in self.w.values())
