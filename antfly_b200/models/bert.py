"""BERT-family encoder (bi-encoder embedder, cross-encoder reranker, token-level heads).

Architecture and weight names follow the reference's bert.forward / embeddings / encoderLayer
(zig/pkg/inference/src/architectures/bert.zig:32-300): word + position + token-type embeddings -> LayerNorm ->
L x (QKV, attention, output projection, add+LayerNorm, GELU FFN, add+LayerNorm), post-LN.  The B200 execution is
different by design: sequences are packed (no padding tokens ever reach a GEMM), Q/K/V are one fused GEMM, bias /
GELU / residual are GEMM epilogues on the tcgen05 kernel, attention is the varlen flash kernel, and pooling +
L2-normalise is one kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import attention as A
from ..ops import dense as Dn


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"
    num_labels: int = 0          # > 0: sequence-classification head (cross-encoder)
    use_pooler: bool = False     # dense+tanh on [CLS] before the classifier (BertForSequenceClassification)
    position_offset: int = 0     # RoBERTa/XLM-R position ids start at padding_idx + 1 = 2
    pooling: str = "mean"

    @classmethod
    def from_hf(cls, d: dict) -> "BertConfig":
        keys = {f for f in cls.__dataclass_fields__}
        cfg = cls(**{k: v for k, v in d.items() if k in keys})
        if d.get("model_type") in ("roberta", "xlm-roberta"):
            cfg.position_offset = int(d.get("pad_token_id", 1)) + 1
        if "id2label" in d and cfg.num_labels == 0 and (d.get("architectures") or [""])[0].endswith(
                "ForSequenceClassification"):
            cfg.num_labels = len(d["id2label"])
        return cfg

    @classmethod
    def base(cls, **kw) -> "BertConfig":
        return cls(**kw)

    @classmethod
    def small_cpu_config(cls) -> "BertConfig":
        """The 6-layer, hidden-384 bi-encoder used for the CPU fp32 plumbing benchmark."""
        return cls(hidden_size=384, num_hidden_layers=6, num_attention_heads=12, intermediate_size=1536)


@dataclass
class PackedBatch:
    """Token ids of a batch of sequences laid end to end (int32), with per-sequence row ranges."""
    ids: torch.Tensor
    type_ids: Optional[torch.Tensor]
    positions: torch.Tensor
    starts: torch.Tensor
    lens: torch.Tensor
    max_len: int

    @property
    def batch(self) -> int:
        return self.starts.numel()

    def to(self, device, non_blocking: bool = False) -> "PackedBatch":
        f = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)
        return PackedBatch(f(self.ids), f(self.type_ids), f(self.positions), f(self.starts), f(self.lens),
                           self.max_len)

    def pin(self) -> "PackedBatch":
        f = lambda t: None if t is None else t.pin_memory()
        return PackedBatch(f(self.ids), f(self.type_ids), f(self.positions), f(self.starts), f(self.lens),
                           self.max_len)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in
                   (self.ids, self.type_ids, self.positions, self.starts, self.lens) if t is not None)


def pack_sequences(seqs: Sequence[Sequence[int]], type_ids: Optional[Sequence[Sequence[int]]] = None,
                   position_offset: int = 0) -> PackedBatch:
    """Concatenate token-id lists into one packed batch (host tensors)."""
    lens = torch.tensor([len(s) for s in seqs], dtype=torch.int32)
    starts = (torch.cumsum(lens, 0) - lens).to(torch.int32)
    ids = torch.tensor([t for s in seqs for t in s], dtype=torch.int32)
    pos = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in lens]) + position_offset if len(seqs) else \
        torch.zeros(0, dtype=torch.int32)
    ty = None
    if type_ids is not None:
        ty = torch.tensor([t for s in type_ids for t in s], dtype=torch.int32)
    return PackedBatch(ids, ty, pos, starts, lens, int(lens.max()) if len(seqs) else 0)


class BertModel:
    """Weights + forward.  Weights are plain bf16 tensors (fp32 on request for the CPU baseline)."""

    def __init__(self, cfg: BertConfig, weights: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.w = weights
        self.device = weights["emb.word"].device
        self.dtype = weights["emb.word"].dtype
        self.tp_rank, self.tp_size, self.comm = 0, 1, None

    def tensor_parallel(self, rank: int, world: int, comm) -> "BertModel":
        """This rank's shard of the encoder under the Megatron split the reference uses for its BERT / RoBERTa
        encoder and cross-encoder (zig/pkg/inference/src/architectures/bert.zig:309-352): query / key / value and the
        FFN's first linear are column-parallel (whole heads, a slice of the intermediate features), the attention
        output and the FFN's second linear are row-parallel and followed by an all-reduce (``comm.all_reduce``, the
        reference's all_sum at ops/mlx_compute.zig:1549); their biases are added once, after the reduction.
        Embeddings, LayerNorms and heads stay replicated."""
        cfg = self.cfg
        H, F, nh = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads
        if world == 1:
            return self
        if H % world or nh % world or F % world:
            raise ValueError(f"hidden {H}, heads {nh} and intermediate size {F} must all be divisible by {world} ranks")
        hs, fs = H // world, F // world
        w = dict(self.w)
        for l in range(cfg.num_hidden_layers):
            p = f"l{l}."
            qkv_w, qkv_b = self.w[p + "qkv.w"], self.w[p + "qkv.b"]
            rows = torch.cat([torch.arange(i * H + rank * hs, i * H + (rank + 1) * hs) for i in range(3)]).to(qkv_w.device)
            w[p + "qkv.w"], w[p + "qkv.b"] = qkv_w[rows].contiguous(), qkv_b[rows].contiguous()
            w[p + "o.w"] = self.w[p + "o.w"][:, rank * hs:(rank + 1) * hs].contiguous()
            w[p + "ff1.w"] = self.w[p + "ff1.w"][rank * fs:(rank + 1) * fs].contiguous()
            w[p + "ff1.b"] = self.w[p + "ff1.b"][rank * fs:(rank + 1) * fs].contiguous()
            w[p + "ff2.w"] = self.w[p + "ff2.w"][:, rank * fs:(rank + 1) * fs].contiguous()
        m = BertModel(cfg, w)
        m.tp_rank, m.tp_size, m.comm = rank, world, comm
        return m

    # ------------------------------------------------------------------------------------------------
    @classmethod
    def random_init(cls, cfg: BertConfig, device="cuda", seed: int = 0, dtype=torch.bfloat16) -> "BertModel":
        g = torch.Generator().manual_seed(seed)
        H, F = cfg.hidden_size, cfg.intermediate_size

        def rnd(*shape, std=0.02):
            return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

        w: Dict[str, torch.Tensor] = {
            "emb.word": rnd(cfg.vocab_size, H), "emb.pos": rnd(cfg.max_position_embeddings + cfg.position_offset, H),
            "emb.type": rnd(cfg.type_vocab_size, H),
            "emb.ln.g": torch.ones(H, dtype=dtype, device=device), "emb.ln.b": torch.zeros(H, dtype=dtype, device=device),
        }
        for l in range(cfg.num_hidden_layers):
            p = f"l{l}."
            w[p + "qkv.w"], w[p + "qkv.b"] = rnd(3 * H, H), rnd(3 * H)
            w[p + "o.w"], w[p + "o.b"] = rnd(H, H), rnd(H)
            w[p + "ln1.g"], w[p + "ln1.b"] = torch.ones(H, dtype=dtype, device=device), rnd(H)
            w[p + "ff1.w"], w[p + "ff1.b"] = rnd(F, H), rnd(F)
            w[p + "ff2.w"], w[p + "ff2.b"] = rnd(H, F), rnd(H)
            w[p + "ln2.g"], w[p + "ln2.b"] = torch.ones(H, dtype=dtype, device=device), rnd(H)
        if cfg.num_labels > 0:
            if cfg.use_pooler:
                w["pooler.w"], w["pooler.b"] = rnd(H, H), rnd(H)
            w["cls.w"], w["cls.b"] = rnd(cfg.num_labels, H, std=0.1), rnd(cfg.num_labels)
        return cls(cfg, w)

    @classmethod
    def from_state_dict(cls, cfg: BertConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "BertModel":
        """Map HF / reference tensor names (zig/pkg/inference/src/architectures/bert.zig:140-296) to the fused
        layout.  Accepts optional ``bert.`` / ``roberta.`` / ``model.`` prefixes."""
        def get(name: str) -> torch.Tensor:
            for pre in ("", "bert.", "roberta.", "model.", "xlm_roberta."):
                if pre + name in sd:
                    return sd[pre + name].to(dtype).to(device)
            raise KeyError(name)

        def opt(name: str):
            try:
                return get(name)
            except KeyError:
                return None

        H = cfg.hidden_size
        w: Dict[str, torch.Tensor] = {
            "emb.word": get("embeddings.word_embeddings.weight"),
            "emb.pos": get("embeddings.position_embeddings.weight"),
            "emb.ln.g": get("embeddings.LayerNorm.weight"), "emb.ln.b": get("embeddings.LayerNorm.bias"),
        }
        ty = opt("embeddings.token_type_embeddings.weight")
        w["emb.type"] = ty if ty is not None else torch.zeros((1, H), dtype=dtype, device=device)
        for l in range(cfg.num_hidden_layers):
            s, p = f"encoder.layer.{l}.", f"l{l}."
            w[p + "qkv.w"] = torch.cat([get(s + f"attention.self.{n}.weight") for n in ("query", "key", "value")], 0)
            w[p + "qkv.b"] = torch.cat([get(s + f"attention.self.{n}.bias") for n in ("query", "key", "value")], 0)
            w[p + "o.w"], w[p + "o.b"] = get(s + "attention.output.dense.weight"), get(s + "attention.output.dense.bias")
            w[p + "ln1.g"], w[p + "ln1.b"] = get(s + "attention.output.LayerNorm.weight"), get(
                s + "attention.output.LayerNorm.bias")
            w[p + "ff1.w"], w[p + "ff1.b"] = get(s + "intermediate.dense.weight"), get(s + "intermediate.dense.bias")
            w[p + "ff2.w"], w[p + "ff2.b"] = get(s + "output.dense.weight"), get(s + "output.dense.bias")
            w[p + "ln2.g"], w[p + "ln2.b"] = get(s + "output.LayerNorm.weight"), get(s + "output.LayerNorm.bias")
        pw = opt("pooler.dense.weight")
        for cw, cb in (("classifier.weight", "classifier.bias"), ("classifier.out_proj.weight", "classifier.out_proj.bias")):
            if cw in sd:
                w["cls.w"], w["cls.b"] = sd[cw].to(dtype).to(device), sd[cb].to(dtype).to(device)
                cfg.num_labels = w["cls.w"].shape[0]
        if "classifier.dense.weight" in sd:  # RoBERTa classification head: dense -> tanh -> out_proj
            w["pooler.w"], w["pooler.b"] = sd["classifier.dense.weight"].to(dtype).to(device), sd[
                "classifier.dense.bias"].to(dtype).to(device)
            cfg.use_pooler = True
        elif pw is not None and cfg.num_labels > 0:
            w["pooler.w"], w["pooler.b"] = pw, get("pooler.dense.bias")
            cfg.use_pooler = True
        return cls(cfg, w)

    def state_dict_hf(self) -> Dict[str, torch.Tensor]:
        """Inverse of from_state_dict (used by tests and the safetensors writer)."""
        H = self.cfg.hidden_size
        sd = {
            "embeddings.word_embeddings.weight": self.w["emb.word"],
            "embeddings.position_embeddings.weight": self.w["emb.pos"],
            "embeddings.token_type_embeddings.weight": self.w["emb.type"],
            "embeddings.LayerNorm.weight": self.w["emb.ln.g"], "embeddings.LayerNorm.bias": self.w["emb.ln.b"],
        }
        for l in range(self.cfg.num_hidden_layers):
            s, p = f"encoder.layer.{l}.", f"l{l}."
            for i, n in enumerate(("query", "key", "value")):
                sd[s + f"attention.self.{n}.weight"] = self.w[p + "qkv.w"][i * H:(i + 1) * H]
                sd[s + f"attention.self.{n}.bias"] = self.w[p + "qkv.b"][i * H:(i + 1) * H]
            sd[s + "attention.output.dense.weight"], sd[s + "attention.output.dense.bias"] = self.w[p + "o.w"], self.w[p + "o.b"]
            sd[s + "attention.output.LayerNorm.weight"], sd[s + "attention.output.LayerNorm.bias"] = self.w[p + "ln1.g"], self.w[p + "ln1.b"]
            sd[s + "intermediate.dense.weight"], sd[s + "intermediate.dense.bias"] = self.w[p + "ff1.w"], self.w[p + "ff1.b"]
            sd[s + "output.dense.weight"], sd[s + "output.dense.bias"] = self.w[p + "ff2.w"], self.w[p + "ff2.b"]
            sd[s + "output.LayerNorm.weight"], sd[s + "output.LayerNorm.bias"] = self.w[p + "ln2.g"], self.w[p + "ln2.b"]
        if "cls.w" in self.w:
            sd["classifier.weight"], sd["classifier.bias"] = self.w["cls.w"], self.w["cls.b"]
        if "pooler.w" in self.w:
            sd["pooler.dense.weight"], sd["pooler.dense.bias"] = self.w["pooler.w"], self.w["pooler.b"]
        return {k: v.contiguous() for k, v in sd.items()}

    # ------------------------------------------------------------------------------------------------
    def encode(self, b: PackedBatch) -> torch.Tensor:
        """Hidden states of every token, packed: [T, H] bf16."""
        cfg, w = self.cfg, self.w
        H, nh = cfg.hidden_size, cfg.num_attention_heads
        D = H // nh
        x = Dn.bert_embed_ln(b.ids, b.positions, b.type_ids, w["emb.word"], w["emb.pos"], w["emb.type"],
                             w["emb.ln.g"], w["emb.ln.b"], cfg.layer_norm_eps)
        T = x.shape[0]
        if self.tp_size > 1:
            return self._encode_tp(b, x)
        for l in range(cfg.num_hidden_layers):
            p = f"l{l}."
            qkv = Dn.gemm_bf16(x, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            q = qkv[:, :H].view(T, nh, D)
            k = qkv[:, H:2 * H].view(T, nh, D)
            v = qkv[:, 2 * H:].view(T, nh, D)
            ctx = A.varlen_attention(q, k, v, b.starts, b.lens, b.max_len).view(T, H)
            h = Dn.gemm_bf16(ctx, w[p + "o.w"], bias=w[p + "o.b"], residual=x)
            x = Dn.norm(h, w[p + "ln1.g"], w[p + "ln1.b"], eps=cfg.layer_norm_eps)
            f = Dn.gemm_bf16(x, w[p + "ff1.w"], bias=w[p + "ff1.b"], act=cfg.hidden_act)
            h = Dn.gemm_bf16(f, w[p + "ff2.w"], bias=w[p + "ff2.b"], residual=x)
            x = Dn.norm(h, w[p + "ln2.g"], w[p + "ln2.b"], eps=cfg.layer_norm_eps)
        return x

    def _encode_tp(self, b: PackedBatch, x: torch.Tensor) -> torch.Tensor:
        """Tensor-parallel layers: local heads / local FFN slice, two all-reduces per layer (fp32 partial sums, so
        the result does not depend on how a bf16 rounding of each rank's partial would fall)."""
        cfg, w = self.cfg, self.w
        H, nh = cfg.hidden_size, cfg.num_attention_heads
        D, hs, nl = H // nh, H // self.tp_size, nh // self.tp_size
        T = x.shape[0]
        for l in range(cfg.num_hidden_layers):
            p = f"l{l}."
            qkv = Dn.gemm_bf16(x, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            q, k, v = (qkv[:, i * hs:(i + 1) * hs].view(T, nl, D) for i in range(3))
            ctx = A.varlen_attention(q, k, v, b.starts, b.lens, b.max_len).view(T, hs)
            part = Dn.gemm_bf16(ctx, w[p + "o.w"], out_dtype=torch.float32)
            part = self.comm.all_reduce(part)
            h = (part + w[p + "o.b"].float() + x.float()).to(x.dtype)
            x = Dn.norm(h, w[p + "ln1.g"], w[p + "ln1.b"], eps=cfg.layer_norm_eps)
            f = Dn.gemm_bf16(x, w[p + "ff1.w"], bias=w[p + "ff1.b"], act=cfg.hidden_act)
            part = self.comm.all_reduce(Dn.gemm_bf16(f, w[p + "ff2.w"], out_dtype=torch.float32))
            h = (part + w[p + "ff2.b"].float() + x.float()).to(x.dtype)
            x = Dn.norm(h, w[p + "ln2.g"], w[p + "ln2.b"], eps=cfg.layer_norm_eps)
        return x

    def embed(self, b: PackedBatch, pooling: Optional[str] = None, normalize: bool = True) -> torch.Tensor:
        """Sentence embeddings, fp32 [B, H]."""
        h = self.encode(b)
        return Dn.pool(h, b.starts, b.lens, mode=pooling or self.cfg.pooling, normalize=normalize)

    def classify(self, b: PackedBatch) -> torch.Tensor:
        """Sequence-classification logits, fp32 [B, num_labels] (cross-encoder head on [CLS])."""
        assert "cls.w" in self.w, "model has no classification head"
        h = self.encode(b)
        cls = Dn.pool(h, b.starts, b.lens, mode="cls", normalize=False).to(h.dtype)
        if "pooler.w" in self.w:
            # tanh is not a GEMM epilogue; B x H is tiny, do it in torch.
            cls = torch.tanh(Dn.gemm_bf16(cls, self.w["pooler.w"], bias=self.w["pooler.b"],
                                          out_dtype=torch.float32)).to(h.dtype)
        return Dn.gemm_bf16(cls, self.w["cls.w"], bias=self.w["cls.b"], out_dtype=torch.float32)

    def token_logits(self, b: PackedBatch) -> torch.Tensor:
        """Token-classification logits, fp32 [T, num_labels] (the classifier applied to every token's hidden
        state, no pooler): NER / chunk-boundary heads."""
        assert "cls.w" in self.w, "model has no classification head"
        h = self.encode(b)
        return Dn.gemm_bf16(h, self.w["cls.w"], bias=self.w["cls.b"], out_dtype=torch.float32)

    def param_count(self) -> int:
        return sum(t.numel() for t in self.w.values())

    def flops_per_token(self, avg_len: float) -> float:
        c = self.cfg
        H, F = c.hidden_size, c.intermediate_size
        return c.num_hidden_layers * (2 * (4 * H * H + 2 * H * F) + 4 * avg_len * H)
