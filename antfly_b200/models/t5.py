"""T5 / Flan-T5 encoder-decoder (text-to-text: query rewriting, summarisation, extraction prompts).

Pre-RMSNorm blocks without biases; attention scores are *not* scaled by 1 / sqrt(D) and carry a learned bias per
head indexed by the bucketed relative distance (the table lives in the first block of each stack and is shared by
the others; bidirectional buckets in the encoder, causal ones in the decoder, none for cross attention); the FFN is
ReLU (original) or gated GELU (v1.1 / Flan); with tied embeddings the decoder output is scaled by d_model^-0.5
before the vocabulary projection.  The reference's version is zig/pkg/inference/src/architectures/t5.zig driven by
pipelines/encoder_decoder.zig (greedy decoding with cached self- and cross-attention keys / values).

Execution: all projections, FFN GEMMs and norms are the shared kernels (tcgen05 GEMM with ReLU / GELU / residual
epilogues, RMSNorm); the attention core with its additive bias is tensor ops per sequence.  Decoding keeps the
self-attention keys / values of generated tokens and the cross-attention keys / values of the encoder output, so a
step costs one token's projections.  Sequences are handled one at a time (this family serves short rewriting
prompts, not the batch-throughput path).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import dense as Dn
from ..ops import reference as R


@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 512
    d_kv: int = 64
    d_ff: int = 2048
    num_layers: int = 6
    num_decoder_layers: Optional[int] = None
    num_heads: int = 8
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6
    feed_forward_proj: str = "relu"
    tie_word_embeddings: bool = True
    scale_decoder_outputs: Optional[bool] = None   # None: scale exactly when the embeddings are tied
    decoder_start_token_id: int = 0
    eos_token_id: int = 1
    pad_token_id: int = 0

    @classmethod
    def from_hf(cls, d: dict) -> "T5Config":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys and v is not None})

    @property
    def gated(self) -> bool:
        return self.feed_forward_proj.startswith("gated")

    @property
    def act(self) -> str:
        a = self.feed_forward_proj.split("-")[-1]
        return {"gelu": "gelu_new" if self.gated else "gelu"}.get(a, a)


def relative_bucket(rel: torch.Tensor, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bucket of ``key - query`` distances: exact for small ones, logarithmic up to max_distance; the encoder
    spends half of the buckets on each direction, the decoder all of them on the past."""
    out = torch.zeros_like(rel)
    if bidirectional:
        num_buckets //= 2
        out = out + (rel > 0).long() * num_buckets
        rel = rel.abs()
    else:
        rel = -torch.clamp(rel, max=0)
    max_exact = num_buckets // 2
    large = max_exact + (torch.log(rel.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact)
                         * (num_buckets - max_exact)).long()
    large = torch.clamp(large, max=num_buckets - 1)
    return out + torch.where(rel < max_exact, rel, large)


class T5Model:
    def __init__(self, cfg: T5Config, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["shared"].device
        self.n_dec = cfg.num_decoder_layers if cfg.num_decoder_layers is not None else cfg.num_layers

    @classmethod
    def from_state_dict(cls, cfg: T5Config, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "T5Model":
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {"shared": t(sd["shared.weight"] if "shared.weight" in sd
                                                  else sd["encoder.embed_tokens.weight"])}
        n_dec = cfg.num_decoder_layers if cfg.num_decoder_layers is not None else cfg.num_layers

        def attn(dst: str, src: str, fuse_qkv: bool) -> None:
            if fuse_qkv:
                w[dst + "qkv"] = t(torch.cat([sd[src + f"{n}.weight"] for n in ("q", "k", "v")], 0))
            else:
                w[dst + "q"] = t(sd[src + "q.weight"])
                w[dst + "kv"] = t(torch.cat([sd[src + "k.weight"], sd[src + "v.weight"]], 0))
            w[dst + "o"] = t(sd[src + "o.weight"])

        def ffn(dst: str, src: str) -> None:
            if cfg.gated:
                w[dst + "wi"] = t(torch.cat([sd[src + "wi_0.weight"], sd[src + "wi_1.weight"]], 0))
            else:
                w[dst + "wi"] = t(sd[src + "wi.weight"])
            w[dst + "wo"] = t(sd[src + "wo.weight"])

        for stack, n, ff_idx in (("encoder", cfg.num_layers, 1), ("decoder", n_dec, 2)):
            for l in range(n):
                s, p = f"{stack}.block.{l}.layer.", f"{stack[:3]}.l{l}."
                attn(p + "sa.", s + "0.SelfAttention.", True)
                w[p + "ln1"] = t(sd[s + "0.layer_norm.weight"])
                if stack == "decoder":
                    attn(p + "ca.", s + "1.EncDecAttention.", False)
                    w[p + "lnc"] = t(sd[s + "1.layer_norm.weight"])
                ffn(p + "ff.", s + f"{ff_idx}.DenseReluDense.")
                w[p + "ln2"] = t(sd[s + f"{ff_idx}.layer_norm.weight"])
            w[f"{stack[:3]}.bias"] = sd[f"{stack}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"].float().to(
                device)                                                     # [buckets, heads]
            w[f"{stack[:3]}.lnf"] = t(sd[f"{stack}.final_layer_norm.weight"])
        if "lm_head.weight" in sd and (not cfg.tie_word_embeddings or cfg.scale_decoder_outputs is False) and \
                not torch.equal(sd["lm_head.weight"], sd.get("shared.weight", sd["lm_head.weight"][:0])):
            w["lm_head"] = t(sd["lm_head.weight"])
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def _norm(self, x, g):
        return Dn.norm(x, g, None, eps=self.cfg.layer_norm_epsilon, rms=True)

    def _bias(self, stack: str, q_pos: torch.Tensor, k_pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        b = relative_bucket(k_pos[None, :] - q_pos[:, None], stack == "enc", cfg.relative_attention_num_buckets,
                            cfg.relative_attention_max_distance)
        return self.w[stack + ".bias"][b].permute(2, 0, 1)                # [heads, Lq, Lk]

    def _attend(self, q, k, v, bias=None, causal=False):
        """q [Lq, nh * dk], k / v [Lk, nh * dk] -> [Lq, nh * dk]; scores are unscaled."""
        nh, dk = self.cfg.num_heads, self.cfg.d_kv
        qq = q.float().view(-1, nh, dk).transpose(0, 1)
        kk = k.float().view(-1, nh, dk).transpose(0, 1)
        vv = v.float().view(-1, nh, dk).transpose(0, 1)
        sc = qq @ kk.transpose(1, 2)
        if bias is not None:
            sc = sc + bias
        if causal and sc.shape[1] > 1:
            Lq, Lk = sc.shape[1], sc.shape[2]
            m = torch.ones(Lq, Lk, dtype=torch.bool, device=sc.device).tril(Lk - Lq)
            sc = sc.masked_fill(~m, float("-inf"))
        return (sc.softmax(-1) @ vv).transpose(0, 1).reshape(-1, nh * dk).to(q.dtype)

    def _ffn(self, x, p):
        cfg, w = self.cfg, self.w
        if cfg.gated:
            ag = Dn.gemm_bf16(x, w[p + "wi"])
            F = ag.shape[1] // 2
            h = Dn.gated_act(ag, cfg.act)
        else:
            h = Dn.gemm_bf16(x, w[p + "wi"], act=cfg.act)
        return h

    def encode(self, ids: Sequence[int]) -> torch.Tensor:
        """Encoder hidden states of one sequence: [L, d_model]."""
        cfg, w = self.cfg, self.w
        inner = cfg.num_heads * cfg.d_kv
        x = w["shared"].index_select(0, torch.tensor(list(ids), device=self.device))
        pos = torch.arange(len(ids), device=self.device)
        bias = self._bias("enc", pos, pos)
        for l in range(cfg.num_layers):
            p = f"enc.l{l}."
            qkv = Dn.gemm_bf16(self._norm(x, w[p + "ln1"]), w[p + "sa.qkv"])
            ctx = self._attend(qkv[:, :inner], qkv[:, inner:2 * inner], qkv[:, 2 * inner:], bias)
            x = Dn.gemm_bf16(ctx, w[p + "sa.o"], residual=x)
            x = Dn.gemm_bf16(self._ffn(self._norm(x, w[p + "ln2"]), p + "ff."), w[p + "ff.wo"], residual=x)
        return self._norm(x, w["enc.lnf"])

    def start_decoding(self, enc: torch.Tensor) -> dict:
        """Per-sequence decoder state: cross-attention keys / values of every layer, empty self-attention caches."""
        w, inner = self.w, self.cfg.num_heads * self.cfg.d_kv
        cross = [Dn.gemm_bf16(enc, w[f"dec.l{l}.ca.kv"]) for l in range(self.n_dec)]
        return {"cross": [(c[:, :inner], c[:, inner:]) for c in cross], "k": [None] * self.n_dec,
                "v": [None] * self.n_dec, "len": 0}

    def decode(self, state: dict, ids: Sequence[int]) -> torch.Tensor:
        """Feed the next decoder token(s); returns fp32 logits [len(ids), vocab] and extends the caches."""
        cfg, w = self.cfg, self.w
        inner = cfg.num_heads * cfg.d_kv
        x = w["shared"].index_select(0, torch.tensor(list(ids), device=self.device))
        n0, n = state["len"], len(ids)
        q_pos = torch.arange(n0, n0 + n, device=self.device)
        bias = self._bias("dec", q_pos, torch.arange(n0 + n, device=self.device))
        for l in range(self.n_dec):
            p = f"dec.l{l}."
            qkv = Dn.gemm_bf16(self._norm(x, w[p + "ln1"]), w[p + "sa.qkv"])
            k, v = qkv[:, inner:2 * inner], qkv[:, 2 * inner:]
            if state["k"][l] is not None:
                k, v = torch.cat([state["k"][l], k]), torch.cat([state["v"][l], v])
            state["k"][l], state["v"][l] = k, v
            ctx = self._attend(qkv[:, :inner], k, v, bias, causal=True)
            x = Dn.gemm_bf16(ctx, w[p + "sa.o"], residual=x)
            q = Dn.gemm_bf16(self._norm(x, w[p + "lnc"]), w[p + "ca.q"])
            ck, cv = state["cross"][l]
            x = Dn.gemm_bf16(self._attend(q, ck, cv), w[p + "ca.o"], residual=x)
            x = Dn.gemm_bf16(self._ffn(self._norm(x, w[p + "ln2"]), p + "ff."), w[p + "ff.wo"], residual=x)
        state["len"] = n0 + n
        h = self._norm(x, w["dec.lnf"])
        # The original T5 (tied embeddings) scales the decoder output before the vocabulary projection; v1.1 / Flan
        # checkpoints (config says untied, with or without a separate lm_head tensor) do not.
        scaled = cfg.scale_decoder_outputs if cfg.scale_decoder_outputs is not None else cfg.tie_word_embeddings
        return Dn.gemm_bf16(h, w.get("lm_head", w["shared"]), out_dtype=torch.float32,
                            alpha=cfg.d_model ** -0.5 if scaled else 1.0)

    def generate(self, ids: Sequence[int], max_new_tokens: int = 64) -> List[int]:
        """Greedy text-to-text generation for one input sequence (token ids without the start token)."""
        state = self.start_decoding(self.encode(ids))
        tok, out = self.cfg.decoder_start_token_id, []
        for _ in range(max_new_tokens):
            tok = int(self.decode(state, [tok])[-1].argmax())
            if tok == self.cfg.eos_token_id:
                break
            out.append(tok)
        return out
