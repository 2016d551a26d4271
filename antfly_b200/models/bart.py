"""BART encoder-decoder (summarisation / rewriting checkpoints, and REBEL-style relation extraction, which is a
BART fine-tune that writes triplets as text).

Post-LayerNorm blocks with biased linears and GELU; learned position embeddings whose table is offset by two rows;
a LayerNorm on the embeddings; optional sqrt(d_model) embedding scale; the output projection is the shared
embedding plus a per-token logit bias.  The reference runs this family through its encoder-decoder pipeline
(zig/pkg/inference/src/pipelines/encoder_decoder.zig; REBEL parsing in pipelines/rebel.zig).  Same execution split
as the other encoder-decoders here: projections / MLPs / norms are the shared GEMM and LayerNorm kernels with bias,
GELU and residual in epilogues, encoder self attention is the packed flash kernel, the one-token decoder attention
products are tensor ops over cached keys / values.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import attention as A
from ..ops import dense as Dn


@dataclass
class BartConfig:
    vocab_size: int = 50265
    d_model: int = 1024
    encoder_layers: int = 12
    decoder_layers: int = 12
    encoder_attention_heads: int = 16
    decoder_attention_heads: int = 16
    encoder_ffn_dim: int = 4096
    decoder_ffn_dim: int = 4096
    max_position_embeddings: int = 1024
    activation_function: str = "gelu"
    scale_embedding: bool = False
    decoder_start_token_id: int = 2
    eos_token_id: int = 2
    bos_token_id: int = 0
    pad_token_id: int = 1
    forced_bos_token_id: int = -1

    @classmethod
    def from_hf(cls, d: dict) -> "BartConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys and v is not None})


class BartModel:
    """Interface of :class:`antfly_b200.models.t5.T5Model` (``encode``, ``start_decoding``, ``decode``,
    ``generate``), so the text-to-text pipeline drives either."""

    def __init__(self, cfg: BartConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["shared"].device
        self.scale = math.sqrt(cfg.d_model) if cfg.scale_embedding else 1.0

    @classmethod
    def from_state_dict(cls, cfg: BartConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "BartModel":
        pre = "model." if any(k.startswith("model.") for k in sd) else ""
        t = lambda x: x.to(dtype).to(device).contiguous()
        shared = sd.get(pre + "shared.weight", sd.get(pre + "encoder.embed_tokens.weight"))
        w: Dict[str, torch.Tensor] = {"shared": t(shared)}
        if "final_logits_bias" in sd:
            w["logit_bias"] = t(sd["final_logits_bias"].reshape(-1))

        def attn(dst: str, src: str, fused: bool) -> None:
            names = ("q", "k", "v")
            if fused:
                w[dst + "qkv.w"] = t(torch.cat([sd[src + f"{n}_proj.weight"] for n in names], 0))
                w[dst + "qkv.b"] = t(torch.cat([sd[src + f"{n}_proj.bias"] for n in names], 0))
            else:
                w[dst + "q.w"], w[dst + "q.b"] = t(sd[src + "q_proj.weight"]), t(sd[src + "q_proj.bias"])
                w[dst + "kv.w"] = t(torch.cat([sd[src + "k_proj.weight"], sd[src + "v_proj.weight"]], 0))
                w[dst + "kv.b"] = t(torch.cat([sd[src + "k_proj.bias"], sd[src + "v_proj.bias"]], 0))
            w[dst + "o.w"], w[dst + "o.b"] = t(sd[src + "out_proj.weight"]), t(sd[src + "out_proj.bias"])

        for stack, n in (("encoder", cfg.encoder_layers), ("decoder", cfg.decoder_layers)):
            s0, p0 = f"{pre}{stack}.", stack[:3] + "."
            w[p0 + "pos"] = t(sd[s0 + "embed_positions.weight"])
            w[p0 + "lne.g"], w[p0 + "lne.b"] = t(sd[s0 + "layernorm_embedding.weight"]), t(
                sd[s0 + "layernorm_embedding.bias"])
            for l in range(n):
                s, p = f"{s0}layers.{l}.", f"{p0}l{l}."
                attn(p + "sa.", s + "self_attn.", True)
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "self_attn_layer_norm.weight"]), t(
                    sd[s + "self_attn_layer_norm.bias"])
                if stack == "decoder":
                    attn(p + "ca.", s + "encoder_attn.", False)
                    w[p + "lnc.g"], w[p + "lnc.b"] = t(sd[s + "encoder_attn_layer_norm.weight"]), t(
                        sd[s + "encoder_attn_layer_norm.bias"])
                w[p + "fc1.w"], w[p + "fc1.b"] = t(sd[s + "fc1.weight"]), t(sd[s + "fc1.bias"])
                w[p + "fc2.w"], w[p + "fc2.b"] = t(sd[s + "fc2.weight"]), t(sd[s + "fc2.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "final_layer_norm.weight"]), t(
                    sd[s + "final_layer_norm.bias"])
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def _embed(self, ids: Optional[Sequence[int]], first_pos: int, stack: str,
               token_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Token rows (scaled) + learned positions -> LayerNorm.  ``token_embeds`` [T, d_model] replaces the table
        lookup (already scaled): a caller that mixes in rows of another modality builds them itself."""
        w = self.w
        if token_embeds is None:
            tok = torch.tensor(list(ids), device=self.device)
            token_embeds = w["shared"].index_select(0, tok).float() * self.scale
        n = token_embeds.shape[0]
        pos = torch.arange(first_pos, first_pos + n, device=self.device) + 2             # the table's two-row offset
        x = token_embeds.float() + w[stack + ".pos"].index_select(0, pos).float()
        return Dn.norm(x.to(w["shared"].dtype), w[stack + ".lne.g"], w[stack + ".lne.b"], eps=1e-5)

    def _attend(self, q, k, v, nh: int, causal: bool) -> torch.Tensor:
        D = q.shape[1] // nh
        qq = q.float().view(-1, nh, D).transpose(0, 1)
        kk = k.float().view(-1, nh, D).transpose(0, 1)
        vv = v.float().view(-1, nh, D).transpose(0, 1)
        sc = qq @ kk.transpose(1, 2) / math.sqrt(D)
        if causal and sc.shape[1] > 1:
            Lq, Lk = sc.shape[1], sc.shape[2]
            sc = sc.masked_fill(~torch.ones(Lq, Lk, dtype=torch.bool, device=sc.device).tril(Lk - Lq), float("-inf"))
        return (sc.softmax(-1) @ vv).transpose(0, 1).reshape(-1, nh * D).to(q.dtype)

    def _ffn(self, x, p):
        w = self.w
        m = Dn.gemm_bf16(x, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=self.cfg.activation_function)
        h = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
        return Dn.norm(h, w[p + "ln2.g"], w[p + "ln2.b"], eps=1e-5)

    def encode(self, ids: Optional[Sequence[int]], token_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        H, nh = cfg.d_model, cfg.encoder_attention_heads
        D = H // nh
        x = self._embed(ids, 0, "enc", token_embeds)
        T = x.shape[0]
        starts = torch.zeros(1, dtype=torch.int32, device=self.device)
        lens = torch.full((1,), T, dtype=torch.int32, device=self.device)
        for l in range(cfg.encoder_layers):
            p = f"enc.l{l}."
            qkv = Dn.gemm_bf16(x, w[p + "sa.qkv.w"], bias=w[p + "sa.qkv.b"])
            ctx = A.varlen_attention(qkv[:, :H].view(T, nh, D), qkv[:, H:2 * H].view(T, nh, D),
                                     qkv[:, 2 * H:].view(T, nh, D), starts, lens, T).view(T, H)
            h = Dn.gemm_bf16(ctx, w[p + "sa.o.w"], bias=w[p + "sa.o.b"], residual=x)
            x = self._ffn(Dn.norm(h, w[p + "ln1.g"], w[p + "ln1.b"], eps=1e-5), p)
        return x

    def start_decoding(self, enc: torch.Tensor) -> dict:
        H = self.cfg.d_model
        cross = [Dn.gemm_bf16(enc, self.w[f"dec.l{l}.ca.kv.w"], bias=self.w[f"dec.l{l}.ca.kv.b"])
                 for l in range(self.cfg.decoder_layers)]
        return {"cross": [(c[:, :H], c[:, H:]) for c in cross], "k": [None] * len(cross), "v": [None] * len(cross),
                "len": 0}

    def decode(self, state: dict, ids: Sequence[int]) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        H, nh = cfg.d_model, cfg.decoder_attention_heads
        n0 = state["len"]
        x = self._embed(ids, n0, "dec")
        for l in range(cfg.decoder_layers):
            p = f"dec.l{l}."
            qkv = Dn.gemm_bf16(x, w[p + "sa.qkv.w"], bias=w[p + "sa.qkv.b"])
            k, v = qkv[:, H:2 * H], qkv[:, 2 * H:]
            if state["k"][l] is not None:
                k, v = torch.cat([state["k"][l], k]), torch.cat([state["v"][l], v])
            state["k"][l], state["v"][l] = k, v
            h = Dn.gemm_bf16(self._attend(qkv[:, :H], k, v, nh, True), w[p + "sa.o.w"], bias=w[p + "sa.o.b"],
                             residual=x)
            x = Dn.norm(h, w[p + "ln1.g"], w[p + "ln1.b"], eps=1e-5)
            q = Dn.gemm_bf16(x, w[p + "ca.q.w"], bias=w[p + "ca.q.b"])
            ck, cv = state["cross"][l]
            h = Dn.gemm_bf16(self._attend(q, ck, cv, nh, False), w[p + "ca.o.w"], bias=w[p + "ca.o.b"], residual=x)
            x = self._ffn(Dn.norm(h, w[p + "lnc.g"], w[p + "lnc.b"], eps=1e-5), p)
        state["len"] = n0 + len(ids)
        logits = Dn.gemm_bf16(x, w["shared"], out_dtype=torch.float32).float()
        return logits + w["logit_bias"].float() if "logit_bias" in w else logits

    def generate(self, ids: Sequence[int], max_new_tokens: int = 64) -> List[int]:
        """Greedy decoding from the start token (and the forced first token, if the checkpoint has one)."""
        cfg = self.cfg
        state = self.start_decoding(self.encode(ids))
        prefix = [cfg.decoder_start_token_id] + ([cfg.forced_bos_token_id] if cfg.forced_bos_token_id >= 0 else [])
        logits = self.decode(state, prefix)[-1]
        out: List[int] = []
        for _ in range(max_new_tokens):
            tok = int(logits.argmax())
            if tok == cfg.eos_token_id:
                break
            out.append(tok)
            logits = self.decode(state, [tok])[-1]
        return out
