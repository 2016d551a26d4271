"""Optical character recognition with a vision encoder-decoder: a ViT encoder over image patches and the TrOCR
text decoder attending to the patch states (the ``readers`` task of the reference: zig/pkg/inference/src/pipelines/
ocr_multistage.zig and the vision2seq pipeline of go/pkg/termite/lib/pipelines/vision2seq.go).

* ViT: stride-``patch`` convolution as one GEMM over unfolded patches, class token, learned positions, pre-LayerNorm
  blocks (``layernorm_before`` / ``layernorm_after``), final LayerNorm; attention is the packed bidirectional flash
  kernel, the rest the shared GEMM / LayerNorm kernels.
* TrOCR decoder: BART-style post-LayerNorm blocks whose cross-attention keys / values are projected from the
  encoder width (which may differ from the decoder's), learned positions with the two-row offset or fairseq
  sinusoidal positions, optional embedding LayerNorm and sqrt(d) embedding scale, an un-biased output projection.
Weight names are the Hugging Face ``VisionEncoderDecoderModel`` ones (``encoder.*`` ViT, ``decoder.model.decoder.*``,
``decoder.output_projection``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import torch

from ..ops import attention as A
from ..ops import dense as Dn


@dataclass
class VitConfig:
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    image_size: int = 384
    patch_size: int = 16
    num_channels: int = 3
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"
    qkv_bias: bool = True


@dataclass
class TrOCRDecoderConfig:
    vocab_size: int = 50265
    d_model: int = 1024
    decoder_layers: int = 12
    decoder_attention_heads: int = 16
    decoder_ffn_dim: int = 4096
    activation_function: str = "gelu"
    max_position_embeddings: int = 512
    use_learned_position_embeddings: bool = True
    layernorm_embedding: bool = True
    scale_embedding: bool = False
    decoder_start_token_id: int = 2
    eos_token_id: int = 2
    pad_token_id: int = 1


@dataclass
class TrOCRConfig:
    encoder: VitConfig = field(default_factory=VitConfig)
    decoder: TrOCRDecoderConfig = field(default_factory=TrOCRDecoderConfig)

    @classmethod
    def from_hf(cls, d: dict) -> "TrOCRConfig":
        def pick(klass, src):
            keys = set(klass.__dataclass_fields__)
            return klass(**{k: v for k, v in (src or {}).items() if k in keys and v is not None})

        cfg = cls(pick(VitConfig, d.get("encoder")), pick(TrOCRDecoderConfig, d.get("decoder")))
        for k in ("decoder_start_token_id", "eos_token_id", "pad_token_id"):
            if d.get(k) is not None:
                setattr(cfg.decoder, k, d[k])
        return cfg


class TrOCRModel:
    def __init__(self, cfg: TrOCRConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["dec.embed"].device

    @classmethod
    def from_state_dict(cls, cfg: TrOCRConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "TrOCRModel":
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}
        e, vc = "encoder.", cfg.encoder
        w["enc.patch.w"] = t(sd[e + "embeddings.patch_embeddings.projection.weight"].reshape(vc.hidden_size, -1))
        w["enc.patch.b"] = t(sd[e + "embeddings.patch_embeddings.projection.bias"])
        w["enc.cls"] = t(sd[e + "embeddings.cls_token"].reshape(1, -1))
        w["enc.pos"] = t(sd[e + "embeddings.position_embeddings"].reshape(-1, vc.hidden_size))
        zeros = torch.zeros(vc.hidden_size)
        for l in range(vc.num_hidden_layers):
            s, p = f"{e}encoder.layer.{l}.", f"enc.l{l}."
            a = s + "attention.attention."
            w[p + "qkv.w"] = t(torch.cat([sd[a + f"{n}.weight"] for n in ("query", "key", "value")], 0))
            w[p + "qkv.b"] = t(torch.cat([sd.get(a + f"{n}.bias", zeros) for n in ("query", "key", "value")], 0))
            w[p + "o.w"], w[p + "o.b"] = t(sd[s + "attention.output.dense.weight"]), t(sd[s + "attention.output.dense.bias"])
            w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "layernorm_before.weight"]), t(sd[s + "layernorm_before.bias"])
            w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "layernorm_after.weight"]), t(sd[s + "layernorm_after.bias"])
            w[p + "fc1.w"], w[p + "fc1.b"] = t(sd[s + "intermediate.dense.weight"]), t(sd[s + "intermediate.dense.bias"])
            w[p + "fc2.w"], w[p + "fc2.b"] = t(sd[s + "output.dense.weight"]), t(sd[s + "output.dense.bias"])
        w["enc.lnf.g"], w["enc.lnf.b"] = t(sd[e + "layernorm.weight"]), t(sd[e + "layernorm.bias"])
        d, dc = "decoder.model.decoder.", cfg.decoder
        w["dec.embed"] = t(sd[d + "embed_tokens.weight"])
        if dc.use_learned_position_embeddings:
            w["dec.pos"] = t(sd[d + "embed_positions.weight"])
        if dc.layernorm_embedding:
            w["dec.lne.g"], w["dec.lne.b"] = t(sd[d + "layernorm_embedding.weight"]), t(sd[d + "layernorm_embedding.bias"])
        for l in range(dc.decoder_layers):
            s, p = f"{d}layers.{l}.", f"dec.l{l}."
            w[p + "sa.qkv.w"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0))
            w[p + "sa.qkv.b"] = t(torch.cat([sd[s + f"self_attn.{n}_proj.bias"] for n in "qkv"], 0))
            w[p + "sa.o.w"], w[p + "sa.o.b"] = t(sd[s + "self_attn.out_proj.weight"]), t(sd[s + "self_attn.out_proj.bias"])
            w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s + "self_attn_layer_norm.weight"]), t(sd[s + "self_attn_layer_norm.bias"])
            w[p + "ca.q.w"], w[p + "ca.q.b"] = t(sd[s + "encoder_attn.q_proj.weight"]), t(sd[s + "encoder_attn.q_proj.bias"])
            w[p + "ca.kv.w"] = t(torch.cat([sd[s + "encoder_attn.k_proj.weight"], sd[s + "encoder_attn.v_proj.weight"]], 0))
            w[p + "ca.kv.b"] = t(torch.cat([sd[s + "encoder_attn.k_proj.bias"], sd[s + "encoder_attn.v_proj.bias"]], 0))
            w[p + "ca.o.w"], w[p + "ca.o.b"] = t(sd[s + "encoder_attn.out_proj.weight"]), t(sd[s + "encoder_attn.out_proj.bias"])
            w[p + "lnc.g"], w[p + "lnc.b"] = t(sd[s + "encoder_attn_layer_norm.weight"]), t(sd[s + "encoder_attn_layer_norm.bias"])
            w[p + "fc1.w"], w[p + "fc1.b"] = t(sd[s + "fc1.weight"]), t(sd[s + "fc1.bias"])
            w[p + "fc2.w"], w[p + "fc2.b"] = t(sd[s + "fc2.weight"]), t(sd[s + "fc2.bias"])
            w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s + "final_layer_norm.weight"]), t(sd[s + "final_layer_norm.bias"])
        w["dec.out"] = t(sd["decoder.output_projection.weight"])
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        """Preprocessed pixels [3, S, S] -> patch states [1 + (S / patch)^2, hidden]."""
        vc, w = self.cfg.encoder, self.w
        C, S, _ = pixels.shape
        P, H, nh = vc.patch_size, vc.hidden_size, vc.num_attention_heads
        g, D = S // P, H // nh
        dt = w["enc.patch.w"].dtype
        patches = pixels.to(self.device).to(dt).view(C, g, P, g, P).permute(1, 3, 0, 2, 4).reshape(g * g, C * P * P)
        x = torch.cat([w["enc.cls"], Dn.gemm_bf16(patches.contiguous(), w["enc.patch.w"], bias=w["enc.patch.b"])])
        T = x.shape[0]
        x = (x.float() + w["enc.pos"][:T].float()).to(dt).contiguous()
        starts = torch.zeros(1, dtype=torch.int32, device=self.device)
        lens = torch.full((1,), T, dtype=torch.int32, device=self.device)
        for l in range(vc.num_hidden_layers):
            p = f"enc.l{l}."
            h = Dn.norm(x, w[p + "ln1.g"], w[p + "ln1.b"], eps=vc.layer_norm_eps)
            qkv = Dn.gemm_bf16(h, w[p + "qkv.w"], bias=w[p + "qkv.b"])
            ctx = A.varlen_attention(qkv[:, :H].view(T, nh, D), qkv[:, H:2 * H].view(T, nh, D),
                                     qkv[:, 2 * H:].view(T, nh, D), starts, lens, T).view(T, H)
            x = Dn.gemm_bf16(ctx, w[p + "o.w"], bias=w[p + "o.b"], residual=x)
            h = Dn.norm(x, w[p + "ln2.g"], w[p + "ln2.b"], eps=vc.layer_norm_eps)
            m = Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=vc.hidden_act)
            x = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
        return Dn.norm(x, w["enc.lnf.g"], w["enc.lnf.b"], eps=vc.layer_norm_eps)

    def _positions(self, first: int, n: int) -> torch.Tensor:
        dc, w = self.cfg.decoder, self.w
        if "dec.pos" in w:
            return w["dec.pos"][first + 2: first + 2 + n].float()
        half = dc.d_model // 2
        freq = torch.exp(torch.arange(half, dtype=torch.float32) * -(math.log(10000) / (half - 1)))
        pos = torch.arange(first, first + n, dtype=torch.float32) + dc.pad_token_id + 1
        ang = pos[:, None] * freq[None, :]
        emb = torch.cat([ang.sin(), ang.cos()], 1)
        if dc.d_model % 2:
            emb = torch.nn.functional.pad(emb, (0, 1))
        return emb.to(self.device)

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

    def start_decoding(self, enc: torch.Tensor) -> dict:
        H = self.cfg.decoder.d_model
        cross = [Dn.gemm_bf16(enc, self.w[f"dec.l{l}.ca.kv.w"], bias=self.w[f"dec.l{l}.ca.kv.b"])
                 for l in range(self.cfg.decoder.decoder_layers)]
        return {"cross": [(c[:, :H], c[:, H:]) for c in cross], "k": [None] * len(cross), "v": [None] * len(cross),
                "len": 0}

    def decode(self, state: dict, ids: Sequence[int]) -> torch.Tensor:
        dc, w = self.cfg.decoder, self.w
        H, nh = dc.d_model, dc.decoder_attention_heads
        n0, n = state["len"], len(ids)
        tok = torch.tensor(list(ids), device=self.device)
        scale = math.sqrt(H) if dc.scale_embedding else 1.0
        x = (w["dec.embed"].index_select(0, tok).float() * scale + self._positions(n0, n)).to(w["dec.embed"].dtype)
        if "dec.lne.g" in w:
            x = Dn.norm(x, w["dec.lne.g"], w["dec.lne.b"], eps=1e-5)
        for l in range(dc.decoder_layers):
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
            x = Dn.norm(h, w[p + "lnc.g"], w[p + "lnc.b"], eps=1e-5)
            m = Dn.gemm_bf16(x, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=dc.activation_function)
            h = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
            x = Dn.norm(h, w[p + "ln2.g"], w[p + "ln2.b"], eps=1e-5)
        state["len"] = n0 + n
        return Dn.gemm_bf16(x, w["dec.out"], out_dtype=torch.float32).float()

    def read_ids(self, pixels: torch.Tensor, max_new_tokens: int = 64) -> List[int]:
        """Greedy decoding of the text in one preprocessed image."""
        dc = self.cfg.decoder
        state = self.start_decoding(self.encode(pixels))
        tok, out = dc.decoder_start_token_id, []
        for _ in range(min(max_new_tokens, dc.max_position_embeddings - 1)):
            tok = int(self.decode(state, [tok])[-1].argmax())
            if tok == dc.eos_token_id:
                break
            out.append(tok)
        return out
