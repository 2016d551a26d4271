"""Whisper speech-to-text: a convolutional stem + pre-LayerNorm transformer encoder over 30 s of log-mel features,
and a pre-LayerNorm decoder with cached self attention and cross attention to the encoder output.

The reference implements it in zig/pkg/inference/src/architectures/whisper.zig with the transcription pipeline in
pipelines/transcription.zig (greedy decoding from the forced ``<|startoftranscript|> <|lang|> <|transcribe|>
<|notimestamps|>`` prompt).  Execution here:

* the two 1-D convolutions of the stem (kernel 3, the second with stride 2) are GEMMs over unfolded windows
  ([frames, 3 * channels] x [out, 3 * channels]) with the GELU in the GEMM epilogue -- the tensor-core form of the
  reference's direct convolution kernel (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:652);
* encoder self attention is the packed bidirectional flash kernel over the 1500 frames; projections, MLPs and
  LayerNorms are the shared GEMM / norm kernels (bias, GELU and residual in epilogues);
* decoder steps are one token wide: self-attention keys / values are appended to a cache, cross-attention keys /
  values are projected once per utterance; the small attention products are tensor ops.
Weight names are the Hugging Face ones (``model.encoder.*``, ``model.decoder.*``, tied ``proj_out``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import attention as A
from ..ops import dense as Dn


@dataclass
class WhisperConfig:
    vocab_size: int = 51865
    num_mel_bins: int = 80
    d_model: int = 384
    encoder_layers: int = 4
    encoder_attention_heads: int = 6
    decoder_layers: int = 4
    decoder_attention_heads: int = 6
    encoder_ffn_dim: int = 1536
    decoder_ffn_dim: int = 1536
    max_source_positions: int = 1500
    max_target_positions: int = 448
    activation_function: str = "gelu"
    decoder_start_token_id: int = 50258
    eos_token_id: int = 50257

    @classmethod
    def from_hf(cls, d: dict) -> "WhisperConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys and v is not None})


class WhisperModel:
    def __init__(self, cfg: WhisperConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        self.device = weights["dec.embed"].device

    @classmethod
    def from_state_dict(cls, cfg: WhisperConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "WhisperModel":
        pre = "model." if any(k.startswith("model.") for k in sd) else ""
        t = lambda x: x.to(dtype).to(device).contiguous()
        w: Dict[str, torch.Tensor] = {}
        e = pre + "encoder."
        # Conv1d weight [out, in, k] -> GEMM weight [out, k * in] matching windows laid out as (tap, channel)
        w["enc.conv1.w"] = t(sd[e + "conv1.weight"].permute(0, 2, 1).reshape(cfg.d_model, -1))
        w["enc.conv1.b"] = t(sd[e + "conv1.bias"])
        w["enc.conv2.w"] = t(sd[e + "conv2.weight"].permute(0, 2, 1).reshape(cfg.d_model, -1))
        w["enc.conv2.b"] = t(sd[e + "conv2.bias"])
        w["enc.pos"] = t(sd[e + "embed_positions.weight"])
        H = cfg.d_model
        zeros = torch.zeros(H, dtype=sd[e + "conv1.bias"].dtype)

        def attn(dst: str, src: str, fused: bool) -> None:
            q, k, v = (sd[src + f"{n}_proj.weight"] for n in "qkv")
            qb, vb = sd[src + "q_proj.bias"], sd[src + "v_proj.bias"]
            if fused:
                w[dst + "qkv.w"], w[dst + "qkv.b"] = t(torch.cat([q, k, v], 0)), t(torch.cat([qb, zeros, vb], 0))
            else:
                w[dst + "q.w"], w[dst + "q.b"] = t(q), t(qb)
                w[dst + "kv.w"], w[dst + "kv.b"] = t(torch.cat([k, v], 0)), t(torch.cat([zeros, vb], 0))
            w[dst + "o.w"], w[dst + "o.b"] = t(sd[src + "out_proj.weight"]), t(sd[src + "out_proj.bias"])

        def block(dst: str, src: str, cross: bool) -> None:
            attn(dst + "sa.", src + "self_attn.", True)
            w[dst + "ln1.g"], w[dst + "ln1.b"] = t(sd[src + "self_attn_layer_norm.weight"]), t(
                sd[src + "self_attn_layer_norm.bias"])
            if cross:
                attn(dst + "ca.", src + "encoder_attn.", False)
                w[dst + "lnc.g"], w[dst + "lnc.b"] = t(sd[src + "encoder_attn_layer_norm.weight"]), t(
                    sd[src + "encoder_attn_layer_norm.bias"])
            w[dst + "fc1.w"], w[dst + "fc1.b"] = t(sd[src + "fc1.weight"]), t(sd[src + "fc1.bias"])
            w[dst + "fc2.w"], w[dst + "fc2.b"] = t(sd[src + "fc2.weight"]), t(sd[src + "fc2.bias"])
            w[dst + "ln2.g"], w[dst + "ln2.b"] = t(sd[src + "final_layer_norm.weight"]), t(
                sd[src + "final_layer_norm.bias"])

        for l in range(cfg.encoder_layers):
            block(f"enc.l{l}.", f"{e}layers.{l}.", False)
        w["enc.lnf.g"], w["enc.lnf.b"] = t(sd[e + "layer_norm.weight"]), t(sd[e + "layer_norm.bias"])
        d = pre + "decoder."
        w["dec.embed"], w["dec.pos"] = t(sd[d + "embed_tokens.weight"]), t(sd[d + "embed_positions.weight"])
        for l in range(cfg.decoder_layers):
            block(f"dec.l{l}.", f"{d}layers.{l}.", True)
        w["dec.lnf.g"], w["dec.lnf.b"] = t(sd[d + "layer_norm.weight"]), t(sd[d + "layer_norm.bias"])
        return cls(cfg, w)

    # ------------------------------------------------------------------------------------------------------
    @staticmethod
    def _unfold(x: torch.Tensor, stride: int) -> torch.Tensor:
        """x [frames, C] -> kernel-3, padding-1 windows [ceil(frames / stride), 3 * C] laid out (tap, channel)."""
        xp = torch.nn.functional.pad(x, (0, 0, 1, 1))
        n = (x.shape[0] + 2 - 3) // stride + 1
        idx = torch.arange(n, device=x.device)[:, None] * stride + torch.arange(3, device=x.device)[None, :]
        return xp[idx].reshape(n, -1).contiguous()

    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        """Log-mel features [n_mels, frames] (frames = 2 * max_source_positions) -> [frames / 2, d_model]."""
        cfg, w = self.cfg, self.w
        dt = w["enc.conv1.w"].dtype
        x = mel.to(self.device).to(dt).T.contiguous()                          # [frames, n_mels]
        x = Dn.gemm_bf16(self._unfold(x, 1), w["enc.conv1.w"], bias=w["enc.conv1.b"], act="gelu")
        x = Dn.gemm_bf16(self._unfold(x, 2), w["enc.conv2.w"], bias=w["enc.conv2.b"], act="gelu")
        T = x.shape[0]
        x = (x.float() + w["enc.pos"][:T].float()).to(dt)
        H, nh = cfg.d_model, cfg.encoder_attention_heads
        D = H // nh
        starts = torch.zeros(1, dtype=torch.int32, device=self.device)
        lens = torch.full((1,), T, dtype=torch.int32, device=self.device)
        for l in range(cfg.encoder_layers):
            p = f"enc.l{l}."
            h = Dn.norm(x, w[p + "ln1.g"], w[p + "ln1.b"], eps=1e-5)
            qkv = Dn.gemm_bf16(h, w[p + "sa.qkv.w"], bias=w[p + "sa.qkv.b"])
            ctx = A.varlen_attention(qkv[:, :H].view(T, nh, D), qkv[:, H:2 * H].view(T, nh, D),
                                     qkv[:, 2 * H:].view(T, nh, D), starts, lens, T).view(T, H)
            x = Dn.gemm_bf16(ctx, w[p + "sa.o.w"], bias=w[p + "sa.o.b"], residual=x)
            h = Dn.norm(x, w[p + "ln2.g"], w[p + "ln2.b"], eps=1e-5)
            m = Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=cfg.activation_function)
            x = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
        return Dn.norm(x, w["enc.lnf.g"], w["enc.lnf.b"], eps=1e-5)

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
        H = self.cfg.d_model
        cross = [Dn.gemm_bf16(enc, self.w[f"dec.l{l}.ca.kv.w"], bias=self.w[f"dec.l{l}.ca.kv.b"])
                 for l in range(self.cfg.decoder_layers)]
        return {"cross": [(c[:, :H], c[:, H:]) for c in cross], "k": [None] * len(cross), "v": [None] * len(cross),
                "len": 0}

    def decode(self, state: dict, ids: Sequence[int]) -> torch.Tensor:
        """Feed the next decoder token(s): fp32 logits [len(ids), vocab]; the caches grow."""
        cfg, w = self.cfg, self.w
        H, nh = cfg.d_model, cfg.decoder_attention_heads
        n0, n = state["len"], len(ids)
        if n0 + n > cfg.max_target_positions:
            raise ValueError("decoder context exceeded")
        tok = torch.tensor(list(ids), device=self.device)
        x = (w["dec.embed"].index_select(0, tok).float() + w["dec.pos"][n0:n0 + n].float()).to(w["dec.embed"].dtype)
        for l in range(cfg.decoder_layers):
            p = f"dec.l{l}."
            h = Dn.norm(x, w[p + "ln1.g"], w[p + "ln1.b"], eps=1e-5)
            qkv = Dn.gemm_bf16(h, w[p + "sa.qkv.w"], bias=w[p + "sa.qkv.b"])
            k, v = qkv[:, H:2 * H], qkv[:, 2 * H:]
            if state["k"][l] is not None:
                k, v = torch.cat([state["k"][l], k]), torch.cat([state["v"][l], v])
            state["k"][l], state["v"][l] = k, v
            x = Dn.gemm_bf16(self._attend(qkv[:, :H], k, v, nh, True), w[p + "sa.o.w"], bias=w[p + "sa.o.b"],
                             residual=x)
            h = Dn.norm(x, w[p + "lnc.g"], w[p + "lnc.b"], eps=1e-5)
            q = Dn.gemm_bf16(h, w[p + "ca.q.w"], bias=w[p + "ca.q.b"])
            ck, cv = state["cross"][l]
            x = Dn.gemm_bf16(self._attend(q, ck, cv, nh, False), w[p + "ca.o.w"], bias=w[p + "ca.o.b"], residual=x)
            h = Dn.norm(x, w[p + "ln2.g"], w[p + "ln2.b"], eps=1e-5)
            m = Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=cfg.activation_function)
            x = Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)
        state["len"] = n0 + n
        return Dn.gemm_bf16(Dn.norm(x, w["dec.lnf.g"], w["dec.lnf.b"], eps=1e-5), w["dec.embed"],
                            out_dtype=torch.float32)

    def transcribe_ids(self, mel: torch.Tensor, prompt: Sequence[int], max_new_tokens: int = 224,
                       suppress: Sequence[int] = ()) -> List[int]:
        """Greedy decoding from the forced prompt until the end-of-text token."""
        state = self.start_decoding(self.encode(mel))
        logits = self.decode(state, list(prompt))[-1]
        out: List[int] = []
        sup = torch.tensor(list(suppress), dtype=torch.long, device=logits.device) if suppress else None
        for _ in range(min(max_new_tokens, self.cfg.max_target_positions - len(prompt))):
            if sup is not None:
                logits = logits.index_fill(0, sup, float("-inf"))
            tok = int(logits.argmax())
            if tok == self.cfg.eos_token_id:
                break
            out.append(tok)
            if state["len"] >= self.cfg.max_target_positions:
                break
            logits = self.decode(state, [tok])[-1]
        return out
