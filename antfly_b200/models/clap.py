"""CLAP: an audio tower (HTS-AT, a Swin transformer over the mel spectrogram) and a RoBERTa text tower that embed
sound clips and captions into one space.

Audio path: per-mel-bin batch norm (folded to a scale and a shift at load), the spectrogram folded into a square
"image", a stride-4 patch convolution done as a GEMM over unfolded patches, four stages of windowed attention
(8x8 windows with a learned relative-position bias, every second block on a half-window cyclic shift) joined by
2x2 patch merging, a final LayerNorm, the mean over all tokens, and a two-layer projection.  Fused checkpoints
describe clips longer than ten seconds by four planes (the whole spectrogram shrunk, plus three crops); the
crops go through a wider convolution and are blended into the global plane by an attentional gate.  Linear
layers run on the tcgen05 bf16 GEMM (bias / GELU / residual epilogues) and LayerNorms on the norm kernel; the 64-
token window attention with its additive bias is batched tensor arithmetic.

Text path: :class:`antfly_b200.models.bert.BertModel` with RoBERTa position ids, the tanh pooler on the first
token, and a two-layer projection.

The reference serves the same two towers (zig/pkg/inference/src/architectures/clap.zig:24 ``textEncoderForward``,
:60 ``audioEncoderForward``; zig/pkg/inference/src/pipelines/embedding.zig:634 ``embedAudioPcm``).  Weight names are
the Hugging Face ones (``audio_model.audio_encoder.*``, ``text_model.*``, ``audio_projection.*``,
``text_projection.*``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import dense as Dn
from .bert import BertConfig, BertModel, pack_sequences


@dataclass
class ClapAudioConfig:
    spec_size: int = 256
    num_mel_bins: int = 64
    patch_size: int = 4
    patch_stride: int = 4
    patch_embeds_hidden_size: int = 96
    depths: List[int] = field(default_factory=lambda: [2, 2, 6, 2])
    num_attention_heads: List[int] = field(default_factory=lambda: [4, 8, 16, 32])
    window_size: int = 8
    mlp_ratio: float = 4.0
    hidden_size: int = 768
    layer_norm_eps: float = 1e-5
    hidden_act: str = "gelu"
    projection_hidden_act: str = "relu"
    enable_fusion: bool = False
    fusion_type: Optional[str] = None
    aff_block_r: int = 4
    qkv_bias: bool = True
    enable_patch_layer_norm: bool = True


@dataclass
class ClapConfig:
    audio: ClapAudioConfig
    text: BertConfig
    projection_dim: int = 512

    @classmethod
    def from_hf(cls, d: dict) -> "ClapConfig":
        a = d.get("audio_config", {})
        keys = ClapAudioConfig.__dataclass_fields__
        ac = ClapAudioConfig(**{k: v for k, v in a.items() if k in keys and v is not None})
        for name in ("patch_size", "patch_stride"):            # configs may spell these as [h, w]
            v = getattr(ac, name)
            if isinstance(v, (list, tuple)):
                setattr(ac, name, int(v[0]))
        t = dict(d.get("text_config", {}))
        t.setdefault("model_type", "roberta")
        tc = BertConfig.from_hf(t)
        tc.position_offset = int(t.get("pad_token_id", 1)) + 1
        return cls(ac, tc, d.get("projection_dim", 512))


def _relative_index(ws: int) -> torch.Tensor:
    """[ws*ws, ws*ws] index into the (2 ws - 1)^2 bias table for every (query, key) pair of a window."""
    c = torch.stack(torch.meshgrid(torch.arange(ws), torch.arange(ws), indexing="ij")).flatten(1)
    rel = (c[:, :, None] - c[:, None, :]).permute(1, 2, 0) + (ws - 1)
    return rel[..., 0] * (2 * ws - 1) + rel[..., 1]


def _shift_mask(h: int, w: int, ws: int, shift: int) -> torch.Tensor:
    """[windows, ws*ws, ws*ws] additive mask (0 / -100) that keeps tokens brought together by the cyclic shift
    from attending across the seam."""
    img = torch.zeros(h, w)
    n = 0
    for hs in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
        for wsl in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
            img[hs, wsl] = n
            n += 1
    win = img.view(h // ws, ws, w // ws, ws).permute(0, 2, 1, 3).reshape(-1, ws * ws)
    diff = win[:, None, :] - win[:, :, None]
    return torch.where(diff != 0, torch.full_like(diff, -100.0), torch.zeros_like(diff))


class ClapModel:
    def __init__(self, cfg: ClapConfig, weights: Dict[str, torch.Tensor], text: BertModel):
        self.cfg, self.w, self.text = cfg, weights, text
        self.device = weights["a.patch.w"].device
        self._rel = _relative_index(cfg.audio.window_size)
        self._bias_cache: Dict[Tuple[int, int], torch.Tensor] = {}
        self._mask_cache: Dict[Tuple[int, int, int, int], torch.Tensor] = {}

    @classmethod
    def from_state_dict(cls, cfg: ClapConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "ClapModel":
        t = lambda x: x.to(dtype).to(device).contiguous()
        f32 = lambda x: x.float().to(device).contiguous()
        a = "audio_model.audio_encoder."
        ac = cfg.audio
        w: Dict[str, torch.Tensor] = {}

        def fold_bn(prefix: str, eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
            """Inference batch norm as y = x * scale + shift."""
            s = sd[prefix + "weight"].float() / torch.sqrt(sd[prefix + "running_var"].float() + eps)
            return s, sd[prefix + "bias"].float() - sd[prefix + "running_mean"].float() * s

        s, b = fold_bn(a + "batch_norm.")
        w["a.bn.s"], w["a.bn.b"] = f32(s), f32(b)
        w["a.patch.w"] = t(sd[a + "patch_embed.proj.weight"].flatten(1))
        w["a.patch.b"] = t(sd[a + "patch_embed.proj.bias"])
        if ac.enable_patch_layer_norm:
            w["a.patch.ln.g"], w["a.patch.ln.b"] = t(sd[a + "patch_embed.norm.weight"]), t(sd[a + "patch_embed.norm.bias"])
        if ac.enable_fusion:
            w["a.mel.w"] = t(sd[a + "patch_embed.mel_conv2d.weight"].flatten(1))
            w["a.mel.b"] = t(sd[a + "patch_embed.mel_conv2d.bias"])
            for branch, idx in (("local_att", (0, 1, 3, 4)), ("global_att", (1, 2, 4, 5))):
                p = a + f"patch_embed.fusion_model.{branch}."
                for n, (conv, bn) in enumerate(((idx[0], idx[1]), (idx[2], idx[3]))):
                    s, b = fold_bn(p + f"{bn}.")
                    cw = sd[p + f"{conv}.weight"].float().flatten(1)
                    w[f"a.aff.{branch}.{n}.w"] = f32(cw * s[:, None])
                    w[f"a.aff.{branch}.{n}.b"] = f32(sd[p + f"{conv}.bias"].float() * s + b)
        for i, depth in enumerate(ac.depths):
            for j in range(depth):
                s_, p = a + f"layers.{i}.blocks.{j}.", f"a.s{i}.b{j}."
                w[p + "ln1.g"], w[p + "ln1.b"] = t(sd[s_ + "layernorm_before.weight"]), t(sd[s_ + "layernorm_before.bias"])
                w[p + "ln2.g"], w[p + "ln2.b"] = t(sd[s_ + "layernorm_after.weight"]), t(sd[s_ + "layernorm_after.bias"])
                w[p + "qkv.w"] = t(torch.cat([sd[s_ + f"attention.self.{n}.weight"] for n in ("query", "key", "value")], 0))
                if ac.qkv_bias:
                    w[p + "qkv.b"] = t(torch.cat([sd[s_ + f"attention.self.{n}.bias"] for n in ("query", "key", "value")], 0))
                w[p + "rel"] = f32(sd[s_ + "attention.self.relative_position_bias_table"])
                w[p + "o.w"], w[p + "o.b"] = t(sd[s_ + "attention.output.dense.weight"]), t(sd[s_ + "attention.output.dense.bias"])
                w[p + "fc1.w"], w[p + "fc1.b"] = t(sd[s_ + "intermediate.dense.weight"]), t(sd[s_ + "intermediate.dense.bias"])
                w[p + "fc2.w"], w[p + "fc2.b"] = t(sd[s_ + "output.dense.weight"]), t(sd[s_ + "output.dense.bias"])
            if i < len(ac.depths) - 1:
                p = f"a.s{i}.merge."
                w[p + "ln.g"], w[p + "ln.b"] = t(sd[a + f"layers.{i}.downsample.norm.weight"]), t(
                    sd[a + f"layers.{i}.downsample.norm.bias"])
                w[p + "w"] = t(sd[a + f"layers.{i}.downsample.reduction.weight"])
        w["a.lnf.g"], w["a.lnf.b"] = t(sd[a + "norm.weight"]), t(sd[a + "norm.bias"])
        for tower, pre in (("a", "audio_projection."), ("t", "text_projection.")):
            for n in (1, 2):
                w[f"{tower}.proj{n}.w"], w[f"{tower}.proj{n}.b"] = t(sd[pre + f"linear{n}.weight"]), t(sd[pre + f"linear{n}.bias"])
        w["t.pool.w"], w["t.pool.b"] = t(sd["text_model.pooler.dense.weight"]), t(sd["text_model.pooler.dense.bias"])
        text_sd = {k[len("text_model."):]: v for k, v in sd.items() if k.startswith("text_model.")}
        text = BertModel.from_state_dict(cfg.text, text_sd, device=device, dtype=dtype)
        return cls(cfg, w, text)

    # -- audio tower ---------------------------------------------------------------------------------------
    def _to_image(self, feats: torch.Tensor) -> torch.Tensor:
        """[B, C, T, F] normalised spectrograms -> [B, C, spec, spec]: time is stretched to ``spec * ratio`` frames
        (bicubic), cut into ``ratio`` consecutive pieces, and the pieces are stacked along the frequency axis."""
        ac = self.cfg.audio
        ratio = ac.spec_size // ac.num_mel_bins
        B, C, T, F = feats.shape
        width, height = ac.spec_size * ratio, ac.spec_size // ratio
        if T > width or F > height:
            raise ValueError("spectrogram larger than the audio tower's input")
        if T < width:
            feats = torch.nn.functional.interpolate(feats, (width, F), mode="bicubic", align_corners=True)
        if F < height:
            feats = torch.nn.functional.interpolate(feats, (feats.shape[2], height), mode="bicubic", align_corners=True)
        B, C, T, F = feats.shape
        x = feats.reshape(B, C * ratio, T // ratio, F).permute(0, 1, 3, 2)
        return x.reshape(B, C, F * ratio, T // ratio)

    def _conv(self, x: torch.Tensor, wk: str, bk: str, kh: int, kw: int) -> torch.Tensor:
        """Non-overlapping ``kh x kw`` convolution of [N, Cin, H, W] as one GEMM -> [N, H/kh * W/kw, Cout]."""
        N_, C, H, W = x.shape
        gh, gw = H // kh, W // kw
        dt = self.w[wk].dtype
        cols = x[:, :, : gh * kh, : gw * kw].reshape(N_, C, gh, kh, gw, kw).permute(0, 2, 4, 1, 3, 5)
        cols = cols.reshape(N_ * gh * gw, C * kh * kw).to(dt).contiguous()
        return Dn.gemm_bf16(cols, self.w[wk], bias=self.w[bk]).view(N_, gh * gw, -1)

    def _fuse(self, glob: torch.Tensor, local: torch.Tensor) -> torch.Tensor:
        """Attentional feature fusion on [n, L, E] token grids: a per-token gate (two 1x1 convolutions) plus a
        per-clip gate (the same on the token mean) decide, per channel, how much of each input to keep."""
        w = self.w
        g, l = glob.float(), local.float()
        x = g + l

        def branch(name: str, t: torch.Tensor) -> torch.Tensor:
            h = torch.relu(t @ w[f"a.aff.{name}.0.w"].T + w[f"a.aff.{name}.0.b"])
            return h @ w[f"a.aff.{name}.1.w"].T + w[f"a.aff.{name}.1.b"]

        gate = torch.sigmoid(branch("local_att", x) + branch("global_att", x.mean(1, keepdim=True)))
        return (2 * g * gate + 2 * l * (1 - gate)).to(glob.dtype)

    def _patch_embed(self, img: torch.Tensor, is_longer: Sequence[bool]) -> torch.Tensor:
        ac, w = self.cfg.audio, self.w
        P = ac.patch_size
        if ac.patch_stride != P:
            raise ValueError("overlapping audio patches are not supported")
        x = self._conv(img[:, 0:1], "a.patch.w", "a.patch.b", P, P)                  # [B, g*g, E]
        idx = [i for i, f in enumerate(is_longer) if f] if ac.enable_fusion else []
        if idx:
            g = ac.spec_size // P
            crops = img[idx, 1:]                                                      # [n, 3, S, S]
            n, k = crops.shape[:2]
            loc = self._conv(crops.reshape(n * k, 1, *crops.shape[2:]), "a.mel.w", "a.mel.b", P, 3 * P)
            gw = loc.shape[1] // g                                                   # columns per crop
            # the crops sit side by side along the time axis: column = crop * gw + c, zero-padded to g columns
            loc = loc.view(n, k, g, gw, -1).permute(0, 2, 1, 3, 4).reshape(n, g, k * gw, -1)
            loc = torch.nn.functional.pad(loc, (0, 0, 0, g - k * gw)).reshape(n, g * g, -1)
            x = x.clone()
            x[idx] = self._fuse(x[idx], loc)
        if ac.enable_patch_layer_norm:
            B, L, E = x.shape
            x = Dn.norm(x.reshape(B * L, E).contiguous(), w["a.patch.ln.g"], w["a.patch.ln.b"],
                        eps=1e-5).view(B, L, E)
        return x

    def _window_bias(self, stage: int, block: int, nh: int) -> torch.Tensor:
        key = (stage, block)
        if key not in self._bias_cache:
            ws = self.cfg.audio.window_size
            table = self.w[f"a.s{stage}.b{block}.rel"]                               # [(2 ws - 1)^2, nh]
            self._bias_cache[key] = table[self._rel.to(table.device).flatten()].view(ws * ws, ws * ws, nh).permute(
                2, 0, 1).contiguous()
        return self._bias_cache[key]

    def _block(self, x: torch.Tensor, stage: int, block: int, res: Tuple[int, int], nh: int) -> torch.Tensor:
        """One Swin block on tokens [B * H * W, C]: windowed attention (shifted on odd blocks), then the MLP."""
        ac, w = self.cfg.audio, self.w
        p = f"a.s{stage}.b{block}."
        Hh, Ww = res
        ws = ac.window_size
        shift = ws // 2 if block % 2 == 1 else 0
        if min(res) <= ws:                       # a grid that is one window wide has nothing to shift into
            shift, ws = 0, min(res)
        if Hh % ws or Ww % ws:
            raise ValueError("token grid is not a whole number of windows")
        C = x.shape[1]
        B = x.shape[0] // (Hh * Ww)
        D = C // nh
        h = Dn.norm(x, w[p + "ln1.g"], w[p + "ln1.b"], eps=ac.layer_norm_eps)
        qkv = Dn.gemm_bf16(h, w[p + "qkv.w"], bias=w.get(p + "qkv.b")).view(B, Hh, Ww, 3 * C)
        if shift:
            qkv = torch.roll(qkv, (-shift, -shift), (1, 2))
        nwh, nww = Hh // ws, Ww // ws
        win = qkv.view(B, nwh, ws, nww, ws, 3, nh, D).permute(5, 0, 1, 3, 6, 2, 4, 7).reshape(
            3, B, nwh * nww, nh, ws * ws, D).float()
        s = torch.matmul(win[0], win[1].transpose(-1, -2)) * (D ** -0.5) + self._window_bias(stage, block, nh)
        if shift:
            mk = (Hh, Ww, ws, shift)
            if mk not in self._mask_cache:
                self._mask_cache[mk] = _shift_mask(Hh, Ww, ws, shift).to(x.device)
            s = s + self._mask_cache[mk][None, :, None]
        ctx = torch.matmul(torch.softmax(s, -1), win[2])                              # [B, nW, nh, ws*ws, D]
        ctx = ctx.view(B, nwh, nww, nh, ws, ws, D).permute(0, 1, 4, 2, 5, 3, 6).reshape(B, Hh, Ww, C)
        if shift:
            ctx = torch.roll(ctx, (shift, shift), (1, 2))
        ctx = ctx.reshape(B * Hh * Ww, C).to(x.dtype).contiguous()
        x = Dn.gemm_bf16(ctx, w[p + "o.w"], bias=w[p + "o.b"], residual=x)
        h = Dn.norm(x, w[p + "ln2.g"], w[p + "ln2.b"], eps=ac.layer_norm_eps)
        m = Dn.gemm_bf16(h, w[p + "fc1.w"], bias=w[p + "fc1.b"], act=ac.hidden_act)
        return Dn.gemm_bf16(m, w[p + "fc2.w"], bias=w[p + "fc2.b"], residual=x)

    def audio_hidden(self, feats: torch.Tensor, is_longer: Optional[Sequence[bool]] = None) -> torch.Tensor:
        """[B, C, T, F] spectrograms (dB) -> pooled tower output, fp32 [B, hidden]."""
        ac, w = self.cfg.audio, self.w
        B = feats.shape[0]
        x = feats.to(self.device).float() * w["a.bn.s"] + w["a.bn.b"]
        img = self._to_image(x)
        tok = self._patch_embed(img, list(is_longer) if is_longer is not None else [False] * B)
        g = ac.spec_size // ac.patch_stride
        res = (g, g)
        C = tok.shape[-1]
        x = tok.reshape(B * g * g, C).contiguous()
        for i, depth in enumerate(ac.depths):
            for j in range(depth):
                x = self._block(x, i, j, res, ac.num_attention_heads[i])
            if i < len(ac.depths) - 1:
                Hh, Ww = res
                if Hh % 2 or Ww % 2:
                    raise ValueError("odd token grid at a merge")
                v = x.view(B, Hh // 2, 2, Ww // 2, 2, C)
                # channel order of a merged 2x2 cell: (0,0), (1,0), (0,1), (1,1)
                m = torch.cat([v[:, :, 0, :, 0], v[:, :, 1, :, 0], v[:, :, 0, :, 1], v[:, :, 1, :, 1]], -1)
                m = m.reshape(B * (Hh // 2) * (Ww // 2), 4 * C).contiguous()
                m = Dn.norm(m, w[f"a.s{i}.merge.ln.g"], w[f"a.s{i}.merge.ln.b"], eps=1e-5)
                x = Dn.gemm_bf16(m, w[f"a.s{i}.merge.w"])
                res, C = (Hh // 2, Ww // 2), 2 * C
        x = Dn.norm(x, w["a.lnf.g"], w["a.lnf.b"], eps=1e-5)
        return x.view(B, res[0] * res[1], C).float().mean(1)

    def _project(self, tower: str, pooled: torch.Tensor, normalize: bool) -> torch.Tensor:
        w = self.w
        dt = w[f"{tower}.proj1.w"].dtype
        h = Dn.gemm_bf16(pooled.to(dt).contiguous(), w[f"{tower}.proj1.w"], bias=w[f"{tower}.proj1.b"],
                         act=self.cfg.audio.projection_hidden_act)
        e = Dn.gemm_bf16(h, w[f"{tower}.proj2.w"], bias=w[f"{tower}.proj2.b"], out_dtype=torch.float32).float()
        return torch.nn.functional.normalize(e, dim=-1) if normalize else e

    def embed_audio(self, feats: torch.Tensor, is_longer: Optional[Sequence[bool]] = None,
                    normalize: bool = True) -> torch.Tensor:
        """Spectrogram planes from :func:`antfly_b200.ops.audio_ops.clap_features` -> fp32 [B, projection_dim]."""
        return self._project("a", self.audio_hidden(feats, is_longer), normalize)

    def embed_text(self, seqs: Sequence[Sequence[int]], normalize: bool = True) -> torch.Tensor:
        """Token id sequences (with ``<s>`` / ``</s>``) -> fp32 [B, projection_dim]."""
        w = self.w
        b = pack_sequences(seqs, position_offset=self.cfg.text.position_offset).to(self.device)
        h = self.text.encode(b)
        first = h.index_select(0, b.starts.long())
        pooled = torch.tanh(Dn.gemm_bf16(first.contiguous(), w["t.pool.w"], bias=w["t.pool.b"],
                                         out_dtype=torch.float32).float())
        return self._project("t", pooled, normalize)
