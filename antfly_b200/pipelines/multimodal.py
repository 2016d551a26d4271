"""Image / text embedding with a CLIP-style dual encoder.

``ClipEmbedder.embed_images`` takes decoded images (uint8 HWC tensors / arrays) or file paths (decoded with
Pillow when it is installed), runs the preprocessing kernel (resize shorter side, centre crop, normalise) and the
vision tower; ``embed_texts`` tokenises with the model's tokenizer (begin / end tokens added, truncated to the
context length) and runs the text tower.  Both return L2-normalised fp32 rows of the shared space, so
``text @ image.T`` is the usual similarity.  Mirrors the reference's ``embedImages`` / text path for CLIP models
(zig/pkg/inference/src/pipelines/embedding.zig:432-634).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..models.clip import ClipModel
from ..ops import image_ops as I

ImageLike = Union[str, np.ndarray, torch.Tensor]


def decode_image_bytes(data: bytes) -> torch.Tensor:
    """Encoded image bytes (PNG / JPEG / ...) -> uint8 [H, W, 3] tensor (needs Pillow)."""
    import io

    from PIL import Image

    with Image.open(io.BytesIO(data)) as im:
        return torch.from_numpy(np.asarray(im.convert("RGB")).copy())


def decode_data_url(url: str) -> torch.Tensor:
    """``data:image/png;base64,...`` -> uint8 [H, W, 3]."""
    import base64

    if not url.startswith("data:") or "," not in url:
        raise ValueError("only data: URLs are accepted (this server does not fetch remote images)")
    head, payload = url.split(",", 1)
    raw = base64.b64decode(payload) if head.endswith(";base64") else payload.encode("latin-1")
    return decode_image_bytes(raw)


def load_image(src: ImageLike) -> torch.Tensor:
    """-> uint8 [H, W, 3 or 4] tensor on the host."""
    if isinstance(src, torch.Tensor):
        t = src
    elif isinstance(src, np.ndarray):
        t = torch.from_numpy(np.ascontiguousarray(src))
    else:
        try:
            from PIL import Image
        except ImportError as e:  # pragma: no cover
            raise RuntimeError("decoding image files needs Pillow; pass decoded uint8 arrays instead") from e
        with Image.open(src) as im:
            t = torch.from_numpy(np.asarray(im.convert("RGB")).copy())
    if t.dim() == 2:
        t = t[..., None].expand(-1, -1, 3)
    assert t.dtype == torch.uint8 and t.dim() == 3 and t.shape[-1] in (3, 4), "expected a uint8 HWC image"
    return t.contiguous()


class ClipEmbedder:
    def __init__(self, model: ClipModel, tokenizer=None, bos_id: Optional[int] = None, eos_id: Optional[int] = None,
                 resample: str = "bicubic"):
        self.model, self.tokenizer, self.resample = model, tokenizer, resample
        self.bos_id, self.eos_id = bos_id, eos_id
        if tokenizer is not None:
            self.bos_id = bos_id if bos_id is not None else tokenizer.special.bos_id
            self.eos_id = eos_id if eos_id is not None else tokenizer.special.eos_id

    @property
    def dim(self) -> int:
        return self.model.cfg.projection_dim

    def embed_images(self, images: Sequence[ImageLike], batch_size: int = 64) -> torch.Tensor:
        size = self.model.cfg.vision.image_size
        dev = self.model.device
        pix: List[torch.Tensor] = []
        for src in images:
            img = load_image(src)
            pix.append(I.clip_preprocess(img.to(dev) if dev.type == "cuda" else img, size=size, mode=self.resample)[0])
        out = [self.model.embed_images(torch.stack(pix[i:i + batch_size])) for i in range(0, len(pix), batch_size)]
        return torch.cat(out, 0) if out else torch.zeros((0, self.dim))

    def embed(self, texts: Sequence[str], task_type: Optional[str] = None, dimensions: Optional[int] = None):
        """The text-embedding contract of the HTTP endpoint: (fp32 [N, dims] on the host, prompt tokens)."""
        e = self.embed_texts(texts).cpu()
        if dimensions:
            if dimensions > e.shape[1]:
                raise ValueError(f"dimensions {dimensions} exceeds the model's {e.shape[1]}")
            e = torch.nn.functional.normalize(e[:, :dimensions], dim=-1)
        limit = self.model.cfg.text.max_position_embeddings
        return e, sum(min(len(self.tokenizer.encode(t)) + 2, limit) for t in texts)

    def embed_token_ids(self, seqs: Sequence[Sequence[int]]) -> torch.Tensor:
        return self.model.embed_text(seqs)

    def embed_texts(self, texts: Sequence[str]) -> torch.Tensor:
        if self.tokenizer is None:
            raise RuntimeError("this embedder has no tokenizer")
        limit = self.model.cfg.text.max_position_embeddings
        seqs = []
        for t in texts:
            ids = self.tokenizer.encode(t)[: limit - 2]
            seqs.append(([self.bos_id] if self.bos_id is not None else []) + ids +
                        ([self.eos_id] if self.eos_id is not None else []))
        return self.model.embed_text(seqs)


AudioLike = Union[str, bytes, torch.Tensor, tuple]


class ClapEmbedder:
    """Audio / text embedding with a CLAP dual encoder.

    ``embed_audio`` takes WAV bytes or paths, waveforms at 48 kHz, or ``(waveform, rate)`` pairs; each clip is
    resampled to 48 kHz, turned into the tower's spectrogram planes (short clips repeated and padded to ten
    seconds, long ones described by a shrunk overview plus three crops) and embedded.  ``embed_texts`` runs the
    RoBERTa tower.  Rows are L2-normalised fp32 in the shared space (zig/pkg/inference/src/pipelines/embedding.zig:634
    ``embedAudioPcm``)."""

    def __init__(self, model, tokenizer=None, bos_id: Optional[int] = None, eos_id: Optional[int] = None):
        self.model, self.tokenizer = model, tokenizer
        self.bos_id, self.eos_id = bos_id, eos_id
        if tokenizer is not None:
            self.bos_id = bos_id if bos_id is not None else tokenizer.special.bos_id
            self.eos_id = eos_id if eos_id is not None else tokenizer.special.eos_id

    @property
    def dim(self) -> int:
        return self.model.cfg.projection_dim

    def embed_audio(self, clips: Sequence[AudioLike], batch_size: int = 16) -> torch.Tensor:
        from ..ops import audio_ops as Au

        channels = 4 if self.model.cfg.audio.enable_fusion else 1
        feats: List[torch.Tensor] = []
        longer: List[bool] = []
        for c in clips:
            if isinstance(c, (bytes, bytearray, str)):
                wave, rate = Au.read_wav(c)
            elif isinstance(c, tuple):
                wave, rate = torch.as_tensor(c[0]).float().flatten(), int(c[1])
            else:
                wave, rate = torch.as_tensor(c).float().flatten(), Au.CLAP_RATE
            if rate != Au.CLAP_RATE:
                wave = Au.resample(wave, rate, Au.CLAP_RATE)
            f, is_long = Au.clap_features(wave, channels)
            if not self.model.cfg.audio.enable_fusion:
                f = f[:1]                                   # unfused towers see the first plane only
            feats.append(f)
            longer.append(is_long)
        out = [self.model.embed_audio(torch.stack(feats[i:i + batch_size]), longer[i:i + batch_size])
               for i in range(0, len(feats), batch_size)]
        return torch.cat(out, 0) if out else torch.zeros((0, self.dim))

    def embed_texts(self, texts: Sequence[str]) -> torch.Tensor:
        if self.tokenizer is None:
            raise RuntimeError("this embedder has no tokenizer")
        limit = self.model.cfg.text.max_position_embeddings - self.model.cfg.text.position_offset
        seqs = []
        for t in texts:
            ids = self.tokenizer.encode(t)[: limit - 2]
            seqs.append(([self.bos_id] if self.bos_id is not None else []) + ids +
                        ([self.eos_id] if self.eos_id is not None else []))
        return self.model.embed_text(seqs)

    def embed_token_ids(self, seqs: Sequence[Sequence[int]]) -> torch.Tensor:
        return self.model.embed_text(seqs)

    def embed(self, texts: Sequence[str], task_type: Optional[str] = None, dimensions: Optional[int] = None):
        """The text-embedding contract of the HTTP endpoint: (fp32 [N, dims] on the host, prompt tokens)."""
        e = self.embed_texts(texts).cpu()
        if dimensions:
            if dimensions > e.shape[1]:
                raise ValueError(f"dimensions {dimensions} exceeds the model's {e.shape[1]}")
            e = torch.nn.functional.normalize(e[:, :dimensions], dim=-1)
        limit = self.model.cfg.text.max_position_embeddings - self.model.cfg.text.position_offset
        return e, sum(min(len(self.tokenizer.encode(t)) + 2, limit) for t in texts)
