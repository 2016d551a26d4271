"""Image preprocessing for vision encoders: crop -> resize -> rescale -> normalise, uint8 HWC -> planar CHW.

CUDA tensors run ``afb_image_preprocess`` (one launch per batch of equally sized images); CPU tensors run the
same per-sample code on the host.  ``clip_preprocess`` is the CLIP recipe: resize so the shorter side matches the
target with the aspect ratio kept, centre-crop a square -- expressed as one resize of the centred source square.
Semantics of the reference's preprocessing (zig/lib/image/src/processing.zig:41-177)."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native as N

MODES = {"nearest": 0, "bilinear": 1, "bicubic": 2}
CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def preprocess(images: torch.Tensor, out_size: Tuple[int, int], mean: Sequence[float] = CLIP_MEAN,
               std: Sequence[float] = CLIP_STD, mode: str = "bilinear", rescale: float = 1.0 / 255.0,
               crop: Optional[Tuple[float, float, float, float]] = None,
               dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """images: uint8 [B, H, W, C] (C = 3 or 4) or [H, W, C]; out_size: (height, width); crop: (x, y, w, h) source
    rectangle that maps onto the output (default: the whole image).  Returns [B, 3, out_h, out_w]."""
    if images.dim() == 3:
        images = images[None]
    assert images.dtype == torch.uint8 and images.dim() == 4 and images.shape[-1] in (3, 4)
    B, H, W, C = images.shape
    oh, ow = out_size
    cx, cy, cw, chh = crop if crop is not None else (0.0, 0.0, float(W), float(H))
    m = (ctypes.c_float * 3)(*mean)
    s = (ctypes.c_float * 3)(*std)
    images = images.contiguous()
    if images.is_cuda:
        assert dtype in (torch.float32, torch.bfloat16)
        out = torch.empty((B, 3, oh, ow), dtype=dtype, device=images.device)
        rc = N.cuda().afb_image_preprocess(
            N.ptr(images), ctypes.c_int(B), ctypes.c_int(W), ctypes.c_int(H), ctypes.c_int(C), ctypes.c_float(cx),
            ctypes.c_float(cy), ctypes.c_float(cw), ctypes.c_float(chh), ctypes.c_int(ow), ctypes.c_int(oh),
            ctypes.c_int(MODES[mode]), ctypes.c_float(rescale), m, s, N.ptr(out),
            ctypes.c_int(1 if dtype == torch.bfloat16 else 0), N.stream_ptr())
        N.check(rc, "afb_image_preprocess")
        N.count_launch()
        return out
    out = np.empty((B, 3, oh, ow), dtype=np.float32)
    src = images.numpy()
    for b in range(B):
        rc = N.host().afb_image_preprocess_host(
            src[b].ctypes.data_as(ctypes.c_void_p), ctypes.c_int(W), ctypes.c_int(H), ctypes.c_int(C),
            ctypes.c_float(cx), ctypes.c_float(cy), ctypes.c_float(cw), ctypes.c_float(chh), ctypes.c_int(ow),
            ctypes.c_int(oh), ctypes.c_int(MODES[mode]), ctypes.c_float(rescale), m, s,
            out[b].ctypes.data_as(ctypes.c_void_p))
        if rc != 0:
            raise ValueError("bad image geometry")
    return torch.from_numpy(out).to(dtype)


def clip_preprocess(images: torch.Tensor, size: int = 224, mode: str = "bicubic",
                    dtype: torch.dtype = torch.float32) -> torch.Tensor:
    H, W = (images.shape[-3], images.shape[-2])
    side = float(min(H, W))
    crop = ((W - side) / 2.0, (H - side) / 2.0, side, side)
    return preprocess(images, (size, size), CLIP_MEAN, CLIP_STD, mode, 1.0 / 255.0, crop, dtype)
