"""Image preprocessing (host path = the code the GPU kernel runs per sample) against torch's interpolate."""
import pytest
import torch
import torch.nn.functional as F

from antfly_b200.ops import image_ops as I


def _ref(img_u8, out_hw, mode, mean, std, crop=None):
    x = img_u8[..., :3].permute(2, 0, 1)[None].float()
    if crop is not None:
        cx, cy, cw, ch = (int(v) for v in crop)
        x = x[:, :, cy:cy + ch, cx:cx + cw]
    kw = {} if mode == "nearest" else {"align_corners": False}
    y = F.interpolate(x, size=out_hw, mode=mode, **kw)[0] / 255.0
    m, s = torch.tensor(mean)[:, None, None], torch.tensor(std)[:, None, None]
    return (y - m) / s


@pytest.mark.parametrize("mode", ["nearest", "bilinear", "bicubic"])
@pytest.mark.parametrize("shape,out", [((37, 53, 3), (24, 24)), ((64, 48, 4), (80, 100)), ((20, 20, 3), (20, 20))])
def test_resize_normalise_matches_torch(mode, shape, out):
    g = torch.Generator().manual_seed(0)
    img = torch.randint(0, 256, shape, generator=g, dtype=torch.uint8)
    got = I.preprocess(img, out, mode=mode)[0]
    want = _ref(img, out, mode, I.CLIP_MEAN, I.CLIP_STD)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=1e-4)


def test_crop_and_clip_recipe_and_batch():
    g = torch.Generator().manual_seed(1)
    imgs = torch.randint(0, 256, (3, 60, 90, 3), generator=g, dtype=torch.uint8)
    got = I.preprocess(imgs, (32, 32), mode="bilinear", crop=(15.0, 0.0, 60.0, 60.0))
    assert got.shape == (3, 3, 32, 32)
    for b in range(3):
        torch.testing.assert_close(got[b], _ref(imgs[b], (32, 32), "bilinear", I.CLIP_MEAN, I.CLIP_STD,
                                                crop=(15, 0, 60, 60)), atol=2e-4, rtol=1e-4)
    clip = I.clip_preprocess(imgs, size=30, mode="bilinear")
    torch.testing.assert_close(clip, got_same := I.preprocess(imgs, (30, 30), mode="bilinear",
                                                              crop=(15.0, 0.0, 60.0, 60.0)))
    assert I.preprocess(imgs[0], (8, 8), dtype=torch.bfloat16).dtype == torch.bfloat16
