"""Image preprocessing kernel against the host path (same per-sample code) and torch's interpolate."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["nearest", "bilinear", "bicubic"])
def test_device_preprocess_matches_host(mode):
    from antfly_b200.ops import image_ops as I

    g = torch.Generator().manual_seed(0)
    imgs = torch.randint(0, 256, (5, 181, 240, 3), generator=g, dtype=torch.uint8)
    want = I.clip_preprocess(imgs, size=224, mode=mode)
    got = I.clip_preprocess(imgs.cuda(), size=224, mode=mode)
    torch.testing.assert_close(got.cpu(), want, atol=1e-4, rtol=1e-4)
    got16 = I.clip_preprocess(imgs.cuda(), size=224, mode=mode, dtype=torch.bfloat16)
    torch.testing.assert_close(got16.float().cpu(), want, atol=2e-2, rtol=1e-2)
    rgba = torch.randint(0, 256, (2, 50, 70, 4), generator=g, dtype=torch.uint8)
    torch.testing.assert_close(I.preprocess(rgba.cuda(), (64, 96), mode=mode).cpu(), I.preprocess(rgba, (64, 96), mode=mode),
                               atol=1e-4, rtol=1e-4)
