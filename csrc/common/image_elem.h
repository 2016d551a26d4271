// Image preprocessing for vision encoders, per output sample, compiled for both the host and the device:
// crop -> resize (nearest / bilinear / bicubic, half-pixel centres) -> rescale -> normalise, from an interleaved
// 8-bit image (RGB or RGBA, row-major HWC) to planar fp32 CHW.  The device kernel (csrc/kernels/image.cu) runs
// this once per output pixel and channel; the host entry point runs the same code, which is what the CPU tests
// compare with torch's interpolate.
//
// Sampling convention of the reference (zig/lib/image/src/processing.zig:382-453): source coordinate
// (dst + 0.5) * scale - 0.5, neighbours clamped to the image, value * rescale - mean, divided by std.  One
// deliberate difference: the interpolation weights are clamped to [0, 1] at the borders (the usual convention,
// torch / PIL), where the reference extrapolates slightly.
#pragma once
#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define AFB_IMG_HD __host__ __device__ __forceinline__
#else
#define AFB_IMG_HD inline
#endif

namespace afb {
namespace image {

struct Params {
  int src_w, src_h, channels;           // channels: 3 or 4 (alpha ignored)
  float crop_x, crop_y, crop_w, crop_h;  // source rectangle that maps onto the output
  int out_w, out_h;
  int mode;                              // 0 nearest, 1 bilinear, 2 bicubic (a = -0.75)
  float rescale;                         // usually 1 / 255
  float mean[3], inv_std[3];
};

AFB_IMG_HD int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

AFB_IMG_HD float pixel(const uint8_t* img, const Params& p, int x, int y, int ch) {
  x = clampi(x, 0, p.src_w - 1);
  y = clampi(y, 0, p.src_h - 1);
  return static_cast<float>(img[(static_cast<long>(y) * p.src_w + x) * p.channels + ch]);
}

AFB_IMG_HD float cubic_weight(float t, int k) {
  // Keys kernel with a = -0.75 for the four taps at offsets -1, 0, 1, 2 (k = 0..3) and fraction t
  const float a = -0.75f;
  const float x = k == 0 ? t + 1.0f : (k == 1 ? t : (k == 2 ? 1.0f - t : 2.0f - t));
  if (k == 1 || k == 2) return ((a + 2.0f) * x - (a + 3.0f)) * x * x + 1.0f;
  return ((a * x - 5.0f * a) * x + 8.0f * a) * x - 4.0f * a;
}

// Normalised value of output sample (ox, oy, ch).
AFB_IMG_HD float sample(const uint8_t* img, const Params& p, int ox, int oy, int ch) {
  const float sx = p.crop_w / p.out_w, sy = p.crop_h / p.out_h;
  float fx = (ox + 0.5f) * sx - 0.5f + p.crop_x;
  float fy = (oy + 0.5f) * sy - 0.5f + p.crop_y;
  float v;
  if (p.mode == 0) {
    // nearest: floor of the un-shifted coordinate, the convention of torch's 'nearest'
    const int x = static_cast<int>(floorf(ox * sx + p.crop_x)), y = static_cast<int>(floorf(oy * sy + p.crop_y));
    v = pixel(img, p, x, y, ch);
  } else if (p.mode == 1) {
    if (fx < 0.0f) fx = 0.0f;
    if (fy < 0.0f) fy = 0.0f;
    const int x0 = static_cast<int>(floorf(fx)), y0 = static_cast<int>(floorf(fy));
    const float tx = fx - x0, ty = fy - y0;
    const float top = pixel(img, p, x0, y0, ch) * (1.0f - tx) + pixel(img, p, x0 + 1, y0, ch) * tx;
    const float bot = pixel(img, p, x0, y0 + 1, ch) * (1.0f - tx) + pixel(img, p, x0 + 1, y0 + 1, ch) * tx;
    v = top * (1.0f - ty) + bot * ty;
  } else {
    const int x0 = static_cast<int>(floorf(fx)), y0 = static_cast<int>(floorf(fy));
    const float tx = fx - x0, ty = fy - y0;
    v = 0.0f;
    for (int j = 0; j < 4; ++j) {
      float row = 0.0f;
      for (int i = 0; i < 4; ++i) row += cubic_weight(tx, i) * pixel(img, p, x0 - 1 + i, y0 - 1 + j, ch);
      v += cubic_weight(ty, j) * row;
    }
  }
  return (v * p.rescale - p.mean[ch]) * p.inv_std[ch];
}

}  // namespace image
}  // namespace afb
