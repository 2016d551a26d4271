// Host path of the image preprocessing (crop, resize, normalise to planar fp32): the same per-sample code as the
// device kernel, looped over the output.  Used on machines without a GPU and as the oracle of the GPU test.
#include "../common/image_elem.h"

extern "C" {

int afb_image_preprocess_host(const uint8_t* img, int src_w, int src_h, int channels, float crop_x, float crop_y,
                              float crop_w, float crop_h, int out_w, int out_h, int mode, float rescale,
                              const float* mean3, const float* std3, float* out_chw) {
  if (!img || !out_chw || src_w <= 0 || src_h <= 0 || out_w <= 0 || out_h <= 0 || (channels != 3 && channels != 4) ||
      mode < 0 || mode > 2 || crop_w <= 0 || crop_h <= 0)
    return -1;
  afb::image::Params p;
  p.src_w = src_w; p.src_h = src_h; p.channels = channels;
  p.crop_x = crop_x; p.crop_y = crop_y; p.crop_w = crop_w; p.crop_h = crop_h;
  p.out_w = out_w; p.out_h = out_h; p.mode = mode; p.rescale = rescale;
  for (int c = 0; c < 3; ++c) { p.mean[c] = mean3[c]; p.inv_std[c] = 1.0f / std3[c]; }
  for (int ch = 0; ch < 3; ++ch)
    for (int y = 0; y < out_h; ++y)
      for (int x = 0; x < out_w; ++x)
        out_chw[(static_cast<long>(ch) * out_h + y) * out_w + x] = afb::image::sample(img, p, x, y, ch);
  return 0;
}

}  // extern "C"
