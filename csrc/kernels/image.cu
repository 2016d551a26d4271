// Image preprocessing on the GPU for the vision towers (CLIP-style): crop -> resize -> rescale -> normalise, from
// interleaved 8-bit HWC to planar CHW fp32 or bf16, a batch of equally sized images per launch.  One thread per
// output pixel computes the three channels (the neighbours' bytes are shared by the channels, so they stay in
// L1); the per-sample arithmetic is csrc/common/image_elem.h, shared with the host path.
// Counterpart of the reference's CPU preprocessing (zig/lib/image/src/processing.zig:41-177).
#include <cuda_bf16.h>

#include "../common/image_elem.h"
#include "../common/tmap.cuh"

namespace afb {

template <typename OutT>
__global__ void image_preprocess_kernel(const uint8_t* __restrict__ imgs, OutT* __restrict__ out, image::Params p,
                                        int batch) {
  const long per_img_in = static_cast<long>(p.src_w) * p.src_h * p.channels;
  const long plane = static_cast<long>(p.out_w) * p.out_h;
  const long total = plane * batch;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int b = static_cast<int>(i / plane);
    const long r = i - b * plane;
    const int oy = static_cast<int>(r / p.out_w), ox = static_cast<int>(r - static_cast<long>(oy) * p.out_w);
    const uint8_t* img = imgs + b * per_img_in;
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) {
      const float v = image::sample(img, p, ox, oy, ch);
      const long o = (static_cast<long>(b) * 3 + ch) * plane + r;
      if constexpr (sizeof(OutT) == 2) out[o] = __float2bfloat16(v);
      else out[o] = v;
    }
  }
}

}  // namespace afb

extern "C" {

// imgs: [batch, src_h, src_w, channels] uint8; out: [batch, 3, out_h, out_w] fp32 (out_bf16 = 0) or bf16 (1).
int afb_image_preprocess(const void* imgs, int batch, int src_w, int src_h, int channels, float crop_x, float crop_y,
                         float crop_w, float crop_h, int out_w, int out_h, int mode, float rescale,
                         const float* mean3, const float* std3, void* out, int out_bf16, cudaStream_t stream) {
  using namespace afb;
  if (batch <= 0) return 0;
  if (src_w <= 0 || src_h <= 0 || out_w <= 0 || out_h <= 0 || (channels != 3 && channels != 4) || mode < 0 ||
      mode > 2 || crop_w <= 0 || crop_h <= 0) {
    set_last_error("afb_image_preprocess: bad geometry (src %dx%dx%d, out %dx%d, mode %d)", src_w, src_h, channels,
                   out_w, out_h, mode);
    return -1;
  }
  image::Params p;
  p.src_w = src_w; p.src_h = src_h; p.channels = channels;
  p.crop_x = crop_x; p.crop_y = crop_y; p.crop_w = crop_w; p.crop_h = crop_h;
  p.out_w = out_w; p.out_h = out_h; p.mode = mode; p.rescale = rescale;
  for (int c = 0; c < 3; ++c) { p.mean[c] = mean3[c]; p.inv_std[c] = 1.0f / std3[c]; }
  const long total = static_cast<long>(out_w) * out_h * batch;
  long blocks = (total + 255) / 256;
  if (blocks > 148L * 16) blocks = 148L * 16;
  if (out_bf16)
    image_preprocess_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint8_t*>(imgs), static_cast<__nv_bfloat16*>(out), p, batch);
  else
    image_preprocess_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint8_t*>(imgs), static_cast<float*>(out), p, batch);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
