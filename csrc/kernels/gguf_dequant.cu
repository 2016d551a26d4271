// GGUF block formats expanded on the GPU (artifact-format parity for quantised checkpoints: Q8_0, Q4_0, Q4_K,
// Q5_K, Q6_K, MXFP4): raw block bytes -> bf16 (or fp32) elements, one element per thread in a grid-stride loop,
// using the same per-element decoders the host path is checked with.  The expanded tile then feeds the tcgen05
// GEMMs, or is re-packed once at load time into the block-fp8 layout the decode kernels stream.
// Counterpart of the reference's Q8_0 / Q4_0 / Q4_K linears
// (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:873-1553), which decode inside a scalar
// dot-product loop.
#include <cuda_bf16.h>

#include "../common/gguf_elem.h"
#include "../common/tmap.cuh"

namespace afb {

template <typename OutT>
__global__ void gguf_dequant_kernel(int type, const uint8_t* __restrict__ src, OutT* __restrict__ dst, long n,
                                    int bv, int bb) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long blk = i / bv;
    const int j = static_cast<int>(i - blk * bv);
    const float v = gguf::element(type, src + blk * bb, j);
    if constexpr (sizeof(OutT) == 2) dst[i] = __float2bfloat16(v);
    else dst[i] = v;
  }
}

}  // namespace afb

extern "C" {

// src: n_values / block_values(type) blocks; dst: bf16 (out_f32 = 0) or fp32 (1), n_values elements.
int afb_gguf_dequant_device(int type, const void* src, void* dst, long n_values, int out_f32, cudaStream_t stream) {
  using namespace afb;
  const long bv = gguf::block_values(type), bb = gguf::block_bytes(type);
  if (bv < 0) {
    set_last_error("afb_gguf_dequant_device: unsupported GGUF tensor type %d", type);
    return -1;
  }
  if (n_values <= 0) return 0;
  if (n_values % bv) {
    set_last_error("afb_gguf_dequant_device: %ld values is not a whole number of %ld-value blocks", n_values, bv);
    return -1;
  }
  long blocks = (n_values + 255) / 256;
  if (blocks > 148L * 32) blocks = 148L * 32;
  if (out_f32)
    gguf_dequant_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        type, static_cast<const uint8_t*>(src), static_cast<float*>(dst), n_values, static_cast<int>(bv),
        static_cast<int>(bb));
  else
    gguf_dequant_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        type, static_cast<const uint8_t*>(src), static_cast<__nv_bfloat16*>(dst), n_values, static_cast<int>(bv),
        static_cast<int>(bb));
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
