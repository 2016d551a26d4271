// Gated MLP activation in one pass:  out[t, j] = act(gate[t, j]) * up[t, j]  (bf16 in, fp32 arithmetic, bf16 out).
//
// The decoder families whose gated MLP does not run through the block-fp8 SwiGLU GEMM (GeGLU of Gemma and
// ModernBERT, T5 v1.1's gated GELU, BitNet's squared ReLU, DeepSeek-V4's clamped SwiGLU, the per-sequence models)
// produce gate and up with one bf16 GEMM and then need this elementwise step; as tensor ops it is a chain of four
// launches that each re-read and re-write the [T, F] activations.  The reference folds the same step into its
// feed-forward (zig/pkg/inference/src/architectures/gpt.zig:5416 feedForward; gated variants by activation).
//
// Layouts of the GEMM output: halves (gate = columns [0, F), up = [F, 2F)) or interleaved (gate_j, up_j adjacent:
// the order the fused SwiGLU weights are packed in).  Memory-bound: 16-byte loads and stores when F, the row
// pitches and the base addresses allow, scalar otherwise.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

// 1 gelu, 2 gelu(tanh), 3 relu, 4 silu, 5 quick-gelu, 6 squared relu
__device__ __forceinline__ float gate_act(float g, int act) {
  switch (act) {
    case 1: return gelu_erf(g);
    case 2: return gelu_tanh(g);
    case 3: return fmaxf(g, 0.0f);
    case 4: return silu(g);
    case 5: return quick_gelu(g);
    case 6: { const float r = fmaxf(g, 0.0f); return r * r; }
    default: return g;
  }
}

struct GatedActParams {
  const __nv_bfloat16* gate;
  const __nv_bfloat16* up;
  __nv_bfloat16* out;
  long ld_in, ld_out;  // row pitches in elements (gate and up share one)
  long T;
  int F, act, interleaved;
  float limit;  // > 0: gate <- min(gate, limit), up <- clamp(up, -limit, limit) before the activation
};

__device__ __forceinline__ float gated_one(float g, float u, const GatedActParams& p) {
  if (p.limit > 0.0f) {
    g = fminf(g, p.limit);
    u = fminf(fmaxf(u, -p.limit), p.limit);
  }
  return gate_act(g, p.act) * u;
}

// One thread per 8 output columns.
__global__ void __launch_bounds__(256) gated_act_vec_kernel(const GatedActParams p) {
  const long groups_per_row = p.F / 8;
  const long total = p.T * groups_per_row;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / groups_per_row;
    const int c = static_cast<int>(i % groups_per_row) * 8;
    float g[8], u[8];
    if (p.interleaved) {
      // columns 2c .. 2c + 15 of the row hold (gate, up) pairs of outputs c .. c + 7
      const uint4 a = *reinterpret_cast<const uint4*>(p.gate + t * p.ld_in + 2 * c);
      const uint4 b = *reinterpret_cast<const uint4*>(p.gate + t * p.ld_in + 2 * c + 8);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(pa[j]), y = __bfloat1622float2(pb[j]);
        g[j] = x.x; u[j] = x.y;
        g[4 + j] = y.x; u[4 + j] = y.y;
      }
    } else {
      const uint4 a = *reinterpret_cast<const uint4*>(p.gate + t * p.ld_in + c);
      const uint4 b = *reinterpret_cast<const uint4*>(p.up + t * p.ld_in + c);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(pa[j]), y = __bfloat1622float2(pb[j]);
        g[2 * j] = x.x; g[2 * j + 1] = x.y;
        u[2 * j] = y.x; u[2 * j + 1] = y.y;
      }
    }
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      po[j] = __floats2bfloat162_rn(gated_one(g[2 * j], u[2 * j], p), gated_one(g[2 * j + 1], u[2 * j + 1], p));
    *reinterpret_cast<uint4*>(p.out + t * p.ld_out + c) = o;
  }
}

// Any F, any alignment: one thread per output element.
__global__ void __launch_bounds__(256) gated_act_scalar_kernel(const GatedActParams p) {
  const long total = p.T * p.F;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / p.F;
    const int c = static_cast<int>(i % p.F);
    float g, u;
    if (p.interleaved) {
      g = __bfloat162float(p.gate[t * p.ld_in + 2 * c]);
      u = __bfloat162float(p.gate[t * p.ld_in + 2 * c + 1]);
    } else {
      g = __bfloat162float(p.gate[t * p.ld_in + c]);
      u = __bfloat162float(p.up[t * p.ld_in + c]);
    }
    p.out[t * p.ld_out + c] = __float2bfloat16(gated_one(g, u, p));
  }
}

}  // namespace afb

extern "C" {

// out [T, F] = act(gate) * up.  interleaved = 1: `gate` points at a [T, 2F] matrix whose columns alternate
// gate_j, up_j and `up` is ignored; 0: `gate` and `up` are two [T, F] views with the same row pitch ld_in (the two
// halves of one GEMM output, or separate tensors).  act: 1 gelu, 2 gelu(tanh), 3 relu, 4 silu, 5 quick-gelu,
// 6 squared relu.  limit > 0 clamps gate from above and up to [-limit, limit] first.
int afb_gated_act(const void* gate, const void* up, void* out, long ld_in, long ld_out, long T, int F, int act,
                  int interleaved, float limit, cudaStream_t stream) {
  using namespace afb;
  if (T <= 0 || F <= 0) return 0;
  if (act < 1 || act > 6 || (!interleaved && up == nullptr) || ld_out < F || ld_in < (interleaved ? 2L * F : F)) {
    set_last_error("afb_gated_act: bad arguments (act=%d F=%d ld_in=%ld ld_out=%ld interleaved=%d)", act, F, ld_in,
                   ld_out, interleaved);
    return -1;
  }
  GatedActParams p;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.up = static_cast<const __nv_bfloat16*>(interleaved ? gate : up);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ld_in = ld_in; p.ld_out = ld_out; p.T = T; p.F = F; p.act = act; p.interleaved = interleaved; p.limit = limit;
  const bool aligned = (F % 8 == 0) && (ld_in % 8 == 0) && (ld_out % 8 == 0) &&
                       ((reinterpret_cast<uintptr_t>(p.gate) | reinterpret_cast<uintptr_t>(p.up) |
                         reinterpret_cast<uintptr_t>(p.out)) & 15) == 0;
  const long work = aligned ? T * (F / 8) : T * static_cast<long>(F);
  const long blocks = (work + 255) / 256;
  const unsigned grid = static_cast<unsigned>(blocks < 148L * 16 ? blocks : 148L * 16);
  if (aligned)
    gated_act_vec_kernel<<<grid, 256, 0, stream>>>(p);
  else
    gated_act_scalar_kernel<<<grid, 256, 0, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
