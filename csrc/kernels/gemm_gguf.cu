// Fused GGUF-quantised matrix-vector product for decode batches (1..8 tokens):
//   out[m, n] = act( sum_k X[m, k] * dequant(W)[n, k] + bias[n] )
// with W kept in its GGUF block format (Q8_0, Q4_0, MXFP4, Q4_K, Q5_K, Q6_K: 4.25 - 8.5 bits per weight).  Every weight
// byte crosses HBM once and is expanded in registers; nothing is written back in expanded form.  Expanding to bf16
// and calling the dense GEMM instead moves 2 + 2 extra bytes per weight, several times the quantised size, which
// is what a batch of a few tokens is bound by.  This is the counterpart of the reference's mul_mv family
// (zig/pkg/inference/src/graph/quant_matmul.zig:17-60, backends/metal_kernels.m:2055-2331) and of its CUDA
// Q8_0 / Q4_0 / Q4_K linears (ops/cuda/artifacts/inference_cuda_kernels.cu:873-1553), which keep one thread per
// output and walk K serially.
//
// Work split: a CTA has four warps, a warp owns kMvRows consecutive output rows.  K is walked in chunks of 1024
// values = 32 sub-blocks of 32 values; in a chunk lane l owns sub-block l.  The chunk of X (all tokens) is staged
// once per CTA in shared memory as bf16 with rows padded to 40 elements, so the 16-byte reads of consecutive lanes
// fall into different bank groups; a lane reads its 32 activations per token once and reuses them for all of the
// warp's rows.  Per row the lane decodes its sub-block with the shared per-format decoder (common/gguf_elem.h,
// the code the host tests check) and accumulates in fp32; lanes are summed with shuffles at the end.
// Consecutive lanes read consecutive sub-blocks of a row, so a warp's weight reads are contiguous (a K-quant block
// is shared by eight lanes).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/gguf_elem.h"
#include "../common/tmap.cuh"

namespace afb {

constexpr int kMvWarps = 4;
constexpr int kMvRows = 2;       // output rows per warp
constexpr int kMvChunk = 1024;   // K values per staged chunk (one 32-value sub-block per lane)
constexpr int kMvPad = 40;       // bf16 elements per staged sub-block row (32 + 8 padding)

struct MvParams {
  const uint8_t* w;        // [N] rows of (K / block_values) blocks
  const __nv_bfloat16* x;  // [M, ldx]
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;      // [M, ldc]
  long ldx, ldc;
  int M, N, K, act;
};

__device__ __forceinline__ float mv_act(float v, int act) {
  switch (act) {
    case 1: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    case 2: {
      const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.0f + tanhf(u));
    }
    case 3: return fmaxf(v, 0.0f);
    case 4: return v / (1.0f + __expf(-v));
    default: return v;
  }
}

template <int TYPE, int MT>
__global__ void __launch_bounds__(kMvWarps * 32) gguf_mul_mv_kernel(const MvParams p) {
  extern __shared__ __align__(16) unsigned char mv_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(mv_smem);  // [MT][32 sub-blocks][kMvPad]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bv = static_cast<int>(gguf::block_values(TYPE));
  const int bb = static_cast<int>(gguf::block_bytes(TYPE));
  const long row_bytes = static_cast<long>(p.K / bv) * bb;
  const int n0 = (blockIdx.x * kMvWarps + warp) * kMvRows;

  float acc[kMvRows][MT];
#pragma unroll
  for (int r = 0; r < kMvRows; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

  for (int kc = 0; kc < p.K; kc += kMvChunk) {
    __syncthreads();  // the previous chunk has been consumed by every warp
    // stage X[:, kc : kc + 1024] (zero beyond K or M): 8 elements (16 bytes) per thread and step
    for (int i = threadIdx.x; i < MT * (kMvChunk / 8); i += kMvWarps * 32) {
      const int m = i / (kMvChunk / 8), c8 = i % (kMvChunk / 8);
      const int k = kc + c8 * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m < p.M && k < p.K) v = *reinterpret_cast<const uint4*>(p.x + static_cast<long>(m) * p.ldx + k);
      const int sub = c8 >> 2, within = (c8 & 3) * 8;
      *reinterpret_cast<uint4*>(xs + (m * 32 + sub) * kMvPad + within) = v;
    }
    __syncthreads();
    const int k0 = kc + lane * 32;  // this lane's sub-block
    if (k0 < p.K) {
      uint32_t xp[MT][16];  // this lane's 32 activations per token, as bf16 pairs
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4* src = reinterpret_cast<const uint4*>(xs + (m * 32 + lane) * kMvPad);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 raw = src[q];
          xp[m][q * 4 + 0] = raw.x; xp[m][q * 4 + 1] = raw.y; xp[m][q * 4 + 2] = raw.z; xp[m][q * 4 + 3] = raw.w;
        }
      }
      const int blk = k0 / bv, sub = (k0 % bv) / 32;
#pragma unroll
      for (int r = 0; r < kMvRows; ++r) {
        const int n = n0 + r;
        if (n >= p.N) continue;
        float wv[32];
        gguf::decode32(TYPE, p.w + static_cast<long>(n) * row_bytes + static_cast<long>(blk) * bb, sub, wv);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float s = 0.0f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // bf16 -> fp32 is a 16-bit shift: low half is element 2i, high half element 2i + 1
            s = fmaf(wv[2 * i], __uint_as_float(xp[m][i] << 16), s);
            s = fmaf(wv[2 * i + 1], __uint_as_float(xp[m][i] & 0xffff0000u), s);
          }
          acc[r][m] += s;
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kMvRows; ++r) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      const int n = n0 + r;
      if (lane == 0 && n < p.N && m < p.M) {
        if (p.bias) v += __bfloat162float(p.bias[n]);
        p.out[static_cast<long>(m) * p.ldc + n] = __float2bfloat16(mv_act(v, p.act));
      }
    }
  }
}

template <int TYPE>
int launch_mv(const MvParams& p, cudaStream_t stream) {
  const int rows_per_cta = kMvWarps * kMvRows;
  const unsigned grid = static_cast<unsigned>((p.N + rows_per_cta - 1) / rows_per_cta);
  const int mt = p.M <= 1 ? 1 : p.M <= 2 ? 2 : p.M <= 4 ? 4 : 8;
  const int smem = mt * 32 * kMvPad * 2;
  switch (mt) {
    case 1: gguf_mul_mv_kernel<TYPE, 1><<<grid, kMvWarps * 32, smem, stream>>>(p); break;
    case 2: gguf_mul_mv_kernel<TYPE, 2><<<grid, kMvWarps * 32, smem, stream>>>(p); break;
    case 4: gguf_mul_mv_kernel<TYPE, 4><<<grid, kMvWarps * 32, smem, stream>>>(p); break;
    default: gguf_mul_mv_kernel<TYPE, 8><<<grid, kMvWarps * 32, smem, stream>>>(p); break;
  }
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace afb

extern "C" {

// out [M, ldc] bf16 = act(X [M, ldx] bf16 @ dequant(W)^T + bias); W: N rows of K / block_values(type) GGUF blocks.
// M <= 8; K a multiple of the block size and of 8; act: 0 none, 1 gelu (erf), 2 gelu (tanh), 3 relu, 4 silu.
int afb_gguf_mul_mv(int type, const void* W, const void* X, const void* bias, void* out, int M, int N, int K, long ldx,
                    long ldc, int act, cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const long bv = gguf::block_values(type);
  if (bv < 0) {
    set_last_error("afb_gguf_mul_mv: GGUF tensor type %d has no fused kernel", type);
    return -1;
  }
  if (M > 8 || (K % bv) || (K & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(X) & 15)) {
    set_last_error("afb_gguf_mul_mv: needs M <= 8, K a multiple of %ld, ldx of 8, X 16-byte aligned (M=%d K=%d ldx=%ld)",
                   bv, M, K, ldx);
    return -1;
  }
  MvParams p;
  p.w = static_cast<const uint8_t*>(W); p.x = static_cast<const __nv_bfloat16*>(X);
  p.bias = static_cast<const __nv_bfloat16*>(bias); p.out = static_cast<__nv_bfloat16*>(out);
  p.ldx = ldx; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.act = act;
  switch (type) {
    case 8: return launch_mv<8>(p, stream);
    case 2: return launch_mv<2>(p, stream);
    case 39: return launch_mv<39>(p, stream);
    case 12: return launch_mv<12>(p, stream);
    case 13: return launch_mv<13>(p, stream);
    case 14: return launch_mv<14>(p, stream);
    default:
      set_last_error("afb_gguf_mul_mv: GGUF tensor type %d has no fused kernel", type);
      return -1;
  }
}

}  // extern "C"
