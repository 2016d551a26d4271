// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = act(alpha * A[M,K] · B[N,K]^T + bias) + residual.
//
// Both operands are K-major (row-major activations times row-major nn.Linear weights), which is the only
// GEMM shape the encoder and decoder models need.  Replaces the reference's scalar one-thread-per-output
// linears and their bias / GELU / ReLU / residual variants
// (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:20-388).
//
// Structure (one 128 x BN output tile per CTA, 6 warps):
//   warp 0      TMA producer: streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle) through a
//               STAGES-deep shared-memory ring guarded by full/empty mbarriers.
//   warp 1      allocates BN tensor-memory columns, then one lane issues tcgen05.mma (M=128, N=BN, K=16)
//               four times per stage and commits the stage's empty barrier; a final commit signals the
//               epilogue.
//   warps 2..5  epilogue: tcgen05.ld 32 lanes x 32 columns at a time, fused bias / activation / residual,
//               bf16 or fp32 stores.  Warp w owns TMEM lanes 32*(w%4)..+31.
//
// Split-K (gridDim.z > 1) writes fp32 partial tiles to out + z*M*ldc; the consumer sums them.
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

struct GemmParams {
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int M, N, K;
  int ldc, ldr;
  int act;      // 0 none, 1 gelu(erf), 2 gelu(tanh), 3 relu, 4 silu, 5 quick-gelu
  int out_f32;  // 1: fp32 output
  int kb_per_split;
  float alpha;
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case 1: return gelu_erf(v);
    case 2: return gelu_tanh(v);
    case 3: return fmaxf(v, 0.0f);
    case 4: return silu(v);
    case 5: return quick_gelu(v);
    default: return v;
  }
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = 128 * 64 * 2;
  static constexpr int kBBytes = BN * 64 * 2;
  static constexpr int kBarOffset = STAGES * (kABytes + kBBytes);
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 1) * 8 + 16 + 1024;  // + alignment slack
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 GemmParams p) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * L::kABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * 128;
  const int n0 = blockIdx.x * BN;
  const int num_kb_total = (p.K + 63) / 64;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(num_kb_total, kb_begin + p.kb_per_split);
  const int num_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BN);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, kStatusEmptyWaitTimeout)) break;
        mbar_expect_tx(&full[s], L::kABytes + L::kBBytes);
        tma_load_2d(sA + s * L::kABytes, &tma_a, &full[s], (kb_begin + i) * 64, m0);
        tma_load_2d(sB + s * L::kBBytes, &tma_b, &full[s], (kb_begin + i) * 64, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, BN);
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, kStatusTmaWaitTimeout)) break;
        tcgen05_fence_after();
        const uint64_t adesc = umma_desc_k_sw128(smem_u32(sA + s * L::kABytes));
        const uint64_t bdesc = umma_desc_k_sw128(smem_u32(sB + s * L::kBBytes));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // +32 bytes per K=16 step: the descriptor address field is in 16-byte units.
          umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0);
        }
        umma_commit(&empty[s]);
      }
      umma_commit(tmem_full);
    }
  } else {
    // Epilogue.
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    const bool ok = mbar_wait(tmem_full, 0, kStatusMmaWaitTimeout);
    tcgen05_fence_after();
    if (ok && num_kb > 0) {
      const bool partial = gridDim.z > 1;
      float* outf = reinterpret_cast<float*>(p.out) +
                    (partial ? static_cast<size_t>(blockIdx.z) * p.M * p.ldc : size_t(0));
      __nv_bfloat16* outh = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c, r);
        tmem_ld_wait();
        const int nbase = n0 + c;
        if (row < p.M && nbase < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          const bool full_chunk = (nbase + 32 <= p.N);
          if (!partial) {
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (full_chunk || nbase + j < p.N) v[j] += __bfloat162float(p.bias[nbase + j]);
            }
            // Chosen once per chunk, outside the element loop (a per-element switch is if-converted into
            // evaluating every activation for every element).
            if (p.act == 1) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
            } else if (p.act == 2) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
            } else if (p.act == 3) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
            } else if (p.act == 4) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = silu(v[j]);
            } else if (p.act == 5) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = quick_gelu(v[j]);
            }
            if (p.residual) {
              const __nv_bfloat16* rp = p.residual + static_cast<size_t>(row) * p.ldr + nbase;
              if (full_chunk && (p.ldr & 7) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 u = reinterpret_cast<const uint4*>(rp)[j];
                  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z),
                         d = unpack_bf16x2(u.w);
                  v[8 * j + 0] += a.x; v[8 * j + 1] += a.y; v[8 * j + 2] += b.x; v[8 * j + 3] += b.y;
                  v[8 * j + 4] += cc.x; v[8 * j + 5] += cc.y; v[8 * j + 6] += d.x; v[8 * j + 7] += d.y;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (nbase + j < p.N) v[j] += __bfloat162float(rp[j]);
              }
            }
          }
          if (partial || p.out_f32) {
            float* op = outf + static_cast<size_t>(row) * p.ldc + nbase;
            if (full_chunk && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                reinterpret_cast<float4*>(op)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nbase + j < p.N) op[j] = v[j];
            }
          } else {
            __nv_bfloat16* op = outh + static_cast<size_t>(row) * p.ldc + nbase;
            if (full_chunk && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 u;
                u.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
                u.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                u.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                u.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                reinterpret_cast<uint4*>(op)[j] = u;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nbase + j < p.N) op[j] = __float2bfloat16(v[j]);
            }
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, BN);
}

template <int BN, int STAGES>
int launch_gemm(const void* A, const void* B, GemmParams p, int lda, int ldb, int splits, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  CUtensorMap ta, tb;
  if (make_tmap_2d(&ta, A, 2, p.M, p.K, static_cast<uint64_t>(lda) * 2, 128, 64, 3)) return -1;
  if (make_tmap_2d(&tb, B, 2, p.N, p.K, static_cast<uint64_t>(ldb) * 2, BN, 64, 3)) return -1;
  static_assert(static_cast<long>(BN) * 227 * 1024 <= 512L * L::kTotal,
                "tensor-memory share of a CTA exceeds its shared-memory share");
  AFB_CONFIGURE_KERNEL((gemm_bf16_kernel<BN, STAGES>), L::kTotal, 192, BN);
  dim3 grid((p.N + BN - 1) / BN, (p.M + 127) / 128, splits);
  gemm_bf16_kernel<BN, STAGES><<<grid, 192, L::kTotal, stream>>>(ta, tb, p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace afb

extern "C" {

// C = act(alpha * A · B^T + bias) + residual.  A [M,K] (row pitch lda), B [N,K] (row pitch ldb), bf16.
// out: bf16 [M,ldc], or fp32 when out_f32 != 0.  split_k > 1: out must be fp32 [split_k, M, ldc]; bias,
// activation and residual are then left to the consumer of the partial sums.
// tile_n: 0 = choose, else 64 / 128 / 256.
int afb_gemm_bf16(const void* A, const void* B, void* out, const void* bias, const void* residual, int M, int N,
                  int K, int lda, int ldb, int ldc, int ldr, int act, int out_f32, int split_k, float alpha,
                  int tile_n, cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (lda & 7) || (ldb & 7)) {
    set_last_error("afb_gemm_bf16: K, lda and ldb must be multiples of 8 (got %d, %d, %d)", K, lda, ldb);
    return -1;
  }
  const int num_kb = (K + 63) / 64;
  if (split_k < 1) split_k = 1;
  if (split_k > num_kb) split_k = num_kb;
  int kb_per = (num_kb + split_k - 1) / split_k;
  split_k = (num_kb + kb_per - 1) / kb_per;  // every split gets at least one K block
  GemmParams p;
  p.out = out;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr; p.act = act; p.out_f32 = out_f32;
  p.kb_per_split = kb_per;
  p.alpha = alpha;
  if (tile_n == 0) {
    const long tiles256 = static_cast<long>((M + 127) / 128) * ((N + 255) / 256);
    if (N <= 64) tile_n = 64;
    else if (N <= 128 || tiles256 * split_k < 120) tile_n = 128;
    else tile_n = 256;
  }
  switch (tile_n) {
    case 64: return launch_gemm<64, 8>(A, B, p, lda, ldb, split_k, stream);
    case 128: return launch_gemm<128, 6>(A, B, p, lda, ldb, split_k, stream);
    case 256: return launch_gemm<256, 4>(A, B, p, lda, ldb, split_k, stream);
    default: set_last_error("afb_gemm_bf16: tile_n must be 0, 64, 128 or 256"); return -1;
  }
}

// Number of splits afb_gemm_bf16 will actually use for (K, split_k): lets the caller size the partial buffer.
int afb_gemm_effective_splits(int K, int split_k) {
  const int num_kb = (K + 63) / 64;
  if (split_k < 1) split_k = 1;
  if (split_k > num_kb) split_k = num_kb;
  int kb_per = (num_kb + split_k - 1) / split_k;
  return (num_kb + kb_per - 1) / kb_per;
}

}  // extern "C"
