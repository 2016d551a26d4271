// Block-scaled fp8 weight GEMM with bf16 activations:  out[t, n] = sum_k X[t, k] * (W8[n, k] * 2^(S[k/32, n]-127)).
//
// Weights are stored as e4m3 bytes with one e8m0 power-of-two scale per 32 elements along K (the MX block
// format: zig/pkg/inference/src/gguf/tensor_types.zig MXFP4/MX layouts use the same e8m0 block scale); the
// scale array is laid out [K/32, N] so a tile's scales are one contiguous TMA box.  This is the decoder's
// linear layer: at decode it streams every weight byte exactly once at HBM speed, at prefill it is
// tensor-core bound.
//
// The tile is "swapped": the weight rows (output features) occupy the 128 lanes of the UMMA M dimension and
// the tokens are the UMMA N dimension (BT = 16..256), so a decode batch of 64 tokens wastes no tensor-core
// rows and no tensor memory.  Eleven warps:
//   warp 0      TMA producer for raw fp8 weight tiles (128 x 64 bytes) + their 2 x 128 scale bytes, RAW-deep ring
//   warp 1      tensor-memory owner and tcgen05.mma issuer
//   warps 2..9  dequantise raw fp8 -> bf16 into a 128-byte-swizzled UMMA operand tile (the XOR pattern TMA would
//               have produced), publish it to the async proxy; warps 2..5 later run the epilogue
//   warp 10     TMA producer for the activation tiles (BT x 64 bf16, 128-byte swizzle), its own XST-deep ring so
//               the L2 latency of an activation tile never sits on the MMA critical path
// Epilogue modes: bf16 out (+bias, activation, residual), fp32 split-K partials, or SwiGLU over interleaved
// gate/up rows (row 2i = gate_i, row 2i+1 = up_i -> out[t, i] = silu(gate) * up).
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

// Kept out of line so the unrolled epilogue does not evaluate every activation for every element.
__device__ __noinline__ float act_one_w8(float x, int act) {
  switch (act) {
    case 1: return gelu_erf(x);
    case 2: return gelu_tanh(x);
    case 3: return fmaxf(x, 0.0f);
    case 4: return silu(x);
    default: return x;
  }
}

struct W8Params {
  void* out;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  int M, N, K;                    // tokens, out features, in features
  int ldc, ldr;
  int act;
  int mode;  // 0 bf16 out, 1 fp32 partials [split][M][ldc], 2 swiglu (out is [M, N/2])
  int kb_per_split;
};

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <int BT, int RAW, int ST, int XST>
struct W8Smem {
  static constexpr int kRawBytes = 128 * 64;       // fp8 tile
  static constexpr int kScaleBytes = 2 * 128;      // two 32-wide K blocks x 128 rows
  static constexpr int kRawStage = kRawBytes + kScaleBytes + 768;  // keep stages 1024-byte multiples
  static constexpr int kWBytes = 128 * 64 * 2;     // dequantised bf16 tile
  static constexpr int kXBytes = BT * 64 * 2;
  static constexpr int kXStage = (kXBytes + 1023) / 1024 * 1024;
  static constexpr int kRawOff = 0;
  static constexpr int kWOff = kRawOff + RAW * kRawStage;
  static constexpr int kXOff = kWOff + ST * kWBytes;
  static constexpr int kBarOff = kXOff + XST * kXStage;
  static constexpr int kNumBars = 2 * RAW + 2 * ST + 2 * XST + 1;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16 + 1024;
};

template <int BT, int RAW, int ST, int XST>
__global__ void __launch_bounds__(352, (BT <= 64 ? 2 : 1))
gemm_w8a16_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_s,
                  const __grid_constant__ CUtensorMap tma_x, W8Params p) {
  using L = W8Smem<BT, RAW, ST, XST>;
  constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* raw_full = bars;
  uint64_t* raw_empty = raw_full + RAW;
  uint64_t* x_full = raw_empty + RAW;
  uint64_t* x_empty = x_full + XST;
  uint64_t* w_ready = x_empty + XST;
  uint64_t* mma_done = w_ready + ST;
  uint64_t* tmem_full = mma_done + ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int t0 = blockIdx.y * BT;
  const int num_kb_total = (p.K + 63) / 64;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(num_kb_total, kb_begin + p.kb_per_split);
  const int num_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RAW; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 256);
    }
    for (int s = 0; s < XST; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&x_empty[s], 1);
    }
    for (int s = 0; s < ST; ++s) {
      mbar_init(&w_ready[s], 256);
      mbar_init(&mma_done[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tma_w);
    tma_prefetch_desc(&tma_s);
    tma_prefetch_desc(&tma_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < num_kb; ++i) {
        const int r = i % RAW;
        const uint32_t ph = (i / RAW) & 1;
        if (!mbar_wait(&raw_empty[r], ph ^ 1, kStatusEmptyWaitTimeout)) break;
        uint8_t* dst = smem + L::kRawOff + r * L::kRawStage;
        mbar_expect_tx(&raw_full[r], L::kRawBytes + L::kScaleBytes);
        tma_load_2d(dst, &tma_w, &raw_full[r], (kb_begin + i) * 64, n0);
        tma_load_2d(dst + L::kRawBytes, &tma_s, &raw_full[r], n0, (kb_begin + i) * 2);
      }
    }
  } else if (warp == 10) {
    if (lane == 0) {
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % XST;
        const uint32_t ph = (i / XST) & 1;
        if (!mbar_wait(&x_empty[s], ph ^ 1, kStatusEmptyWaitTimeout)) break;
        mbar_expect_tx(&x_full[s], L::kXBytes);
        tma_load_2d(smem + L::kXOff + s * L::kXStage, &tma_x, &x_full[s], (kb_begin + i) * 64, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, BT);
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % ST;
        const uint32_t ph = (i / ST) & 1;
        const int xs = i % XST;
        const uint32_t xph = (i / XST) & 1;
        if (!mbar_wait(&x_full[xs], xph, kStatusTmaWaitTimeout)) break;
        if (!mbar_wait(&w_ready[s], ph, kStatusDequantWaitTimeout)) break;
        tcgen05_fence_after();
        const uint64_t adesc = umma_desc_k_sw128(smem_u32(smem + L::kWOff + s * L::kWBytes));
        const uint64_t bdesc = umma_desc_k_sw128(smem_u32(smem + L::kXOff + xs * L::kXStage));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0);
        umma_commit(&mma_done[s]);
        umma_commit(&x_empty[xs]);
      }
      umma_commit(tmem_full);
    }
  } else {
    // ---- dequantise: 256 threads, thread handles 16-byte chunk (tid & 3) of rows (tid >> 2) + 64*j ----
    const int tid = threadIdx.x - 64;
    const int chunk = tid & 3;
    const int rbase = tid >> 2;
    bool alive = true;
    for (int i = 0; i < num_kb && alive; ++i) {
      const int r = i % RAW;
      const uint32_t rph = (i / RAW) & 1;
      const int s = i % ST;
      const uint32_t sph = (i / ST) & 1;
      alive = mbar_wait(&raw_full[r], rph, kStatusTmaWaitTimeout) &&
              mbar_wait(&mma_done[s], sph ^ 1, kStatusEmptyWaitTimeout);
      if (!alive) break;
      const uint8_t* raw = smem + L::kRawOff + r * L::kRawStage;
      const uint8_t* sc = raw + L::kRawBytes;
      uint8_t* wdst = smem + L::kWOff + s * L::kWBytes;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int row = rbase + 64 * j;
        const uint4 v = *reinterpret_cast<const uint4*>(raw + row * 64 + chunk * 16);
        // e4m3 -> bf16 without conversion instructions: the 7 exponent+mantissa bits dropped into bf16 bit
        // positions 10..4 read as the same value times 2^-120 (subnormals included), so one packed bf16
        // multiply by 2^120 * block_scale finishes the job exactly.
        const uint32_t e8 = sc[(chunk >> 1) * 128 + row];
        const uint32_t sb = min(e8 + 120u, 254u) << 7;
        const uint32_t scale2 = sb | (sb << 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t lo = __byte_perm(w[q], 0u, 0x1404);  // bytes 0,1 -> high byte of each 16-bit lane
          const uint32_t hi = __byte_perm(w[q], 0u, 0x3424);  // bytes 2,3
          const uint32_t blo = ((lo >> 4) & 0x07F007F0u) | (lo & 0x80008000u);
          const uint32_t bhi = ((hi >> 4) & 0x07F007F0u) | (hi & 0x80008000u);
          o[2 * q] = bf16x2_mul(blo, scale2);
          o[2 * q + 1] = bf16x2_mul(bhi, scale2);
        }
        // bf16 row is 128 bytes = 8 chunks of 16 bytes; this thread produced chunks 2*chunk and 2*chunk+1.
        const int c0 = (2 * chunk) ^ (row & 7);
        const int c1 = (2 * chunk + 1) ^ (row & 7);
        *reinterpret_cast<uint4*>(wdst + row * 128 + c0 * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(wdst + row * 128 + c1 * 16) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&w_ready[s]);
      mbar_arrive(&raw_empty[r]);
    }

    // ---- epilogue (first four dequant warps): lane = output feature, registers = tokens ----
    if (warp < 6) {
    const int q = warp & 3;
    const int n = n0 + q * 32 + lane;
    const bool ok = mbar_wait(tmem_full, 0, kStatusMmaWaitTimeout);
    tcgen05_fence_after();
    if (ok && num_kb > 0) {
      const float bias = (p.bias && p.mode != 1 && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
      constexpr int CH = BT < 32 ? 16 : 32;
#pragma unroll 1
      for (int c = 0; c < BT; c += CH) {
        float v[CH];
        if constexpr (CH == 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        } else {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        }
        if (p.mode == 1) {
          float* op = reinterpret_cast<float*>(p.out) + static_cast<size_t>(blockIdx.z) * p.M * p.ldc;
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int t = t0 + c + j;
              if (t < p.M) op[static_cast<size_t>(t) * p.ldc + n] = v[j];
            }
          }
        } else if (p.mode == 2) {
          // even lane holds gate_i, odd lane holds up_i for feature i = n/2.
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const float mine = v[j] + bias;
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            const int t = t0 + c + j;
            // even lanes write even tokens, odd lanes odd tokens: both lanes of a pair stay busy.
            if (((lane ^ j) & 1) == 0 && t < p.M && n < p.N) {
              const float g = (lane & 1) ? other : mine;
              const float u = (lane & 1) ? mine : other;
              op[static_cast<size_t>(t) * p.ldc + (n >> 1)] = __float2bfloat16(silu(g) * u);
            }
          }
        } else {
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out);
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int t = t0 + c + j;
              if (t < p.M) {
                float x = v[j] + bias;
                if (p.act) x = act_one_w8(x, p.act);
                if (p.residual) x += __bfloat162float(p.residual[static_cast<size_t>(t) * p.ldr + n]);
                op[static_cast<size_t>(t) * p.ldc + n] = __float2bfloat16(x);
              }
            }
          }
        }
      }
    }
    }  // epilogue warps
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int BT, int RAW, int ST, int XST>
int launch_w8(const void* W, const void* S, const void* X, W8Params p, int ldx, int splits, cudaStream_t stream) {
  using L = W8Smem<BT, RAW, ST, XST>;
  CUtensorMap tw, ts, tx;
  if (make_tmap_2d(&tw, W, 1, p.N, p.K, static_cast<uint64_t>(p.K), 128, 64, 0)) return -1;
  if (make_tmap_2d(&ts, S, 1, p.K / 32, p.N, static_cast<uint64_t>(p.N), 2, 128, 0)) return -1;
  if (make_tmap_2d(&tx, X, 2, p.M, p.K, static_cast<uint64_t>(ldx) * 2, BT, 64, 3)) return -1;
  {
    constexpr int TMEM_COLS = BT < 32 ? 32 : BT;  // as in the kernel
    static_assert(static_cast<long>(TMEM_COLS) * 227 * 1024 <= 512L * L::kTotal,
                  "tensor-memory share of a CTA exceeds its shared-memory share");
    AFB_CONFIGURE_KERNEL((gemm_w8a16_kernel<BT, RAW, ST, XST>), L::kTotal, 352, TMEM_COLS);
  }
  dim3 grid((p.N + 127) / 128, (p.M + BT - 1) / BT, splits);
  gemm_w8a16_kernel<BT, RAW, ST, XST><<<grid, 352, L::kTotal, stream>>>(tw, ts, tx, p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace afb

extern "C" {

// X [M, K] bf16 (row pitch ldx); W8 [N, K] e4m3 bytes; S [K/32, N] e8m0 bytes.
// mode 0: out bf16 [M, ldc] = act(X W^T + bias) + residual
// mode 1: out fp32 [split_k, M, ldc] partial sums (split_k >= 1)
// mode 2: out bf16 [M, ldc] with N/2 columns = silu(gate) * up over interleaved rows
int afb_gemm_w8a16(const void* X, const void* W8, const void* S, void* out, const void* bias, const void* residual,
                   int M, int N, int K, int ldx, int ldc, int ldr, int act, int mode, int split_k,
                   cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 32) || (ldx & 7) || (N & 15) || (K & 15)) {
    set_last_error("afb_gemm_w8a16: K must be a multiple of 32, N of 16, ldx of 8 (got K=%d N=%d ldx=%d)", K, N,
                   ldx);
    return -1;
  }
  const int num_kb = (K + 63) / 64;
  if (split_k < 1) split_k = 1;
  if (split_k > num_kb) split_k = num_kb;
  int kb_per = (num_kb + split_k - 1) / split_k;
  split_k = (num_kb + kb_per - 1) / kb_per;
  if (mode != 1 && split_k != 1) {
    set_last_error("afb_gemm_w8a16: split_k > 1 needs mode 1 (fp32 partials)");
    return -1;
  }
  W8Params p;
  p.out = out;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr; p.act = act; p.mode = mode; p.kb_per_split = kb_per;
  // Small token tiles keep the footprint under half an SM's shared memory so two CTAs are co-resident.
  if (M <= 16) return launch_w8<16, 5, 2, 6>(W8, S, X, p, ldx, split_k, stream);
  if (M <= 32) return launch_w8<32, 5, 2, 6>(W8, S, X, p, ldx, split_k, stream);
  if (M <= 64) return launch_w8<64, 4, 3, 3>(W8, S, X, p, ldx, split_k, stream);
  if (M <= 128) return launch_w8<128, 4, 2, 4>(W8, S, X, p, ldx, split_k, stream);
  return launch_w8<256, 3, 2, 4>(W8, S, X, p, ldx, split_k, stream);
}

}  // extern "C"
