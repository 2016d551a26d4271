// Persistent bf16 GEMM  S[M,N] = A[M,K] · B[N,K]^T  with the accumulator double-buffered in tensor memory, so the
// epilogue of one 128x256 tile runs while the tensor core is already working on the next.  One CTA per SM walks
// a list of tiles; what happens to a finished tile is a compile-time "mode":
//
//   kStore    C = act(alpha*S + bias) + residual, bf16 or fp32              (encoder / decoder linears)
//   kFilter   vector search: keep scores whose distance beats the query's current threshold and append
//             (distance, column) to that query's candidate list -- the score matrix is never written
//   kArgmin   k-means assignment: running arg-min over all centroid tiles of  ||c||^2 - 2 x·c  per point
//
// kFilter / kArgmin replace the reference's CPU scoring loops and its thread-per-point Metal k-means kernel
// (zig/lib/vector/src/vector.zig:267-500, zig/lib/vectorindex/src/kmeans.zig:222, kmeans_metal.m:115); kStore is
// the throughput version of gemm_bf16.cu.
//
// Warp roles: 0 TMA producer (ring of STAGES 128x64 + 256x64 tiles, 128-byte swizzle), 1 tcgen05.mma issuer
// (owns all 512 tensor-memory columns: two 256-column accumulators), 2..9 epilogue: two warpgroups that split
// the tile's 256 columns (warp w reads TMEM lanes 32*(w%4)..+31; a lane is one row of the tile).
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

enum PersistMode : int { kStore = 0, kFilter = 1, kArgmin = 2 };

struct PersistParams {
  int M, N, K;
  int m_tiles, n_tiles;
  // kStore
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int ldc, ldr, act, out_f32;
  float alpha;
  // kFilter / kArgmin: distance = row_term[m] + col_term[n] + scale * S  (any of the term pointers may be null)
  const float* row_term;
  const float* col_term;
  float scale;
  // kFilter
  const float* threshold;  // [M] keep distance < threshold[m]
  float* cand_val;         // [M, cap]
  int* cand_idx;           // [M, cap]
  int* cand_count;         // [M]
  int cap;
  long col_offset;         // added to the column index (shard offset)
  int clamp_zero;          // l2: clamp distance at 0
  // kArgmin
  int* assign;             // [M]
  float* best;             // [M]
};

constexpr int kPBN = 256;
constexpr int kPStages = 4;
constexpr int kPABytes = 128 * 64 * 2;
constexpr int kPBBytes = kPBN * 64 * 2;
constexpr int kPBarOff = kPStages * (kPABytes + kPBBytes);
constexpr int kPSmem = kPBarOff + (2 * kPStages + 4) * 8 + 16 + 1024;

__device__ __forceinline__ float persist_act(float v, int act) {
  switch (act) {
    case 1: return gelu_erf(v);
    case 2: return gelu_tanh(v);
    case 3: return fmaxf(v, 0.0f);
    case 4: return silu(v);
    case 5: return quick_gelu(v);
    default: return v;
  }
}

// Tile order.  kStore / kFilter: linear tile index, the M tiles of one B tile adjacent so a B tile (the big
// operand in search) is fetched from HBM once and re-read from L2.  kArgmin: a CTA owns whole rows of tiles
// (every N tile of an M tile, in order) because its epilogue carries a running arg-min across them.
template <int MODE>
__device__ __forceinline__ bool tile_at(const PersistParams& p, long it, int& m_tile, int& n_tile) {
  if (MODE == kArgmin) {
    const long mt = blockIdx.x + (it / p.n_tiles) * gridDim.x;
    if (mt >= p.m_tiles) return false;
    m_tile = static_cast<int>(mt);
    n_tile = static_cast<int>(it % p.n_tiles);
    return true;
  }
  const long idx = blockIdx.x + it * gridDim.x;
  if (idx >= static_cast<long>(p.m_tiles) * p.n_tiles) return false;
  n_tile = static_cast<int>(idx / p.m_tiles);
  m_tile = static_cast<int>(idx % p.m_tiles);
  return true;
}

template <int MODE>
__global__ void __launch_bounds__(320, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       PersistParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kPStages * kPABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kPBarOff);
  uint64_t* empty = full + kPStages;
  uint64_t* acc_full = empty + kPStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
    }
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      long kbi = 0;
      bool alive = true;
      for (long it = 0; alive; ++it) {
        int mt, nt;
        if (!tile_at<MODE>(p, it, mt, nt)) break;
        for (int kb = 0; kb < num_kb; ++kb, ++kbi) {
          const int s = static_cast<int>(kbi % kPStages);
          const uint32_t ph = static_cast<uint32_t>((kbi / kPStages) & 1);
          if (!mbar_wait(&empty[s], ph ^ 1, kStatusEmptyWaitTimeout)) { alive = false; break; }
          mbar_expect_tx(&full[s], kPABytes + kPBBytes);
          tma_load_2d(sA + s * kPABytes, &tma_a, &full[s], kb * 64, mt * 128);
          tma_load_2d(sB + s * kPBBytes, &tma_b, &full[s], kb * 64, nt * kPBN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, kPBN);
      long kbi = 0;
      bool alive = true;
      for (long it = 0; alive; ++it) {
        int mt, nt;
        if (!tile_at<MODE>(p, it, mt, nt)) break;
        const int buf = static_cast<int>(it & 1);
        const uint32_t aph = static_cast<uint32_t>((it >> 1) & 1);
        if (!mbar_wait(&acc_empty[buf], aph ^ 1, kStatusGridFlagTimeout)) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kPBN;
        for (int kb = 0; kb < num_kb; ++kb, ++kbi) {
          const int s = static_cast<int>(kbi % kPStages);
          const uint32_t ph = static_cast<uint32_t>((kbi / kPStages) & 1);
          if (!mbar_wait(&full[s], ph, kStatusTmaWaitTimeout)) { alive = false; break; }
          tcgen05_fence_after();
          const uint64_t adesc = umma_desc_k_sw128(smem_u32(sA + s * kPABytes));
          const uint64_t bdesc = umma_desc_k_sw128(smem_u32(sB + s * kPBBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          umma_commit(&empty[s]);
        }
        umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    const int col_lo = ((warp - 2) >> 2) * (kPBN / 2);  // two epilogue warpgroups split the tile's columns
    float run_best = INFINITY;  // kArgmin running state
    int run_idx = 0;
    for (long it = 0;; ++it) {
      int mt, nt;
      if (!tile_at<MODE>(p, it, mt, nt)) break;
      const int buf = static_cast<int>(it & 1);
      const uint32_t aph = static_cast<uint32_t>((it >> 1) & 1);
      if (!mbar_wait(&acc_full[buf], aph, kStatusMmaWaitTimeout)) break;
      tcgen05_fence_after();
      const int row = mt * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + buf * kPBN + (static_cast<uint32_t>(q * 32) << 16);
      float rterm = 0.0f, thr = 0.0f;
      if (MODE != kStore) {
        rterm = (p.row_term && row_ok) ? p.row_term[row] : 0.0f;
        if (MODE == kFilter) thr = row_ok ? p.threshold[row] : -INFINITY;
        if (MODE == kArgmin && nt == 0) { run_best = INFINITY; run_idx = 0; }
      }
#pragma unroll 1
      for (int c = col_lo; c < col_lo + kPBN / 2; c += 32) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        const int nbase = nt * kPBN + c;
        if (c + 32 == col_lo + kPBN / 2) {
          // Everything of this accumulator is in registers (or consumed): hand it back to the MMA warp.
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (nbase >= p.N) continue;
        if (MODE == kStore) {
          if (!row_ok) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          const bool full_chunk = nbase + 32 <= p.N;
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full_chunk || nbase + j < p.N) v[j] += __bfloat162float(p.bias[nbase + j]);
          }
          // The activation is chosen once per chunk, outside the element loop: a per-element switch gets
          // if-converted into evaluating every activation for every element.
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
                const uint4 u = reinterpret_cast<const uint4*>(rp)[j];
                const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z),
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
          if (p.out_f32) {
            float* op = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ldc + nbase;
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
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldc + nbase;
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
        } else if (MODE == kFilter) {
          if (!row_ok) continue;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = nbase + j;
            float d = rterm + p.scale * __uint_as_float(r[j]);
            if (p.col_term) d += (n < p.N) ? p.col_term[n] : 0.0f;
            if (p.clamp_zero) d = fmaxf(d, 0.0f);
            if (n < p.N && d < thr) {
              const int slot = atomicAdd(&p.cand_count[row], 1);
              if (slot < p.cap) {
                p.cand_val[static_cast<size_t>(row) * p.cap + slot] = d;
                p.cand_idx[static_cast<size_t>(row) * p.cap + slot] = static_cast<int>(p.col_offset + n);
              }
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = nbase + j;
            if (n < p.N) {
              const float d = (p.col_term ? p.col_term[n] : 0.0f) + p.scale * __uint_as_float(r[j]);
              if (d < run_best) { run_best = d; run_idx = n; }
            }
          }
        }
      }
      if (MODE == kArgmin && nt == p.n_tiles - 1) {
        // The two warpgroups each hold the arg-min of their half of the columns: combine through shared memory
        // (lower index wins ties, matching a left-to-right scan).
        __shared__ float s_best[128];
        __shared__ int s_idx[128];
        const int r = q * 32 + lane;
        if (col_lo != 0) { s_best[r] = run_best; s_idx[r] = run_idx; }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (col_lo == 0 && row_ok) {
          const float ob = s_best[r];
          const int oi = s_idx[r];
          if (ob < run_best || (ob == run_best && oi < run_idx)) { run_best = ob; run_idx = oi; }
          p.assign[row] = run_idx;
          if (p.best) p.best[row] = run_best + rterm;
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <int MODE>
int launch_persistent(const void* A, const void* B, PersistParams p, int lda, int ldb, int max_ctas,
                      cudaStream_t stream) {
  CUtensorMap ta, tb;
  if (make_tmap_2d(&ta, A, 2, p.M, p.K, static_cast<uint64_t>(lda) * 2, 128, 64, 3)) return -1;
  if (make_tmap_2d(&tb, B, 2, p.N, p.K, static_cast<uint64_t>(ldb) * 2, kPBN, 64, 3)) return -1;
  // The persistent kernel takes all 512 tensor-memory columns, so it must be alone on its SM: its shared
  // memory has to exceed half of what an SM offers.
  static_assert(kPSmem > 227 * 1024 / 2, "a CTA that allocates all of tensor memory must own the SM");
  AFB_CONFIGURE_KERNEL((gemm_persistent_kernel<MODE>), kPSmem, 320, 512);
  const int sm_count = device_sm_count();
  p.m_tiles = (p.M + 127) / 128;
  p.n_tiles = (p.N + kPBN - 1) / kPBN;
  long work = MODE == kArgmin ? p.m_tiles : static_cast<long>(p.m_tiles) * p.n_tiles;
  int ctas = static_cast<int>(work < sm_count ? work : sm_count);
  if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;
  if (ctas < 1) ctas = 1;
  gemm_persistent_kernel<MODE><<<ctas, 320, kPSmem, stream>>>(ta, tb, p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace afb

extern "C" {

static int check_dims(const char* who, int K, int lda, int ldb) {
  if ((K & 7) || (lda & 7) || (ldb & 7)) {
    afb::set_last_error("%s: K, lda and ldb must be multiples of 8 (got %d, %d, %d)", who, K, lda, ldb);
    return -1;
  }
  return 0;
}

int afb_gemm_persistent(const void* A, const void* B, void* out, const void* bias, const void* residual, int M, int N,
                        int K, int lda, int ldb, int ldc, int ldr, int act, int out_f32, float alpha,
                        cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (check_dims("afb_gemm_persistent", K, lda, ldb)) return -1;
  PersistParams p = {};
  p.M = M; p.N = N; p.K = K; p.out = out;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldc = ldc; p.ldr = ldr; p.act = act; p.out_f32 = out_f32; p.alpha = alpha;
  return launch_persistent<kStore>(A, B, p, lda, ldb, 0, stream);
}

// Vector-search scoring with in-epilogue filtering.  Q [M, K] queries, X [N, K] database rows (bf16).
// distance(m, n) = row_term[m] + col_term[n] + scale * <q_m, x_n>, optionally clamped at 0; pairs with
// distance < threshold[m] are appended to the query's candidate list (count keeps growing past cap so the
// caller can detect overflow).
int afb_score_filter(const void* Q, const void* X, int M, int N, int K, int ldq, int ldx, const float* row_term,
                     const float* col_term, float scale, int clamp_zero, const float* threshold, float* cand_val,
                     int* cand_idx, int* cand_count, int cap, long col_offset, cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0) return 0;
  if (check_dims("afb_score_filter", K, ldq, ldx)) return -1;
  PersistParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.row_term = row_term; p.col_term = col_term; p.scale = scale; p.clamp_zero = clamp_zero;
  p.threshold = threshold; p.cand_val = cand_val; p.cand_idx = cand_idx; p.cand_count = cand_count; p.cap = cap;
  p.col_offset = col_offset;
  return launch_persistent<kFilter>(Q, X, p, ldq, ldx, 0, stream);
}

// k-means assignment: assign[m] = argmin_n (col_term[n] + scale * <x_m, c_n>), best[m] = that minimum + row_term[m].
int afb_assign_argmin(const void* X, const void* C, int M, int N, int K, int ldx, int ldc_, const float* row_term,
                      const float* col_term, float scale, int* assign, float* best, cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0) return 0;
  if (check_dims("afb_assign_argmin", K, ldx, ldc_)) return -1;
  PersistParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.row_term = row_term; p.col_term = col_term; p.scale = scale; p.assign = assign; p.best = best;
  return launch_persistent<kArgmin>(X, C, p, ldx, ldc_, 0, stream);
}

}  // extern "C"
