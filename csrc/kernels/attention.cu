// Flash attention for every attention shape the models need, one templated kernel:
//   * packed variable-length bidirectional attention (BERT-family encoders, cross-encoders),
//   * causal prefill over a paged KV cache (chunked prefill, mixed prefill+decode batches, speculative verify),
//   * paged-KV decode attention with the KV range split across the warps of a CTA and across CTAs, merged by
//     log-sum-exp (a second tiny kernel when more than one CTA shares a sequence).
// GQA is handled by packing the (query position, head-in-group) pairs of one KV head into the rows of a tile,
// so K/V are read once per KV head.  Online softmax in the exp2 domain, fp32 accumulation, bf16 I/O.
//
// Mask semantics follow the reference's gqaPagedAttentionDirect
// (zig/pkg/inference/src/ops/native_compute.zig:35093-35173): the query rows of a sequence are its LAST q_len
// positions; a query at absolute position p sees keys at positions <= p (when causal) and > p - window (when
// a sliding window is set); without the causal mask a window is two-sided, |key - p| < window (the local layers of
// ModernBERT-style encoders).  Replaces the reference's thread-per-output encoder attention
// (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:702-857), which has no paged or GQA
// path on CUDA at all.
//
// Tensor-core path: mma.sync m16n8k16 (bf16) with ldmatrix from XOR-swizzled shared memory, K/V tiles staged
// by cp.async (zero-filled past the end of the sequence) in a two- or three-deep ring.
#include <stdlib.h>

#include "../common/mxquant.cuh"
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"
#include "../include/antfly_b200_noalloc.h"

// Scratch of the allocation-free entry point (see antfly_b200_noalloc.h): split-KV partial outputs followed by
// their log-sum-exps.  In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_afb_noalloc_scratch[AFB_NOALLOC_SCRATCH_BYTES];

namespace afb {

struct AttnParams {
  const __nv_bfloat16* q;
  long q_stride;  // elements between consecutive tokens of q
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  long kv_stride;  // contiguous mode: elements between consecutive tokens of k / v
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;  // paged mode: [num_blocks, page, Hkv, D]
  const int* block_tables;
  int max_blocks;
  int page;
  int page_shift;  // log2(page) when page is a power of two, else -1
  const int* q_starts;  // [B] first token row of each sequence in q / out (and k / v in contiguous mode)
  const int* q_lens;    // [B]
  const int* kv_lens;   // [B] total keys visible to the sequence (contiguous mode: = q_lens)
  __nv_bfloat16* out;
  long out_stride;
  float* part_o;    // [splits, T*Hq, D]
  float* part_lse;  // [splits, T*Hq]
  int T;            // total query tokens
  int Hq, Hkv;
  int causal, window;
  float scale_log2;  // softmax scale * log2(e)
  int num_splits;
  float v_scale;     // fp8 caches: factor that turns stored value codes back into values (1 for bf16 caches)
};

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kTileKeys = 64;

template <int D, bool PAGED>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* sK, __nv_bfloat16* sV, const AttnParams& p, int b,
                                             int hk, int k0, int kv_len, int kv_row_start) {
  // Each thread owns one 16-byte column chunk and every (128 / CH)-th row of the tile, so the swizzle term and
  // the column offset are loop invariants and the per-row work is one block-table read plus a few integer ops.
  constexpr int CH = D / 8;
  constexpr int ROWS_PER_PASS = 128 / CH;
  const int ch = threadIdx.x % CH, r0 = threadIdx.x / CH;
  const int dst0 = r0 * D + ((ch ^ (r0 & 7)) * 8);  // valid when ROWS_PER_PASS is a multiple of 8: row & 7 == r0 & 7
  const int* table = PAGED ? p.block_tables + static_cast<size_t>(b) * p.max_blocks : nullptr;
  const size_t row_elems = PAGED ? static_cast<size_t>(p.Hkv) * D : static_cast<size_t>(p.kv_stride);
  const size_t col_off = static_cast<size_t>(hk) * D + ch * 8;
#pragma unroll
  for (int i = 0; i < kTileKeys / ROWS_PER_PASS; ++i) {
    const int row = r0 + i * ROWS_PER_PASS;
    const int key = k0 + row;
    const bool valid = key < kv_len;
    const int kk = valid ? key : 0;
    size_t off;
    if (PAGED) {
      int blk, in_page;
      if (p.page_shift >= 0) {
        blk = table[kk >> p.page_shift];
        in_page = kk & (p.page - 1);
        off = ((static_cast<size_t>(blk) << p.page_shift) + in_page) * row_elems + col_off;
      } else {
        blk = table[kk / p.page];
        in_page = kk % p.page;
        off = (static_cast<size_t>(blk) * p.page + in_page) * row_elems + col_off;
      }
    } else {
      off = static_cast<size_t>(kv_row_start + kk) * row_elems + col_off;
    }
    // With fewer than 8 rows per pass (256-wide heads) the swizzle term changes from pass to pass.
    const int dst = (ROWS_PER_PASS % 8 == 0) ? dst0 + i * ROWS_PER_PASS * D : row * D + ((ch ^ (row & 7)) * 8);
    cp_async_16(sK + dst, (PAGED ? p.k_cache : p.k) + off, valid ? 16 : 0);
    cp_async_16(sV + dst, (PAGED ? p.v_cache : p.v) + off, valid ? 16 : 0);
  }
}

// fp8 (e4m3) paged cache: a 64-key tile arrives as raw bytes, row-major [64][D], through the same cp.async ring at
// half the traffic; each thread then expands the 16-byte chunks IT loaded (so only its own cp.async groups need to
// have landed) into the swizzled bf16 work tile the ldmatrix / mma code reads.
template <int D>
__device__ __forceinline__ void load_kv_tile8(uint8_t* rK, uint8_t* rV, const AttnParams& p, int b, int hk, int k0,
                                              int kv_len) {
  constexpr int CH = D / 16;
  constexpr int ROWS_PER_PASS = 128 / CH;
  const int ch = threadIdx.x % CH, r0 = threadIdx.x / CH;
  const int* table = p.block_tables + static_cast<size_t>(b) * p.max_blocks;
  const size_t row_bytes = static_cast<size_t>(p.Hkv) * D;
  const size_t col_off = static_cast<size_t>(hk) * D + ch * 16;
  const uint8_t* k8 = reinterpret_cast<const uint8_t*>(p.k_cache);
  const uint8_t* v8 = reinterpret_cast<const uint8_t*>(p.v_cache);
#pragma unroll
  for (int i = 0; i < kTileKeys / ROWS_PER_PASS; ++i) {
    const int row = r0 + i * ROWS_PER_PASS;
    const int key = k0 + row;
    const bool valid = key < kv_len;
    const int kk = valid ? key : 0;
    int blk, in_page;
    if (p.page_shift >= 0) { blk = table[kk >> p.page_shift]; in_page = kk & (p.page - 1); }
    else { blk = table[kk / p.page]; in_page = kk % p.page; }
    const size_t off = (static_cast<size_t>(blk) * p.page + in_page) * row_bytes + col_off;
    cp_async_16(rK + row * D + ch * 16, k8 + off, valid ? 16 : 0);
    cp_async_16(rV + row * D + ch * 16, v8 + off, valid ? 16 : 0);
  }
}

template <int D>
__device__ __forceinline__ void expand_kv_tile8(const uint8_t* rK, const uint8_t* rV, __nv_bfloat16* sK,
                                                __nv_bfloat16* sV) {
  constexpr int CH = D / 16;
  constexpr int ROWS_PER_PASS = 128 / CH;
  const int ch = threadIdx.x % CH, r0 = threadIdx.x / CH;
#pragma unroll
  for (int i = 0; i < kTileKeys / ROWS_PER_PASS; ++i) {
    const int row = r0 + i * ROWS_PER_PASS;
    const int c0 = ((2 * ch) ^ (row & 7)) * 8, c1 = ((2 * ch + 1) ^ (row & 7)) * 8;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const uint4 v = *reinterpret_cast<const uint4*>((which ? rV : rK) + row * D + ch * 16);
      uint32_t o[8];
      e4m3x4_to_bf16x4(v.x, kE4m3ToBf16Unit, o[0], o[1]);
      e4m3x4_to_bf16x4(v.y, kE4m3ToBf16Unit, o[2], o[3]);
      e4m3x4_to_bf16x4(v.z, kE4m3ToBf16Unit, o[4], o[5]);
      e4m3x4_to_bf16x4(v.w, kE4m3ToBf16Unit, o[6], o[7]);
      __nv_bfloat16* dst = which ? sV : sK;
      *reinterpret_cast<uint4*>(dst + row * D + c0) = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4*>(dst + row * D + c1) = make_uint4(o[4], o[5], o[6], o[7]);
    }
  }
}

// SPLIT_KEYS = false: each of the 4 warps owns 16 query rows and all 64 keys of a tile (prefill / encoder).
// SPLIT_KEYS = true : all warps share the same <= 16 query rows and each owns 16 keys of a tile (decode).
// STAGES: depth of the K/V tile ring (2, or 3 for small grids where one or two CTAs per SM must cover the DRAM
// latency by themselves).
template <int D, bool PAGED, bool SPLIT_KEYS, int STAGES>
__global__ void __launch_bounds__(128) flash_attn_kernel(AttnParams p) {
  constexpr int NKB = SPLIT_KEYS ? 2 : 8;  // 8-key blocks per warp per tile
  constexpr int ND = D / 8;                // 8-wide output blocks
  constexpr int KSTEPS = D / 16;
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* sKV = reinterpret_cast<__nv_bfloat16*>(smem_attn);  // [2 stages][K tile, V tile]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  griddep_launch();
  griddep_wait();
  const int b = blockIdx.z / p.num_splits;
  const int split = blockIdx.z % p.num_splits;
  const int hk = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  const int q_start = p.q_starts[b], q_len = p.q_lens[b], kv_len = p.kv_lens[b];
  const int rows_total = q_len * G;
  const int tile_row0 = blockIdx.x * (SPLIT_KEYS ? 16 : 64);
  if (tile_row0 >= rows_total) return;
  const int pos_off = kv_len - q_len;  // absolute position of the first query row

  // Rows this thread's fragments cover.
  const int wrow0 = tile_row0 + (SPLIT_KEYS ? 0 : warp * 16);
  int r_idx[2], r_pos[2], r_head[2];
  bool r_ok[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = wrow0 + (lane >> 2) + 8 * h;
    r_idx[h] = r;
    r_ok[h] = r < rows_total;
    r_pos[h] = r / G;
    r_head[h] = hk * G + r % G;
  }

  // Q fragments straight from global memory (read once).
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t lo = 0, hi = 0;
      if (r_ok[h]) {
        const __nv_bfloat16* qp = p.q + static_cast<size_t>(q_start + r_pos[h]) * p.q_stride + r_head[h] * D +
                                  kk * 16 + 2 * (lane & 3);
        lo = *reinterpret_cast<const uint32_t*>(qp);
        hi = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
      qf[kk][h] = lo;
      qf[kk][2 + h] = hi;
    }
  }

  // KV tile range of this CTA.
  int kv_hi = kv_len;
  if (p.causal) {
    const int last_row = min(rows_total, tile_row0 + (SPLIT_KEYS ? 16 : 64)) - 1;
    kv_hi = min(kv_len, pos_off + last_row / G + 1);
  } else if (p.window > 0) {  // bidirectional local attention: |key - qpos| < window
    const int last_row = min(rows_total, tile_row0 + (SPLIT_KEYS ? 16 : 64)) - 1;
    kv_hi = min(kv_len, pos_off + last_row / G + p.window);
  }
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, pos_off + tile_row0 / G - p.window + 1);
  const int tile_lo = kv_lo / kTileKeys;
  const int tile_hi = (kv_hi + kTileKeys - 1) / kTileKeys;
  const int ntiles_all = max(0, tile_hi - tile_lo);
  const int per_split = (ntiles_all + p.num_splits - 1) / p.num_splits;
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_hi, t_begin + per_split);
  const int ntiles = max(0, t_end - t_begin);

  float o[ND][4];
#pragma unroll
  for (int i = 0; i < ND; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};

  constexpr int TILE_ELEMS = kTileKeys * D;
  // One commit group per tile slot (empty past the end) keeps the group count uniform for wait_group.
#pragma unroll
  for (int s0 = 0; s0 < STAGES - 1; ++s0) {
    if (s0 < ntiles) {
      __nv_bfloat16* nK = sKV + s0 * 2 * TILE_ELEMS;
      load_kv_tile<D, PAGED>(nK, nK + TILE_ELEMS, p, b, hk, (t_begin + s0) * kTileKeys, kv_len, q_start);
    }
    cp_async_commit();
  }
  for (int it = 0; it < ntiles; ++it) {
    const int stage = it % STAGES;
    __nv_bfloat16* sK = sKV + stage * 2 * TILE_ELEMS;
    __nv_bfloat16* sV = sK + TILE_ELEMS;
    if (it + STAGES - 1 < ntiles) {
      __nv_bfloat16* nK = sKV + ((it + STAGES - 1) % STAGES) * 2 * TILE_ELEMS;
      load_kv_tile<D, PAGED>(nK, nK + TILE_ELEMS, p, b, hk, (t_begin + it + STAGES - 1) * kTileKeys, kv_len,
                             q_start);
    }
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();

    const int k0 = (t_begin + it) * kTileKeys;
    const int wkey0 = SPLIT_KEYS ? warp * 16 : 0;  // first key of the tile this warp handles

    // ---- S = Q K^T ----
    float s[NKB][4];
#pragma unroll
    for (int nb = 0; nb < NKB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int nb = 0; nb < NKB; nb += 2) {
        const int mi = lane >> 3, rin = lane & 7;
        const int key = wkey0 + nb * 8 + (mi >> 1) * 8 + rin;
        const int chunk = kk * 2 + (mi & 1);
        uint32_t kb[4];
        ldmatrix_x4(kb, sK + key * D + ((chunk ^ (key & 7)) * 8));
        mma_bf16_16816(s[nb], qf[kk], kb[0], kb[1]);
        mma_bf16_16816(s[nb + 1], qf[kk], kb[2], kb[3]);
      }
    }

    // ---- mask + online softmax ----
    // Tiles that lie wholly inside every row's visible range (the common case in decode) skip the mask; rows past
    // rows_total then hold finite garbage that is never stored.
    const int row_lo = tile_row0 + (SPLIT_KEYS ? 0 : warp * 16);
    const int min_qpos = pos_off + row_lo / G;
    const int max_qpos = pos_off + (min(rows_total, row_lo + 16) - 1) / G;
    const bool full_tile = (k0 + kTileKeys <= kv_len) && (!p.causal || k0 + kTileKeys - 1 <= min_qpos) &&
                           (p.window <= 0 || (k0 > max_qpos - p.window &&
                                              (p.causal || k0 + kTileKeys - 1 < min_qpos + p.window)));
    float mx[2] = {-INFINITY, -INFINITY};
    if (!full_tile) {
#pragma unroll
      for (int nb = 0; nb < NKB; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int key = k0 + wkey0 + nb * 8 + 2 * (lane & 3) + (e & 1);
          const int qpos = pos_off + r_pos[h];
          bool ok = r_ok[h] && key < kv_len;
          if (p.causal) ok = ok && key <= qpos;
          if (p.window > 0) ok = ok && key > qpos - p.window && (p.causal || key < qpos + p.window);
          if (!ok) s[nb][e] = -INFINITY;
        }
      }
    }
#pragma unroll
    for (int nb = 0; nb < NKB; ++nb) {
      mx[0] = fmaxf(mx[0], fmaxf(s[nb][0], s[nb][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[nb][2], s[nb][3]));
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      mx[h] *= p.scale_log2;  // the softmax scale is positive: max and scaling commute; -inf stays -inf
      const float m_new = fmaxf(m_run[h], mx[h]);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      alpha[h] = exp2f(m_run[h] - m_use);  // m_run = -inf -> 0
      m_run[h] = m_new;
      l_run[h] *= alpha[h];
      mx[h] = -m_use;
    }
    uint32_t pf[NKB / 2][4];
#pragma unroll
    for (int nb = 0; nb < NKB; ++nb) {
      const float p0 = exp2f(fmaf(s[nb][0], p.scale_log2, mx[0]));
      const float p1 = exp2f(fmaf(s[nb][1], p.scale_log2, mx[0]));
      const float p2 = exp2f(fmaf(s[nb][2], p.scale_log2, mx[1]));
      const float p3 = exp2f(fmaf(s[nb][3], p.scale_log2, mx[1]));
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2 + 0] = pack_bf16x2(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16x2(p2, p3);
    }
    // The running maximum settles after the first tiles; skip the accumulator rescale when no row of the warp moved.
    if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
        o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
    }

    // ---- O += P V ----
#pragma unroll
    for (int ks = 0; ks < NKB / 2; ++ks) {
#pragma unroll
      for (int db = 0; db < ND / 2; ++db) {
        const int mi = lane >> 3, rin = lane & 7;
        const int key = wkey0 + ks * 16 + (mi & 1) * 8 + rin;
        const int chunk = db * 2 + (mi >> 1);
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, sV + key * D + ((chunk ^ (key & 7)) * 8));
        mma_bf16_16816(o[2 * db], pf[ks], vb[0], vb[1]);
        mma_bf16_16816(o[2 * db + 1], pf[ks], vb[2], vb[3]);
      }
    }
    __syncthreads();
  }

  // Row sums across the four threads that share a row.
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  if constexpr (SPLIT_KEYS) {
    // Merge the four warps (same rows, disjoint keys) through shared memory.
    float* sO = reinterpret_cast<float*>(smem_attn);  // [4][16][D]
    float* sM = sO + 4 * 16 * D;                      // [4][16]
    float* sL = sM + 64;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < ND; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = (lane >> 2) + 8 * (e >> 1);
        const int col = i * 8 + 2 * (lane & 3) + (e & 1);
        sO[(warp * 16 + row) * D + col] = o[i][e];
      }
    }
    if ((lane & 3) == 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sM[warp * 16 + (lane >> 2) + 8 * h] = m_run[h];
        sL[warp * 16 + (lane >> 2) + 8 * h] = l_run[h];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * D; idx += blockDim.x) {
      const int row = idx / D, col = idx % D;
      const int r = tile_row0 + row;
      if (r >= rows_total) continue;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w * 16 + row]);
      float L = 0.0f, acc = 0.0f;
      if (M != -INFINITY) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float f = exp2f(sM[w * 16 + row] - M);
          L += f * sL[w * 16 + row];
          acc += f * sO[(w * 16 + row) * D + col];
        }
      }
      const float val = L > 0.0f ? acc / L : 0.0f;
      const int tok = q_start + r / G;
      const int head = hk * G + r % G;
      if (p.num_splits == 1) {
        p.out[static_cast<size_t>(tok) * p.out_stride + head * D + col] = __float2bfloat16(val);
      } else {
        const size_t prow = static_cast<size_t>(split) * p.T * p.Hq + static_cast<size_t>(tok) * p.Hq + head;
        p.part_o[prow * D + col] = val;
        if (col == 0) p.part_lse[prow] = (L > 0.0f) ? M + log2f(L) : -INFINITY;
      }
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (!r_ok[h]) continue;
      const float inv = l_run[h] > 0.0f ? 1.0f / l_run[h] : 0.0f;
      __nv_bfloat16* op = p.out + static_cast<size_t>(q_start + r_pos[h]) * p.out_stride + r_head[h] * D +
                          2 * (lane & 3);
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        *reinterpret_cast<uint32_t*>(op + i * 8) = pack_bf16x2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Decode attention for at most 8 (position, head-in-group) rows per KV head, i.e. one new token with a GQA
// group of up to 8: the transposed formulation.  Keys sit on the MMA's M axis and the query rows on its N = 8
// axis, S^T = K Q^T and O^T = V^T P^T, so a warp spends one m16n8k16 per 16 keys x 16 dims instead of two with
// three quarters of the rows padding, and the output accumulator is D x 8 (32 registers at D = 128) instead of
// 16 x D (64).  Each of the four warps owns 16 keys of a 64-key tile; P^T goes from accumulator layout to the
// B-operand layout with two movmatrix transposes; warps and KV splits are merged by log-sum-exp as before.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
  return r;
}

// KV8: the cache holds e4m3 bytes (see load_kv_tile8): the ring carries raw tiles and one bf16 work tile pair sits
// behind it.
template <int D, int STAGES, bool KV8>
__global__ void __launch_bounds__(128) decode_attn_t_kernel(AttnParams p) {
  constexpr int KSTEPS = D / 16;  // 16-wide steps over the head dimension
  constexpr int NDB = D / 16;     // 16-row blocks of O^T
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* sKV = reinterpret_cast<__nv_bfloat16*>(smem_attn);
  constexpr int RAW_TILE = kTileKeys * D;  // bytes of one raw fp8 tile (K or V)
  __nv_bfloat16* sWork = reinterpret_cast<__nv_bfloat16*>(smem_attn + STAGES * 2 * RAW_TILE);  // KV8 only
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  griddep_launch();
  griddep_wait();
  const int b = blockIdx.z / p.num_splits;
  const int split = blockIdx.z % p.num_splits;
  const int hk = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  const int q_start = p.q_starts[b], q_len = p.q_lens[b], kv_len = p.kv_lens[b];
  const int rows_total = q_len * G;  // <= 8
  if (rows_total <= 0) return;
  const int pos_off = kv_len - q_len;

  // Q^T as the B operand: lane (g, t) holds Q[row g][16 kk + 2t, +1] and [.. + 8, + 9]; rows >= rows_total are 0.
  uint32_t qf[KSTEPS][2];
  {
    const bool ok = g < rows_total;
    const __nv_bfloat16* qp = p.q + static_cast<size_t>(q_start + (ok ? g / G : 0)) * p.q_stride +
                              (hk * G + (ok ? g % G : 0)) * D + 2 * t;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      qf[kk][0] = ok ? *reinterpret_cast<const uint32_t*>(qp + kk * 16) : 0u;
      qf[kk][1] = ok ? *reinterpret_cast<const uint32_t*>(qp + kk * 16 + 8) : 0u;
    }
  }
  // This thread's two query columns (2t, 2t + 1) and their absolute positions.
  int qpos[2];
  bool qok[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = 2 * t + e;
    qok[e] = r < rows_total;
    qpos[e] = pos_off + r / G;
  }

  int kv_hi = kv_len;
  if (p.causal) kv_hi = min(kv_len, pos_off + (rows_total - 1) / G + 1);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, pos_off - p.window + 1);
  const int tile_lo = kv_lo / kTileKeys;
  const int tile_hi = (kv_hi + kTileKeys - 1) / kTileKeys;
  const int ntiles_all = max(0, tile_hi - tile_lo);
  const int per_split = (ntiles_all + p.num_splits - 1) / p.num_splits;
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_hi, t_begin + per_split);
  const int ntiles = max(0, t_end - t_begin);

  float o[NDB][4];
#pragma unroll
  for (int i = 0; i < NDB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};

  constexpr int TILE_ELEMS = kTileKeys * D;
#pragma unroll
  for (int s0 = 0; s0 < STAGES - 1; ++s0) {
    if (s0 < ntiles) {
      if constexpr (KV8) {
        uint8_t* rK = smem_attn + s0 * 2 * RAW_TILE;
        load_kv_tile8<D>(rK, rK + RAW_TILE, p, b, hk, (t_begin + s0) * kTileKeys, kv_len);
      } else {
        __nv_bfloat16* nK = sKV + s0 * 2 * TILE_ELEMS;
        load_kv_tile<D, true>(nK, nK + TILE_ELEMS, p, b, hk, (t_begin + s0) * kTileKeys, kv_len, q_start);
      }
    }
    cp_async_commit();
  }
  const int mi = lane >> 3, rin = lane & 7;
  for (int it = 0; it < ntiles; ++it) {
    const int stage = it % STAGES;
    const __nv_bfloat16* sK = KV8 ? sWork : sKV + stage * 2 * TILE_ELEMS;
    const __nv_bfloat16* sV = sK + TILE_ELEMS;
    if (it + STAGES - 1 < ntiles) {
      if constexpr (KV8) {
        uint8_t* rK = smem_attn + ((it + STAGES - 1) % STAGES) * 2 * RAW_TILE;
        load_kv_tile8<D>(rK, rK + RAW_TILE, p, b, hk, (t_begin + it + STAGES - 1) * kTileKeys, kv_len);
      } else {
        __nv_bfloat16* nK = sKV + ((it + STAGES - 1) % STAGES) * 2 * TILE_ELEMS;
        load_kv_tile<D, true>(nK, nK + TILE_ELEMS, p, b, hk, (t_begin + it + STAGES - 1) * kTileKeys, kv_len, q_start);
      }
    }
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    if constexpr (KV8) {
      // Each thread expands the chunks it loaded itself (its own groups have landed); the work tile is free:
      // the barrier that ends the previous iteration followed every warp's last read of it.
      const uint8_t* rK = smem_attn + stage * 2 * RAW_TILE;
      expand_kv_tile8<D>(rK, rK + RAW_TILE, sWork, sWork + TILE_ELEMS);
    }
    __syncthreads();

    const int k0 = (t_begin + it) * kTileKeys + warp * 16;  // first key of this warp's slab
    // ---- S^T = K Q^T : two independent accumulators (even / odd k-steps) shorten the dependency chain ----
    float s0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    {
      const int key = warp * 16 + (mi & 1) * 8 + rin;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int chunk = kk * 2 + (mi >> 1);
        uint32_t ka[4];
        ldmatrix_x4(ka, sK + key * D + ((chunk ^ (key & 7)) * 8));
        if (kk & 1) mma_bf16_16816(s1, ka, qf[kk][0], qf[kk][1]);
        else mma_bf16_16816(s0, ka, qf[kk][0], qf[kk][1]);
      }
    }
    float s[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] = s0[e] + s1[e];
    // s[0], s[1]: key k0 + g, queries 2t, 2t + 1;  s[2], s[3]: key k0 + g + 8, same queries.
    const bool full = (k0 + 16 <= kv_len) && (!p.causal || k0 + 15 <= pos_off) && (p.window <= 0 || k0 > pos_off + (rows_total - 1) / G - p.window);
    if (!full) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + g + 8 * (e >> 1);
        const int c = e & 1;
        bool ok = qok[c] && key < kv_len;
        if (p.causal) ok = ok && key <= qpos[c];
        if (p.window > 0) ok = ok && key > qpos[c] - p.window;
        if (!ok) s[e] = -INFINITY;
      }
    }
    float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
    float alpha[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 4));
      mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 8));
      mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 16));
      mx[c] *= p.scale_log2;
      const float m_new = fmaxf(m_run[c], mx[c]);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      alpha[c] = exp2f(m_run[c] - m_use);
      m_run[c] = m_new;
      l_run[c] *= alpha[c];
      mx[c] = -m_use;
    }
    const float p0 = exp2f(fmaf(s[0], p.scale_log2, mx[0]));
    const float p1 = exp2f(fmaf(s[1], p.scale_log2, mx[1]));
    const float p2 = exp2f(fmaf(s[2], p.scale_log2, mx[0]));
    const float p3 = exp2f(fmaf(s[3], p.scale_log2, mx[1]));
    l_run[0] += p0 + p2;
    l_run[1] += p1 + p3;
    // Accumulator layout (key row, query column pair) -> B-operand layout (key pair, query column).
    const uint32_t pb0 = movmatrix_trans(pack_bf16x2(p0, p1));
    const uint32_t pb1 = movmatrix_trans(pack_bf16x2(p2, p3));
    if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < NDB; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[1];
        o[i][2] *= alpha[0]; o[i][3] *= alpha[1];
      }
    }
    // ---- O^T += V^T P^T ----
    {
      const int key = warp * 16 + (mi >> 1) * 8 + rin;
#pragma unroll
      for (int db = 0; db < NDB; ++db) {
        const int chunk = db * 2 + (mi & 1);
        uint32_t va[4];
        ldmatrix_x4_trans(va, sV + key * D + ((chunk ^ (key & 7)) * 8));
        mma_bf16_16816(o[db], va, pb0, pb1);
      }
    }
    __syncthreads();
  }

  // Per-query sums across the eight lane groups that hold different keys.
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    l_run[c] += __shfl_xor_sync(0xffffffffu, l_run[c], 4);
    l_run[c] += __shfl_xor_sync(0xffffffffu, l_run[c], 8);
    l_run[c] += __shfl_xor_sync(0xffffffffu, l_run[c], 16);
  }
  // Merge the four warps (same queries, disjoint keys) through shared memory: sO[warp][query][d].
  float* sO = reinterpret_cast<float*>(smem_attn);
  float* sM = sO + 4 * 8 * D;
  float* sL = sM + 32;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NDB; ++i) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = i * 16 + g + 8 * (e >> 1);
      const int q = 2 * t + (e & 1);
      sO[(warp * 8 + q) * D + d] = o[i][e];
    }
  }
  if (g == 0) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      sM[warp * 8 + 2 * t + c] = m_run[c];
      sL[warp * 8 + 2 * t + c] = l_run[c];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_total * D; idx += blockDim.x) {
    const int r = idx / D, col = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w * 8 + r]);
    float L = 0.0f, acc = 0.0f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(sM[w * 8 + r] - M);
        L += f * sL[w * 8 + r];
        acc += f * sO[(w * 8 + r) * D + col];
      }
    }
    const float val = (L > 0.0f ? acc / L : 0.0f) * (KV8 ? p.v_scale : 1.0f);
    const int tok = q_start + r / G;
    const int head = hk * G + r % G;
    if (p.num_splits == 1) {
      p.out[static_cast<size_t>(tok) * p.out_stride + head * D + col] = __float2bfloat16(val);
    } else {
      const size_t prow = static_cast<size_t>(split) * p.T * p.Hq + static_cast<size_t>(tok) * p.Hq + head;
      p.part_o[prow * D + col] = val;
      if (col == 0) p.part_lse[prow] = (L > 0.0f) ? M + log2f(L) : -INFINITY;
    }
  }
}

// Merge split-KV partials: out = sum_s 2^(lse_s - max) o_s / sum_s 2^(lse_s - max).  Each thread owns 4 adjacent
// columns of one (token, head) row; 128-thread CTAs cover 512 / D rows.  When q0 is given the merged row is also
// written as MX fp8 activations of the [T, Hq * D] matrix the output projection consumes, so no separate
// quantisation pass runs between attention and that GEMM; `out` may then be null.
__global__ void __launch_bounds__(128) attn_merge_kernel(const float* part_o, const float* part_lse,
                                                         __nv_bfloat16* out, long out_stride, int rows /* T*Hq */,
                                                         int Hq, int D, int splits, uint8_t* q0, uint8_t* q1,
                                                         uint8_t* sf0, uint8_t* sf1) {
  griddep_launch();
  griddep_wait();
  const int tpr = D >> 2;  // threads per row
  const int row_raw = blockIdx.x * (128 / tpr) + threadIdx.x / tpr;
  const bool live = row_raw < rows;
  const int row = live ? row_raw : rows - 1;
  const int c = (threadIdx.x % tpr) * 4;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_lse[static_cast<size_t>(s) * rows + row]);
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, den = 0.0f;
  if (M != -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      const float f = exp2f(part_lse[static_cast<size_t>(s) * rows + row] - M);
      const float4 o = *reinterpret_cast<const float4*>(part_o + (static_cast<size_t>(s) * rows + row) * D + c);
      den += f;
      acc[0] += f * o.x; acc[1] += f * o.y; acc[2] += f * o.z; acc[3] += f * o.w;
    }
  }
  const float inv = den > 0.0f ? 1.0f / den : 0.0f;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = acc[j] * inv;
  const int tok = row / Hq, head = row % Hq;
  if (out && live) {
    uint2 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(tok) * out_stride + head * D + c) = o;
  }
  if (q0) {
    // Quantise what the bf16 path would have produced, so both routes feed the GEMM the same values.
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(__float2bfloat16(v[j]));
    mx_quantize4_store(v, tok, head * D + c, Hq * D, q0, q1, sf0, sf1, live);
  }
}

template <int D, bool PAGED, bool SPLIT_KEYS, int STAGES>
int launch_attn_s(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  const int smem_tiles = STAGES * 2 * kTileKeys * D * 2;
  const int smem_merge = SPLIT_KEYS ? (4 * 16 * D + 128) * 4 : 0;
  const int smem = smem_tiles > smem_merge ? smem_tiles : smem_merge;
  // 128 KiB covers every instantiation's request (the opt-in is a ceiling, not a reservation).
  AFB_CONFIGURE_KERNEL((flash_attn_kernel<D, PAGED, SPLIT_KEYS, STAGES>), smem, 128, 0);
  AFB_CHECK_CUDA(launch_pdl(flash_attn_kernel<D, PAGED, SPLIT_KEYS, STAGES>, grid, dim3(128), smem, stream, p));
  return 0;
}

inline bool transposed_decode_disabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ANTFLY_B200_ATTN_LEGACY_DECODE");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

template <int D, int STAGES, bool KV8 = false>
int launch_decode_t_s(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  // bf16 cache: a ring of bf16 tile pairs.  fp8 cache: a ring of raw byte tile pairs plus one bf16 work pair.
  const int smem_tiles = KV8 ? (STAGES * 2 * kTileKeys * D + 2 * kTileKeys * D * 2) : STAGES * 2 * kTileKeys * D * 2;
  const int smem_merge = (4 * 8 * D + 64) * 4;
  const int smem = smem_tiles > smem_merge ? smem_tiles : smem_merge;
  AFB_CONFIGURE_KERNEL((decode_attn_t_kernel<D, STAGES, KV8>), smem, 128, 0);
  AFB_CHECK_CUDA(launch_pdl(decode_attn_t_kernel<D, STAGES, KV8>, grid, dim3(128), smem, stream, p));
  return 0;
}

// fp8 cache, decode organisation with at most 8 rows per KV head (the only fp8-reading tensor-core path).
template <int D>
int launch_decode_t8(const AttnParams& p, int B, cudaStream_t stream) {
  dim3 grid(1, p.Hkv, B * p.num_splits);
  const long ctas = static_cast<long>(grid.y) * grid.z;
  if (ctas <= 2L * device_sm_count()) return launch_decode_t_s<D, 3, true>(p, grid, stream);
  return launch_decode_t_s<D, 2, true>(p, grid, stream);
}

template <int D>
int launch_decode_t(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  const int sms = device_sm_count();
  const long ctas = static_cast<long>(grid.x) * grid.y * grid.z;
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("ANTFLY_B200_ATTN_STAGES");
    forced = e ? atoi(e) : 0;
  }
  if (forced == 3 || (forced == 0 && ctas <= 2L * sms)) return launch_decode_t_s<D, 3>(p, grid, stream);
  return launch_decode_t_s<D, 2>(p, grid, stream);
}

template <int D, bool PAGED, bool SPLIT_KEYS>
int launch_attn(const AttnParams& p, int B, int max_rows, cudaStream_t stream) {
  const int rows_per_cta = SPLIT_KEYS ? 16 : 64;
  dim3 grid((max_rows + rows_per_cta - 1) / rows_per_cta, p.Hkv, B * p.num_splits);
  if constexpr (SPLIT_KEYS && PAGED) {
    if (max_rows <= 8 && !transposed_decode_disabled()) return launch_decode_t<D>(p, grid, stream);
    // A decode grid that leaves at most two CTAs per SM gets a deeper ring.
    const int sms = device_sm_count();
    const long ctas = static_cast<long>(grid.x) * grid.y * grid.z;
    if (ctas <= 2L * sms) return launch_attn_s<D, PAGED, SPLIT_KEYS, 3>(p, grid, stream);
  }
  return launch_attn_s<D, PAGED, SPLIT_KEYS, 2>(p, grid, stream);
}

}  // namespace afb

extern "C" {

// mode 0: contiguous K/V (k, v given; kv rows of sequence b start at q_starts[b], kv_lens == q_lens)
// mode 1: paged K/V (k_cache, v_cache, block_tables)
// split_keys != 0 selects the decode organisation (<= 16 rows per (sequence, KV head) per CTA);
// num_splits > 1 additionally splits the KV range across CTAs and needs part_o / part_lse scratch.
// max_q_len: the largest q_lens[b] (host knowledge, sizes the grid).
int afb_attention_mx(const void* q, long q_stride, const void* k, const void* v, long kv_stride,
                     const void* k_cache, const void* v_cache, const int* block_tables, int max_blocks, int page,
                     const int* q_starts, const int* q_lens, const int* kv_lens, void* out, long out_stride,
                     float* part_o, float* part_lse, int B, int T, int Hq, int Hkv, int D, int max_q_len, int causal,
                     int window, float scale, int paged, int split_keys, int num_splits, void* mx_q0, void* mx_q1,
                     void* mx_sf0, void* mx_sf1, cudaStream_t stream);

int afb_attention(const void* q, long q_stride, const void* k, const void* v, long kv_stride, const void* k_cache,
                  const void* v_cache, const int* block_tables, int max_blocks, int page, const int* q_starts,
                  const int* q_lens, const int* kv_lens, void* out, long out_stride, float* part_o, float* part_lse,
                  int B, int T, int Hq, int Hkv, int D, int max_q_len, int causal, int window, float scale,
                  int paged, int split_keys, int num_splits, cudaStream_t stream) {
  return afb_attention_mx(q, q_stride, k, v, kv_stride, k_cache, v_cache, block_tables, max_blocks, page, q_starts,
                          q_lens, kv_lens, out, out_stride, part_o, part_lse, B, T, Hq, Hkv, D, max_q_len, causal,
                          window, scale, paged, split_keys, num_splits, nullptr, nullptr, nullptr, nullptr, stream);
}

// As afb_attention; with num_splits > 1 and mx_q0 given, the merge kernel also emits the context rows as MX fp8
// activations [T, Hq * D] (mx_q1 / mx_sf1 null: one term) and `out` may be null.
int afb_attention_mx(const void* q, long q_stride, const void* k, const void* v, long kv_stride,
                     const void* k_cache, const void* v_cache, const int* block_tables, int max_blocks, int page,
                     const int* q_starts, const int* q_lens, const int* kv_lens, void* out, long out_stride,
                     float* part_o, float* part_lse, int B, int T, int Hq, int Hkv, int D, int max_q_len, int causal,
                     int window, float scale, int paged, int split_keys, int num_splits, void* mx_q0, void* mx_q1,
                     void* mx_sf0, void* mx_sf1, cudaStream_t stream) {
  using namespace afb;
  if (B <= 0 || T <= 0) return 0;
  if (Hq % Hkv != 0 || (D != 64 && D != 128 && D != 256)) {
    set_last_error("afb_attention: head_dim must be 64, 128 or 256 and Hq a multiple of Hkv (D=%d Hq=%d Hkv=%d)", D,
                   Hq, Hkv);
    return -1;
  }
  if ((q_stride & 7) || (kv_stride & 7) || (out_stride & 3)) {
    set_last_error("afb_attention: q/kv strides must be multiples of 8 elements");
    return -1;
  }
  if (!(scale > 0.0f)) {
    set_last_error("afb_attention: the softmax scale must be positive");
    return -1;
  }
  if (num_splits < 1) num_splits = 1;
  if (!split_keys) num_splits = 1;
  if (num_splits > 1 && (!part_o || !part_lse)) {
    set_last_error("afb_attention: num_splits > 1 needs partial buffers");
    return -1;
  }
  if (mx_q0 && (num_splits < 2 || (Hq * D) % 128 != 0 || !mx_sf0)) {
    set_last_error("afb_attention: MX output needs num_splits > 1 and Hq * D a multiple of 128");
    return -1;
  }
  if (!out && !mx_q0) {
    set_last_error("afb_attention: no output buffer");
    return -1;
  }
  AttnParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q); p.q_stride = q_stride;
  p.k = reinterpret_cast<const __nv_bfloat16*>(k); p.v = reinterpret_cast<const __nv_bfloat16*>(v);
  p.kv_stride = kv_stride;
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.page = page;
  p.page_shift = -1;
  if (page > 0 && (page & (page - 1)) == 0) {
    p.page_shift = 0;
    while ((1 << p.page_shift) < page) ++p.page_shift;
  }
  p.q_starts = q_starts; p.q_lens = q_lens; p.kv_lens = kv_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.out_stride = out_stride;
  p.part_o = part_o; p.part_lse = part_lse;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_splits = num_splits;
  p.v_scale = 1.0f;
  const int G = Hq / Hkv;
  const int max_rows = max_q_len * G;
  int rc;
#define AFB_ATTN_DISPATCH(DD)                                                                      \
  if (paged) {                                                                                     \
    rc = split_keys ? launch_attn<DD, true, true>(p, B, max_rows, stream)                          \
                    : launch_attn<DD, true, false>(p, B, max_rows, stream);                        \
  } else {                                                                                         \
    rc = split_keys ? launch_attn<DD, false, true>(p, B, max_rows, stream)                         \
                    : launch_attn<DD, false, false>(p, B, max_rows, stream);                       \
  }
  if (D == 64) { AFB_ATTN_DISPATCH(64) } else if (D == 128) { AFB_ATTN_DISPATCH(128) } else { AFB_ATTN_DISPATCH(256) }
#undef AFB_ATTN_DISPATCH
  if (rc) return rc;
  if (num_splits > 1) {
    const int rows_per_cta = 128 / (D / 4);
    AFB_CHECK_CUDA(launch_pdl(attn_merge_kernel, dim3((T * Hq + rows_per_cta - 1) / rows_per_cta), dim3(128), 0, stream,
                              static_cast<const float*>(part_o), static_cast<const float*>(part_lse), p.out, out_stride,
                              T * Hq, Hq, D, num_splits, reinterpret_cast<uint8_t*>(mx_q0),
                              reinterpret_cast<uint8_t*>(mx_q1), reinterpret_cast<uint8_t*>(mx_sf0),
                              reinterpret_cast<uint8_t*>(mx_sf1)));
  }
  return 0;
}

// Paged decode attention over an fp8 (e4m3) cache, k_cache / v_cache [num_blocks, page, Hkv, D] bytes: the
// tensor-core decode kernel with the codes expanded to bf16 in shared memory, so the cache crosses HBM at one byte
// per element.  Decode shapes only (q_len * Hq / Hkv <= 8 rows per KV head); k_scale / v_scale turn stored codes
// back into values (1 when keys and values were stored unscaled).  Same split-KV scratch contract as afb_attention.
int afb_attention_kv8(const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_tables,
                      int max_blocks, int page, const int* q_starts, const int* q_lens, const int* kv_lens, void* out,
                      long out_stride, float* part_o, float* part_lse, int B, int T, int Hq, int Hkv, int D,
                      int max_q_len, int window, float scale, float k_scale, float v_scale, int num_splits,
                      void* mx_q0, void* mx_q1, void* mx_sf0, void* mx_sf1, cudaStream_t stream) {
  using namespace afb;
  if (B <= 0 || T <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0 || (D != 64 && D != 128 && D != 256) || max_q_len * (Hq / Hkv) > 8) {
    set_last_error("afb_attention_kv8: needs head_dim 64 / 128 / 256 and q_len * (Hq / Hkv) <= 8 (D=%d Hq=%d Hkv=%d "
                   "q_len=%d)", D, Hq, Hkv, max_q_len);
    return -1;
  }
  if ((q_stride & 7) || (out_stride & 3) || ((static_cast<long>(Hkv) * D) & 15) ||
      (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15)) {
    set_last_error("afb_attention_kv8: q stride must be a multiple of 8 elements and cache rows 16-byte aligned");
    return -1;
  }
  if (!(scale > 0.0f) || !(k_scale > 0.0f) || !(v_scale > 0.0f)) {
    set_last_error("afb_attention_kv8: scales must be positive");
    return -1;
  }
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!part_o || !part_lse)) {
    set_last_error("afb_attention_kv8: num_splits > 1 needs partial buffers");
    return -1;
  }
  if (mx_q0 && (num_splits < 2 || (Hq * D) % 128 != 0 || !mx_sf0)) {
    set_last_error("afb_attention_kv8: MX output needs num_splits > 1 and Hq * D a multiple of 128");
    return -1;
  }
  if (!out && !mx_q0) {
    set_last_error("afb_attention_kv8: no output buffer");
    return -1;
  }
  AttnParams p = {};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q); p.q_stride = q_stride;
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(k_cache);  // read as bytes by the fp8 tile loader
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.page = page;
  p.page_shift = -1;
  if (page > 0 && (page & (page - 1)) == 0) {
    p.page_shift = 0;
    while ((1 << p.page_shift) < page) ++p.page_shift;
  }
  p.q_starts = q_starts; p.q_lens = q_lens; p.kv_lens = kv_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.out_stride = out_stride;
  p.part_o = part_o; p.part_lse = part_lse;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = 1; p.window = window;
  p.scale_log2 = scale * k_scale * 1.4426950408889634f;
  p.num_splits = num_splits;
  p.v_scale = v_scale;
  int rc = D == 64 ? launch_decode_t8<64>(p, B, stream)
                   : D == 128 ? launch_decode_t8<128>(p, B, stream) : launch_decode_t8<256>(p, B, stream);
  if (rc) return rc;
  if (num_splits > 1) {
    const int rows_per_cta = 128 / (D / 4);
    AFB_CHECK_CUDA(launch_pdl(attn_merge_kernel, dim3((T * Hq + rows_per_cta - 1) / rows_per_cta), dim3(128), 0, stream,
                              static_cast<const float*>(part_o), static_cast<const float*>(part_lse), p.out, out_stride,
                              T * Hq, Hq, D, num_splits, reinterpret_cast<uint8_t*>(mx_q0),
                              reinterpret_cast<uint8_t*>(mx_q1), reinterpret_cast<uint8_t*>(mx_sf0),
                              reinterpret_cast<uint8_t*>(mx_sf1)));
  }
  return 0;
}

}  // extern "C"

extern "C" {

// Allocation-free variant of the split-KV paged decode attention; contract in antfly_b200_noalloc.h.
int afb_paged_decode_attention_noalloc(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                                       const int* block_tables, int max_blocks, int page, const int* q_starts,
                                       const int* q_lens, const int* kv_lens, void* out, long out_stride, int B,
                                       int T, int Hq, int Hkv, int D, int max_q_len, int window, float scale,
                                       int num_splits, cudaStream_t stream) {
  using namespace afb;
  if (B <= 0 || T <= 0) return 0;
  if (num_splits < 1) num_splits = 1;
  if (D != 64 && D != 128 && D != 256) {
    set_last_error("afb_paged_decode_attention_noalloc: head_dim must be 64, 128 or 256 (got %d)", D);
    return -1;
  }
  if (Hkv <= 0 || Hq <= 0 || Hq % Hkv != 0 || max_q_len * (Hq / Hkv) > 16) {
    set_last_error("afb_paged_decode_attention_noalloc: needs q_len * (Hq / Hkv) <= 16 (decode shapes only)");
    return -1;
  }
  // A single split writes `out` directly and touches no scratch, so no size limit applies to it.
  const size_t rows = num_splits > 1 ? static_cast<size_t>(num_splits) * T * Hq : 0;
  const size_t o_bytes = (rows * D * sizeof(float) + 255) / 256 * 256;
  const size_t need = o_bytes + rows * sizeof(float);
  if (need > AFB_NOALLOC_SCRATCH_BYTES) {
    set_last_error(
        "afb_paged_decode_attention_noalloc: num_splits * T * Hq = %zu rows of D = %d need %zu bytes of scratch; "
        "the built-in array holds %d",
        rows, D, need, AFB_NOALLOC_SCRATCH_BYTES);
    return -1;
  }
  // One-time, per-device lookup of the array's device address (the symbol itself is not a device pointer).
  static void* scratch_of_device[64] = {nullptr};
  int dev = 0;
  AFB_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_last_error("afb_paged_decode_attention_noalloc: device ordinal %d out of range", dev);
    return -1;
  }
  if (!scratch_of_device[dev]) {
    void* ptr = nullptr;
    AFB_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_afb_noalloc_scratch));
    scratch_of_device[dev] = ptr;
  }
  unsigned char* base = static_cast<unsigned char*>(scratch_of_device[dev]);
  float* part_o = reinterpret_cast<float*>(base);
  float* part_lse = reinterpret_cast<float*>(base + o_bytes);
  return afb_attention(q, q_stride, nullptr, nullptr, 0, k_cache, v_cache, block_tables, max_blocks, page, q_starts,
                       q_lens, kv_lens, out, out_stride, part_o, part_lse, B, T, Hq, Hkv, D, max_q_len, 1, window,
                       scale, 1, 1, num_splits, stream);
}

}  // extern "C"
