// Flash attention on the 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05.mma instructions with the
// score tile S, the probability tile P and the output accumulator O living in tensor memory; Q, K and V tiles are
// staged in shared memory by TMA (128-byte swizzle, loads from this GPU's memory only, no multicast).
//
// Covers the compute-bound attention shapes: packed variable-length encoder attention (bidirectional, optional
// two-sided window) and causal prefill / speculative verification over the paged KV cache (sliding window, GQA).
// Semantics are those of the reference's flashCausalAttentionHost / gqaPagedAttentionDirect
// (zig/lib/linalg/src/attention.zig:88, zig/pkg/inference/src/ops/native_compute.zig:35093-35173); the reference's
// own CUDA kernel for the encoder case is a CTA per (query, head) with scalar loops
// (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:773).
//
// One CTA = one (sequence, query head, tile of 128 query rows); 6 warps:
//   warps 0-3  softmax: thread i of warp w owns query row 32 w + i = tensor-memory lane 32 w + i.  Per key tile it
//              reads S from TMEM (tcgen05.ld), keeps the running row maximum and sum, rescales its row of O in TMEM
//              when the maximum moved, and writes P as packed bf16 INTO S's own columns (tcgen05.st): P aliases S.
//   warp 4     TMA producer: Q once, then a ring of (K tile, V tile) stages.  Paged mode issues one TMA per cache
//              page (the block table gives the row coordinate); contiguous mode one per tile.
//   warp 5     allocates tensor memory and issues the MMAs (one elected lane):
//                S  = Q K^T   A = Q tile (K-major, shared),  B = K tile (K-major, shared)
//                O += P V     A = P (tensor memory),         B = V tile (MN-major, shared: V is [key, d] row-major, the
//                             contiguous dimension is N = d, which is what the TMA box of [keys x 64 d] yields)
// Tensor memory per CTA: BN columns for S / P and D columns for O, 256 allocated, so two CTAs share an SM and one
// CTA's softmax overlaps the other's MMAs.  Tile shapes: (D = 64, BN = 128 keys) and (D = 128, BN = 64 keys).
//
// Every mbarrier wait is bounded; a wait that gives up records a status code, the role leaves its loop, and the
// CTA still frees its tensor memory.  The TMA producer waits (bounded) for the loads it issued before it leaves.
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

struct AttnTcParams {
  const int* q_starts;      // [B] first packed query row of each sequence
  const int* q_lens;        // [B]
  const int* kv_lens;       // [B] keys visible to the sequence (contiguous mode: = q_lens)
  const int* block_tables;  // paged mode: [B, max_blocks]
  int max_blocks, page;
  __nv_bfloat16* out;       // [T, Hq * D]
  long out_stride;
  int Hq, Hkv;
  int causal, window, paged;
  float scale_log2;         // softmax scale * log2(e)
  int kv_box_rows;          // rows of one K / V TMA box (paged: the page size; contiguous: BN)
  long num_cache_rows;      // paged: num_blocks * page (block ids are range-checked against it)
};

template <int D, int BN>
struct AttnTcSmem {
  static constexpr int kPanels = D / 64;                 // 64-column (128-byte) panels per row
  static constexpr int kQBytes = kPanels * 128 * 128;    // 128 query rows
  static constexpr int kKBytes = kPanels * BN * 128;     // one K tile (= one V tile)
  static constexpr int kStages = 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQBytes;
  static constexpr int kVOff = kKOff + kStages * kKBytes;
  static constexpr int kBarOff = kVOff + kStages * kKBytes;
  static constexpr int kNumBars = 1 + 3 * kStages + 3;   // q_full, k_full[], v_full[], kv_empty[], s_full, p_full, o_done
  static constexpr int kNeeded = kBarOff + kNumBars * 8 + 16 + 1024;
  // At least 112 KiB, so that never more than two CTAs (2 x 256 tensor-memory columns = all 512) share an SM;
  // two of them (plus the 1 KiB the hardware reserves per CTA) still fit the SM's 228 KiB.
  static constexpr int kTotal = kNeeded > 112 * 1024 ? kNeeded : 112 * 1024;
  static constexpr int kTmemCols = 256;
  static_assert(BN + D <= kTmemCols, "S and O must fit the tensor-memory allocation");
  static_assert(3 * kTotal > 228 * 1024, "at most two CTAs per SM, or tensor memory is oversubscribed");
  static_assert(kTotal <= 113 * 1024, "two CTAs per SM are the design point");
};

template <int D, int BN>
__global__ void __launch_bounds__(192, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                    const __grid_constant__ CUtensorMap tma_v, AttnTcParams p) {
  using L = AttnTcSmem<D, BN>;
  constexpr int PANELS = L::kPanels;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kQOff;
  uint8_t* sK = smem + L::kKOff;
  uint8_t* sV = smem + L::kVOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = k_full + L::kStages;
  uint64_t* kv_empty = v_full + L::kStages;
  uint64_t* s_full = kv_empty + L::kStages;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_done = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, head = blockIdx.y, q_tile = blockIdx.x;
  const int q_start = p.q_starts[b], q_len = p.q_lens[b], kv_len = p.kv_lens[b];
  const int q0 = q_tile * 128;               // first query row of this tile inside the sequence
  if (q0 >= q_len) return;                   // whole CTA: nothing allocated yet
  const int G = p.Hq / p.Hkv;
  const int hk = head / G;
  const int pos_off = kv_len - q_len;        // absolute position of the sequence's first query row
  // key range this tile can see
  const int q_last = min(q_len, q0 + 128) - 1;
  int kv_hi = kv_len;
  if (p.causal) kv_hi = min(kv_len, pos_off + q_last + 1);
  else if (p.window > 0) kv_hi = min(kv_len, pos_off + q_last + p.window);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, pos_off + q0 - p.window + 1);
  const int tile_lo = kv_lo / BN;
  const int tile_hi = (kv_hi + BN - 1) / BN;
  const int ntiles = max(0, tile_hi - tile_lo);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, L::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;         // S: BN fp32 columns; P: BN / 2 columns of packed bf16, aliased
  const uint32_t tmem_o = tmem_base + BN;    // O: D fp32 columns

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && ntiles > 0) {
      mbar_expect_tx(q_full, L::kQBytes);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn)
        tma_load_2d(sQ + pn * (128 * 128), &tma_q, q_full, head * D + pn * 64, q_start + q0);
      const int* table = p.paged ? p.block_tables + static_cast<size_t>(b) * p.max_blocks : nullptr;
      const int boxes = BN / p.kv_box_rows;
      int issued = 0;
      bool alive = true;
      for (int j = 0; j < ntiles && alive; ++j) {
        const int s = j % L::kStages;
        const uint32_t ph = (j / L::kStages) & 1;
        if (!mbar_wait(&kv_empty[s], ph ^ 1, kStatusEmptyWaitTimeout)) { alive = false; break; }
        const int key0 = (tile_lo + j) * BN;
        mbar_expect_tx(&k_full[s], L::kKBytes);
        mbar_expect_tx(&v_full[s], L::kKBytes);
        for (int bx = 0; bx < boxes; ++bx) {
          const int key = key0 + bx * p.kv_box_rows;
          long row;
          if (p.paged) {
            // Pages past the sequence's last key are never looked at (masked): load page 0 of the table there.
            const int blk = table[min(key, max(kv_len - 1, 0)) / p.page];
            row = static_cast<long>(blk) * p.page;
            if (row < 0 || row + p.page > p.num_cache_rows) {
              status_set(kStatusBadIndex);
              row = 0;
            }
          } else {
            row = static_cast<long>(q_start) + key;   // contiguous: kv rows of the sequence start at q_start
          }
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn) {
            const int col = hk * D + pn * 64;
            const int dst = pn * (BN * 128) + bx * p.kv_box_rows * 128;
            tma_load_2d(sK + s * L::kKBytes + dst, &tma_k, &k_full[s], col, static_cast<int>(row));
            tma_load_2d(sV + s * L::kKBytes + dst, &tma_v, &v_full[s], col, static_cast<int>(row));
          }
        }
        ++issued;
      }
      if (!alive) {
        // Leaving early: wait (bounded) for the loads already issued, so nothing lands in this CTA's shared
        // memory after it has gone.
        for (int j = max(0, issued - L::kStages); j < issued; ++j) {
          const int s = j % L::kStages;
          const uint32_t ph = (j / L::kStages) & 1;
          mbar_wait(&k_full[s], ph, kStatusTmaWaitTimeout);
          mbar_wait(&v_full[s], ph, kStatusTmaWaitTimeout);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && ntiles > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, BN);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, D, 0, 1);   // B = V is MN-major
      bool alive = mbar_wait(q_full, 0, kStatusTmaWaitTimeout);
      for (int j = 0; j < ntiles && alive; ++j) {
        const int s = j % L::kStages;
        const uint32_t ph = (j / L::kStages) & 1;
        // S is overwritten: the previous tile's P V (which reads P out of S's columns) must have completed.
        if (j > 0 && !mbar_wait(o_done, (j - 1) & 1, kStatusMmaWaitTimeout)) { alive = false; break; }
        if (!mbar_wait(&k_full[s], ph, kStatusTmaWaitTimeout)) { alive = false; break; }
        tcgen05_fence_after();
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) {
          const uint64_t adesc = umma_desc_k_sw128(smem_u32(sQ + pn * (128 * 128)));
          const uint64_t bdesc = umma_desc_k_sw128(smem_u32(sK + s * L::kKBytes + pn * (BN * 128)));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_s, adesc + 2 * k, bdesc + 2 * k, idesc_qk, (pn | k) != 0);
        }
        umma_commit(s_full);
        if (!mbar_wait(p_full, j & 1, kStatusGridFlagTimeout)) { alive = false; break; }
        if (!mbar_wait(&v_full[s], ph, kStatusTmaWaitTimeout)) { alive = false; break; }
        tcgen05_fence_after();
        const uint32_t vbase = smem_u32(sV + s * L::kKBytes);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // 16 keys per instruction: two 8-row groups of 1024 bytes; 64-wide d panels BN * 128 bytes apart
          const uint64_t bdesc = umma_desc_mn_sw128(vbase + kk * 2048, BN * 128);
          umma_bf16_ts(tmem_o, tmem_s + kk * 8, bdesc, idesc_pv, (j | kk) != 0);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(o_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 0..3)
    const int row = warp * 32 + lane;                // row of the tile = TMEM lane
    const int qi = q0 + row;                         // query row inside the sequence
    const bool row_ok = qi < q_len;
    const int qpos = pos_off + qi;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.0f;
    bool alive = ntiles > 0;
    for (int j = 0; j < ntiles && alive; ++j) {
      // warp-uniform outcome: the tcgen05.ld / st and votes below need the whole warp
      alive = __all_sync(0xffffffffu, mbar_wait(s_full, j & 1, kStatusMmaWaitTimeout));
      if (!alive) break;
      tcgen05_fence_after();
      const int key0 = (tile_lo + j) * BN;
      // does this tile need per-element masking for this row?
      int k_end = kv_len;                            // keys [k_beg, k_end) are visible
      int k_beg = 0;
      if (p.causal) k_end = min(k_end, qpos + 1);
      else if (p.window > 0) k_end = min(k_end, qpos + p.window);
      if (p.window > 0) k_beg = max(0, qpos - p.window + 1);
      const bool full = row_ok && key0 >= k_beg && key0 + BN <= k_end;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c, r);
        tmem_ld_wait();
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c + i;
            if (key >= k_beg && key < k_end) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = exp2f(m_run - m_use);      // m_run = -inf gives 0: nothing accumulated yet
      m_run = m_new;
      l_run *= alpha;
      // rescale this row of O when some row of the warp moved its maximum (tcgen05.ld / st are warp-wide)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
        for (int c = 0; c < D; c += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_o + lane_addr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x16(tmem_o + lane_addr + c, r);
        }
      }
      // pass 2: probabilities, row sum, P (bf16 pairs) written over the S columns already consumed
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = exp2f(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, -m_use));
          float p1 = exp2f(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, -m_use));
          if (!full) {
            const int key = key0 + c + 2 * i;
            if (!(row_ok && key >= k_beg && key < k_end)) p0 = 0.0f;
            if (!(row_ok && key + 1 >= k_beg && key + 1 < k_end)) p1 = 0.0f;
          }
          l_run += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x32b_x16(tmem_s + lane_addr + (c >> 1), pk);
      }
      tmem_st_wait();
      tcgen05_fence_before();
      mbar_arrive(p_full);
    }
    // epilogue: O / l -> bf16
    if (alive && ntiles > 0)
      alive = __all_sync(0xffffffffu, mbar_wait(o_done, (ntiles - 1) & 1, kStatusMmaWaitTimeout));
    tcgen05_fence_after();
    if (alive && ntiles > 0) {
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      __nv_bfloat16* op = p.out + static_cast<size_t>(q_start + qi) * p.out_stride + head * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_o + lane_addr + c, r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
            *reinterpret_cast<uint4*>(op + c + 8 * i) = u;
          }
        }
      }
    } else if (ntiles == 0 && row_ok) {
      // no visible key at all (cannot happen with the masks above, kept for safety): zeros
      __nv_bfloat16* op = p.out + static_cast<size_t>(q_start + qi) * p.out_stride + head * D;
      for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(op + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, L::kTmemCols);
}

template <int D, int BN>
int launch_attention_tc(const void* q, long q_stride, long q_rows, const void* k, const void* v, long kv_stride,
                        long kv_rows, int kv_cols, AttnTcParams p, int B, int max_q_len, cudaStream_t stream) {
  using L = AttnTcSmem<D, BN>;
  CUtensorMap tq, tk, tv;
  // Q: [q_rows tokens, Hq * D] with row pitch q_stride; boxes of 128 rows x 64 columns
  if (make_tmap_2d(&tq, q, 2, q_rows, static_cast<uint64_t>(p.Hq) * D, static_cast<uint64_t>(q_stride) * 2, 128, 64, 3))
    return -1;
  if (make_tmap_2d(&tk, k, 2, kv_rows, kv_cols, static_cast<uint64_t>(kv_stride) * 2, p.kv_box_rows, 64, 3)) return -1;
  if (make_tmap_2d(&tv, v, 2, kv_rows, kv_cols, static_cast<uint64_t>(kv_stride) * 2, p.kv_box_rows, 64, 3)) return -1;
  AFB_CONFIGURE_KERNEL((attention_tc_kernel<D, BN>), L::kTotal, 192, L::kTmemCols);
  dim3 grid((max_q_len + 127) / 128, p.Hq, B);
  attention_tc_kernel<D, BN><<<grid, 192, L::kTotal, stream>>>(tq, tk, tv, p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace afb

extern "C" {

// Tensor-core flash attention.  paged = 0: k / v are packed [T, Hkv * D]-like rows with token pitch kv_stride
// (the K and V rows of sequence b start at q_starts[b]; kv_lens == q_lens).  paged = 1: k_cache / v_cache
// [num_blocks, page, Hkv, D] with block_tables; query rows are the LAST q_lens[b] positions of a sequence of
// kv_lens[b] keys already in the cache.  D is 64 or 128; the page size must divide the key tile (128 keys at
// D = 64, 64 keys at D = 128) and be a multiple of 8.  Returns -1 with afb_last_error() for shapes it does not
// take (the caller then uses the mma.sync kernel).
int afb_attention_tc(const void* q, long q_stride, const void* k, const void* v, long kv_stride, const void* k_cache,
                     const void* v_cache, const int* block_tables, int max_blocks, int page, long num_blocks,
                     const int* q_starts, const int* q_lens, const int* kv_lens, void* out, long out_stride, int B,
                     int T, int Hq, int Hkv, int D, int max_q_len, int causal, int window, float scale, int paged,
                     cudaStream_t stream) {
  using namespace afb;
  if (B <= 0 || T <= 0 || max_q_len <= 0) return 0;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv != 0) {
    set_last_error("afb_attention_tc: head_dim 64 or 128 and Hq a multiple of Hkv (D=%d Hq=%d Hkv=%d)", D, Hq, Hkv);
    return -1;
  }
  if ((q_stride & 7) || (out_stride & 7) || (reinterpret_cast<uintptr_t>(out) & 15) || !(scale > 0.0f)) {
    set_last_error("afb_attention_tc: q / out token pitch must be a multiple of 8 elements, out 16-byte aligned");
    return -1;
  }
  const int BN = D == 64 ? 128 : 64;
  AttnTcParams p = {};
  p.q_starts = q_starts; p.q_lens = q_lens; p.kv_lens = kv_lens;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.page = page;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.out_stride = out_stride;
  p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.window = window; p.paged = paged;
  p.scale_log2 = scale * 1.4426950408889634f;
  const void* kp = k;
  const void* vp = v;
  long kv_rows = T, pitch = kv_stride;
  if (paged) {
    if (page <= 0 || (page & 7) || BN % page != 0 || !block_tables || max_blocks <= 0 || num_blocks <= 0) {
      set_last_error("afb_attention_tc: the page size must be a multiple of 8 that divides %d (page=%d)", BN, page);
      return -1;
    }
    p.kv_box_rows = page;
    p.num_cache_rows = num_blocks * page;
    kp = k_cache; vp = v_cache;
    kv_rows = p.num_cache_rows;
    pitch = static_cast<long>(Hkv) * D;
  } else {
    if (kv_stride & 7) {
      set_last_error("afb_attention_tc: k / v token pitch must be a multiple of 8 elements");
      return -1;
    }
    p.kv_box_rows = BN;
  }
  const int kv_cols = Hkv * D;
  if (D == 64)
    return launch_attention_tc<64, 128>(q, q_stride, T, kp, vp, pitch, kv_rows, kv_cols, p, B, max_q_len, stream);
  return launch_attention_tc<128, 64>(q, q_stride, T, kp, vp, pitch, kv_rows, kv_cols, p, B, max_q_len, stream);
}

}  // extern "C"
