// IVF list scan: scores the members of every probed posting list against exactly the queries that probe it, in one
// launch, and appends (distance, sorted-row) pairs that beat the query's threshold to that query's candidate list.
//
// The reference walks the probed postings on the CPU, one posting at a time
// (zig/lib/vectorindex/src/hbc_index.zig:1720-1775 scoreLeafMemberIds after selectFlatRabitqPostings,
// spfresh_index.zig:350).  Here the (query, list) pairs of a whole query batch are sorted by list on the device
// and this kernel is a grouped GEMM over them: vectors are stored sorted by list, a list's rows are streamed from
// HBM once and multiplied with the (few) queries that probe it.
//
// Work split: persistent CTAs take lists round-robin (list l -> CTA l % gridDim.x, so the order is fixed and the
// candidate contents are reproducible up to append order).  For a list, queries are processed in groups of 8
// (the N of mma.m16n8k16): the group's query vectors are gathered into shared memory once, then the list's rows
// stream through a cp.async ring in tiles of 64 rows x 128 dims (128-byte-row swizzle, ldmatrix), each of the
// four warps owning 16 rows.  The op is HBM-bound (a row of D bf16 is read for a handful of queries: a few FLOP
// per byte), so the legacy tensor-core instruction is not the limiter; what matters is that a list is read once.
//
// Every index read from the work arrays is range-checked; a bad one records kStatusBadIndex and the item is skipped.
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

struct IvfScanParams {
  const __nv_bfloat16* x;      // [n_rows, D] vectors sorted by list
  long ldx;
  const float* col_term;       // [n_rows] or null
  const __nv_bfloat16* q;      // [n_queries, D]
  long ldq;
  const float* row_term;       // [n_queries] or null
  const float* threshold;      // [n_queries] keep distance < threshold[q]; null: keep everything
  const long* list_off;        // [n_lists + 1] first sorted row of each list
  const int* pair_off;         // [n_lists + 1] first (sorted) pair of each list
  const int* pair_query;       // [n_pairs] query of each pair, pairs sorted by list
  float* cand_val;             // [n_queries, cap]
  int* cand_idx;               // [n_queries, cap]  sorted-row ids
  int* cand_count;             // [n_queries]  (may exceed cap: the consumer detects overflow)
  int n_lists, n_queries, n_pairs, D, cap;
  long n_rows;
  float scale;
  int clamp_zero;
};

constexpr int kIvfRows = 64;      // rows per tile
constexpr int kIvfKc = 128;       // dims per tile
constexpr int kIvfStages = 3;
constexpr int kIvfQ = 8;          // queries per group
constexpr int kIvfMaxD = 2048;

__device__ __forceinline__ void ivf_cp_async_16(void* smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void ivf_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ivf_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ivf_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ivf_mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Loads rows [row0, row0 + 64) x dims [k0, k0 + 128) of x into a swizzled tile: row r at r * 256 bytes, its 16-byte
// chunk c stored at chunk (c ^ (r & 7)).  Rows past row_end and dims past D are zero-filled.
__device__ __forceinline__ void ivf_load_tile(uint8_t* tile, const IvfScanParams& p, long row0, long row_end, int k0) {
  // 64 rows x 16 chunks = 1024 chunks, 128 threads -> 8 each; a thread keeps its chunk column, rows step by 8.
  const int ch = threadIdx.x & 15, r0 = threadIdx.x >> 4;
  const int kk = k0 + ch * 8;
  const int k_bytes = kk < p.D ? min(16, (p.D - kk) * 2) : 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + i * 8;
    const long row = row0 + r;
    const bool ok = row < row_end && k_bytes > 0;
    const __nv_bfloat16* src = p.x + (ok ? row : 0) * p.ldx + (ok ? kk : 0);
    ivf_cp_async_16(tile + r * 256 + ((ch ^ (r & 7)) * 16), src, ok ? k_bytes : 0);
  }
}

__global__ void __launch_bounds__(128) ivf_scan_kernel(IvfScanParams p) {
  extern __shared__ __align__(128) uint8_t ivf_smem[];
  // query group [8][D + 8] bf16 (row padded by 16 bytes: the B-fragment reads of the 8 queries then fall into
  // different banks), then the tile ring
  const int qpitch = p.D + 8;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(ivf_smem);
  const int q_bytes = ((kIvfQ * qpitch * 2) + 127) / 128 * 128;
  uint8_t* ring = ivf_smem + q_bytes;
  __shared__ int s_qid[kIvfQ];
  __shared__ float s_thr[kIvfQ], s_rterm[kIvfQ];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int mi = lane >> 3, rin = lane & 7;
  const int kchunks = (p.D + kIvfKc - 1) / kIvfKc;

  for (int l = blockIdx.x; l < p.n_lists; l += gridDim.x) {
    const int p_begin = p.pair_off[l], p_end = p.pair_off[l + 1];
    if (p_end <= p_begin) continue;
    const long r_begin = p.list_off[l], r_end = p.list_off[l + 1];
    if (r_end <= r_begin) continue;
    if (p_begin < 0 || p_end > p.n_pairs || r_begin < 0 || r_end > p.n_rows) {
      if (threadIdx.x == 0) status_set(kStatusBadIndex);
      continue;
    }
    for (int pg = p_begin; pg < p_end; pg += kIvfQ) {
      const int nq = min(kIvfQ, p_end - pg);
      __syncthreads();  // the previous group's readers of q_s / s_* are done
      if (threadIdx.x < kIvfQ) {
        int qi = threadIdx.x < nq ? p.pair_query[pg + threadIdx.x] : -1;
        if (qi >= p.n_queries || (threadIdx.x < nq && qi < 0)) {
          status_set(kStatusBadIndex);
          qi = -1;
        }
        s_qid[threadIdx.x] = qi;
        s_thr[threadIdx.x] = qi >= 0 ? (p.threshold ? p.threshold[qi] : INFINITY) : -INFINITY;
        s_rterm[threadIdx.x] = (qi >= 0 && p.row_term) ? p.row_term[qi] : 0.0f;
      }
      __syncthreads();
      // gather the group's query vectors (16-byte chunks; D is a multiple of 8)
      for (int i = threadIdx.x; i < kIvfQ * (p.D / 8); i += blockDim.x) {
        const int qq = i / (p.D / 8), c = i % (p.D / 8);
        const int qi = s_qid[qq];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (qi >= 0) v = *reinterpret_cast<const uint4*>(p.q + static_cast<long>(qi) * p.ldq + c * 8);
        *reinterpret_cast<uint4*>(q_s + qq * qpitch + c * 8) = v;
      }
      __syncthreads();

      for (long row0 = r_begin; row0 < r_end; row0 += kIvfRows) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        // ring over the K chunks of this row tile
#pragma unroll
        for (int s0 = 0; s0 < kIvfStages - 1; ++s0) {
          if (s0 < kchunks) ivf_load_tile(ring + s0 * (kIvfRows * 256), p, row0, r_end, s0 * kIvfKc);
          ivf_cp_async_commit();
        }
        for (int kc = 0; kc < kchunks; ++kc) {
          const int nxt = kc + kIvfStages - 1;
          if (nxt < kchunks) ivf_load_tile(ring + (nxt % kIvfStages) * (kIvfRows * 256), p, row0, r_end, nxt * kIvfKc);
          ivf_cp_async_commit();
          ivf_cp_async_wait<kIvfStages - 1>();
          __syncthreads();
          const uint8_t* tile = ring + (kc % kIvfStages) * (kIvfRows * 256);
          const int row = warp * 16 + (mi & 1) * 8 + rin;  // ldmatrix row of this lane
#pragma unroll
          for (int ks = 0; ks < kIvfKc / 16; ++ks) {
            const int chunk = ks * 2 + (mi >> 1);
            uint32_t a[4];
            ivf_ldmatrix_x4(a, tile + row * 256 + ((chunk ^ (row & 7)) * 16));
            const int kabs = kc * kIvfKc + ks * 16 + 2 * t;  // dims beyond D hold zeros in the tile
            uint32_t b0 = 0u, b1 = 0u;
            if (kabs < p.D) b0 = *reinterpret_cast<const uint32_t*>(q_s + g * qpitch + kabs);
            if (kabs + 8 < p.D) b1 = *reinterpret_cast<const uint32_t*>(q_s + g * qpitch + kabs + 8);
            ivf_mma_16816(acc, a, b0, b1);
          }
          __syncthreads();  // the stage may be overwritten by the load issued two iterations on
        }
        // acc[0], acc[1]: row g, queries 2t, 2t + 1;  acc[2], acc[3]: row g + 8, same queries
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const long row = row0 + warp * 16 + g + 8 * (e >> 1);
          const int qq = 2 * t + (e & 1);
          const int qi = s_qid[qq];
          if (row < r_end && qi >= 0) {
            float d = p.scale * acc[e] + s_rterm[qq] + (p.col_term ? p.col_term[row] : 0.0f);
            if (p.clamp_zero) d = fmaxf(d, 0.0f);
            if (d < s_thr[qq]) {
              const int pos = atomicAdd(&p.cand_count[qi], 1);
              if (pos < p.cap) {
                p.cand_val[static_cast<size_t>(qi) * p.cap + pos] = d;
                p.cand_idx[static_cast<size_t>(qi) * p.cap + pos] = static_cast<int>(row);
              }
            }
          }
        }
      }
    }
  }
}

}  // namespace afb

extern "C" {

// One launch scores every (list, query) pair: pairs sorted by list (pair_query), pair_off[l] .. pair_off[l + 1] the
// pairs of list l, list_off the sorted-row ranges.  Appends (distance, sorted row) with distance < threshold[q]
// (threshold null: everything) to the candidate lists; cand_count may end above cap (overflow, seen by the select).
int afb_ivf_scan(const void* x, long ldx, const float* col_term, const void* q, long ldq, const float* row_term,
                 const float* threshold, const long* list_off, const int* pair_off, const int* pair_query,
                 float* cand_val, int* cand_idx, int* cand_count, int n_lists, int n_queries, int n_pairs, long n_rows,
                 int D, int cap, float scale, int clamp_zero, cudaStream_t stream) {
  using namespace afb;
  if (n_lists <= 0 || n_pairs <= 0 || n_queries <= 0) return 0;
  if (D % 8 != 0 || D <= 0 || D > kIvfMaxD || (ldx % 8) != 0 || (ldq % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15)) {
    set_last_error("afb_ivf_scan: dimension must be a multiple of 8 (at most %d) with 16-byte aligned rows (D=%d)",
                   kIvfMaxD, D);
    return -1;
  }
  if (n_rows > 0x7fffffffL) {
    set_last_error("afb_ivf_scan: at most 2^31 - 1 rows per shard (row ids are 32-bit)");
    return -1;
  }
  IvfScanParams p;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.col_term = col_term;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q); p.ldq = ldq; p.row_term = row_term; p.threshold = threshold;
  p.list_off = list_off; p.pair_off = pair_off; p.pair_query = pair_query;
  p.cand_val = cand_val; p.cand_idx = cand_idx; p.cand_count = cand_count;
  p.n_lists = n_lists; p.n_queries = n_queries; p.n_pairs = n_pairs; p.D = D; p.cap = cap; p.n_rows = n_rows;
  p.scale = scale; p.clamp_zero = clamp_zero;
  const int q_bytes = ((kIvfQ * (D + 8) * 2) + 127) / 128 * 128;
  const int smem = q_bytes + kIvfStages * kIvfRows * 256;
  AFB_CONFIGURE_KERNEL(ivf_scan_kernel, smem, 128, 0);
  const int sms = device_sm_count();
  int ctas = sms * 4;
  if (ctas > n_lists) ctas = n_lists;
  ivf_scan_kernel<<<ctas, 128, smem, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
