// Vector-index kernels that are not GEMMs:
//   * top-k selection / merge over per-query candidate lists (sources may live on peer GPUs: the cross-GPU merge
//     of a sharded search reads every shard's candidates straight out of peer memory),
//   * k-means centroid update (vectorised atomic accumulation + finalise with shift, norms, optional normalise),
//   * squared row norms,
//   * RaBitQ 1-bit x 4-bit weighted-popcount scorer fused with the distance estimator.
//
// Semantics follow the reference: search results sorted by ascending distance (zig/lib/vectorindex/src/search.zig),
// Lloyd update where an empty cluster keeps its old centroid and cosine centroids are re-normalised
// (zig/lib/vectorindex/src/kmeans.zig:283-296, 364-420), RaBitQ bitProduct / estimateDistances
// (zig/lib/vector/src/rabitq.zig:40-102, quantizer.zig:317-470).
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

// ---------------------------------------------------------------------------------------------------------
// Top-k select.  One CTA per query.  Gathers up to `max_total` (distance, id) pairs from `n_src` lists
// (source s: vals[s] + q*stride[s], counts[s][q] entries, or a fixed length when counts[s] is null), bitonic-sorts
// them in shared memory and writes the k best.  Ties break on the smaller id so results are deterministic.
// ---------------------------------------------------------------------------------------------------------
constexpr int kMaxSources = 16;

struct SelectParams {
  const float* vals[kMaxSources];
  const int* idxs[kMaxSources];
  const int* counts[kMaxSources];
  long stride[kMaxSources];
  int fixed_len[kMaxSources];
  int n_src;
  int k;
  int sort_cap;  // power of two >= every query's total
  float* out_val;  // [Q, k]
  int* out_idx;    // [Q, k]
  float* out_thr;  // [Q] k-th best distance (+inf when fewer than k candidates), optional
  int* overflow;   // set to 1 when some query had more candidates than sort_cap
  // Cross-GPU merge of a sharded search, push side (the tail of a shard's local search): the k best of query q
  // are ALSO stored into every rank's merge buffer (slot of this rank) through peer pointers, with one flag
  // word per query saying whether any candidate buffer of this shard overflowed, and every rank's arrival
  // counter is bumped once per query CTA (red.release.sys after the stores).
  float* push_val[8];  // rank o's [Q, k] value slot for this rank
  int* push_idx[8];
  int* push_flag[8];   // rank o's [Q] overflow flags for this rank
  int* push_ready[8];  // rank o's arrival counter
  int n_push;
  const int* sticky_overflow;  // overflow word of the earlier selects of this search (they have completed)
  // Merge side: wait (bounded) until this rank's own arrival counter has reached wait_target before reading the
  // sources, which are then all in local memory; src_flag[s][q] != 0 is OR-ed into *overflow.
  const int* wait_ready;
  int wait_target;
  const int* src_flag[kMaxSources];
};

__global__ void topk_select_kernel(SelectParams p) {
  extern __shared__ uint8_t sel_smem[];
  float* sv = reinterpret_cast<float*>(sel_smem);
  int* si = reinterpret_cast<int*>(sel_smem + static_cast<size_t>(p.sort_cap) * 4);
  __shared__ int s_total;
  const int q = blockIdx.x;
  __shared__ int s_ovf;
  if (threadIdx.x == 0) {
    s_total = 0;
    s_ovf = 0;
    // Every rank's list has landed in this GPU's memory once the counter reads the target.  On expiry the status
    // word is set (the host sees it) and the kernel carries on over whatever is there, so it still terminates.
    if (p.wait_ready) peer_wait_counter(p.wait_ready, p.wait_target);
  }
  for (int i = threadIdx.x; i < p.sort_cap; i += blockDim.x) { sv[i] = INFINITY; si[i] = 0x7fffffff; }
  __syncthreads();
  for (int s = 0; s < p.n_src; ++s) {
    if (p.src_flag[s] && threadIdx.x == 0 && p.src_flag[s][q] != 0) {
      s_ovf = 1;
      if (p.overflow) *p.overflow = 1;
    }
    int n = p.counts[s] ? p.counts[s][q] : p.fixed_len[s];
    if (p.counts[s] && n > p.fixed_len[s]) {  // producer overflowed its buffer
      if (threadIdx.x == 0) {
        s_ovf = 1;
        if (p.overflow) *p.overflow = 1;
      }
      n = p.fixed_len[s];
    }
    __shared__ int s_base;
    if (threadIdx.x == 0) { s_base = s_total; s_total += n; }
    __syncthreads();
    const int base = s_base;
    const float* v = p.vals[s] + static_cast<size_t>(q) * p.stride[s];
    const int* ix = p.idxs[s] + static_cast<size_t>(q) * p.stride[s];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      if (base + i < p.sort_cap) { sv[base + i] = v[i]; si[base + i] = ix[i]; }
      else {
        s_ovf = 1;
        if (p.overflow) *p.overflow = 1;
      }
    }
    __syncthreads();
  }
  const int total = min(s_total, p.sort_cap);
  int n2 = 1;
  while (n2 < total) n2 <<= 1;
  if (n2 < 2) n2 = 2;
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n2 / 2; i += blockDim.x) {
        const int lo = (i / stride) * (stride << 1) + (i % stride);
        const int hi = lo + stride;
        const bool asc = ((lo & size) == 0);
        const float a = sv[lo], b = sv[hi];
        const int ia = si[lo], ib = si[hi];
        const bool a_gt_b = (a > b) || (a == b && ia > ib);
        if (a_gt_b == asc) { sv[lo] = b; sv[hi] = a; si[lo] = ib; si[hi] = ia; }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < p.k; i += blockDim.x) {
    const bool ok = i < total;
    p.out_val[static_cast<size_t>(q) * p.k + i] = ok ? sv[i] : INFINITY;
    p.out_idx[static_cast<size_t>(q) * p.k + i] = ok ? si[i] : -1;
  }
  if (p.out_thr && threadIdx.x == 0) p.out_thr[q] = (total >= p.k) ? sv[p.k - 1] : INFINITY;
  // A rank whose status word carries a cross-GPU timeout pushes nothing more (its counters and its peers' no
  // longer agree; rows of a later search must not complete a slower peer's older arrival target).
  if (p.n_push && !(status_peek() & kStatusPeerFlagTimeout)) {
    for (int o = 0; o < p.n_push; ++o) {
      float* pv = p.push_val[o] + static_cast<size_t>(q) * p.k;
      int* pi = p.push_idx[o] + static_cast<size_t>(q) * p.k;
      for (int i = threadIdx.x; i < p.k; i += blockDim.x) {
        const bool ok = i < total;
        pv[i] = ok ? sv[i] : INFINITY;
        pi[i] = ok ? si[i] : -1;
      }
    }
    __syncthreads();  // every thread's peer stores are issued (and s_ovf is final) before the release below
    if (threadIdx.x == 0) {
      const int flag = (s_ovf || (p.sticky_overflow && *p.sticky_overflow)) ? 1 : 0;
      for (int o = 0; o < p.n_push; ++o) p.push_flag[o][q] = flag;
      __threadfence_system();
      for (int o = 0; o < p.n_push; ++o) peer_red_release_add(p.push_ready[o], 1);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// k-means update
// ---------------------------------------------------------------------------------------------------------
// One warp per point: sums[assign[m], :] += x[m, :], counts[assign[m]] += 1.
__global__ void kmeans_accumulate_kernel(const __nv_bfloat16* x, long ldx, const int* assign, float* sums,
                                         int* counts, int M, int D, int K) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= M) return;
  const int c = assign[warp];
  if (c < 0 || c >= K) { if (lane == 0) status_set(kStatusBadIndex); return; }
  const __nv_bfloat16* row = x + static_cast<size_t>(warp) * ldx;
  float* dst = sums + static_cast<size_t>(c) * D;
  for (int i = lane * 4; i < D; i += 128) {
    const uint2 u = *reinterpret_cast<const uint2*>(row + i);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    atomicAdd(reinterpret_cast<float4*>(dst + i), make_float4(a.x, a.y, b.x, b.y));
  }
  if (lane == 0) atomicAdd(&counts[c], 1);
}

// One CTA per centroid: new = sums / count (old centroid kept when the cluster is empty), optional L2 normalise,
// bf16 + fp32 copies, squared norm, and the squared shift accumulated into *shift.
__global__ void kmeans_finalize_kernel(const float* sums, const int* counts, float* cent_f32, __nv_bfloat16* cent_bf16,
                                       float* cent_sqnorm, float* shift, int D, int normalize) {
  __shared__ float red[32];
  const int c = blockIdx.x;
  const int n = counts[c];
  float ss = 0.0f;
  if (n > 0 && normalize) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      const float v = sums[static_cast<size_t>(c) * D + i] / n;
      ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = (threadIdx.x & 31) < ((blockDim.x + 31) >> 5) ? red[threadIdx.x & 31] : 0.0f;
    ss = warp_sum(ss);
    __syncthreads();
  }
  const float inv = (n > 0 && normalize && ss > 0.0f) ? rsqrtf(ss) : 1.0f;
  float dsum = 0.0f, nsum = 0.0f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const size_t o = static_cast<size_t>(c) * D + i;
    const float old = cent_f32[o];
    const float nv = n > 0 ? sums[o] / n * inv : old;
    const float d = nv - old;
    dsum += d * d;
    cent_f32[o] = nv;
    const __nv_bfloat16 hb = __float2bfloat16(nv);
    cent_bf16[o] = hb;
    const float hv = __bfloat162float(hb);
    nsum += hv * hv;  // norm of what the assignment GEMM will actually multiply
  }
  dsum = warp_sum(dsum);
  nsum = warp_sum(nsum);
  __shared__ float red2[32], red3[32];
  if ((threadIdx.x & 31) == 0) { red2[threadIdx.x >> 5] = dsum; red3[threadIdx.x >> 5] = nsum; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = (blockDim.x + 31) >> 5;
    float a = threadIdx.x < nw ? red2[threadIdx.x] : 0.0f;
    float b = threadIdx.x < nw ? red3[threadIdx.x] : 0.0f;
    a = warp_sum(a);
    b = warp_sum(b);
    if (threadIdx.x == 0) {
      atomicAdd(shift, a);
      cent_sqnorm[c] = b;
    }
  }
}

// out[m] = sum_d x[m, d]^2 (fp32), one warp per row.
__global__ void row_sqnorm_kernel(const __nv_bfloat16* x, long ldx, float* out, int M, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= M) return;
  const __nv_bfloat16* row = x + static_cast<size_t>(warp) * ldx;
  float s = 0.0f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(row + i));
    s += v.x * v.x + v.y * v.y;
  }
  s = warp_sum(s);
  if (lane == 0) out[warp] = s;
}

// Gathers rows (e.g. exact re-scoring of a short list): out[i, :] = x[idx[i], :].
__global__ void gather_rows_kernel(const __nv_bfloat16* x, long ldx, const int* idx, __nv_bfloat16* out, int n, int D,
                                   long rows) {
  const int r = blockIdx.x;
  long src = idx[r];
  if (src < 0 || src >= rows) src = 0;
  for (int i = threadIdx.x * 8; i < D; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * D + i) =
        *reinterpret_cast<const uint4*>(x + static_cast<size_t>(src) * ldx + i);
}

// ---------------------------------------------------------------------------------------------------------
// RaBitQ: bit_product(code, q1..q4) = pop(code&q1) + 2 pop(code&q2) + 4 pop(code&q3) + 8 pop(code&q4), then the
// estimator  est = (t1 * bp + t2 * code_count - t34) * inv_dot  and the metric-specific distance / error bound.
// metric: 0 l2_squared, 1 inner_product, 2 cosine.
// ---------------------------------------------------------------------------------------------------------
struct RabitqParams {
  const unsigned long long* codes;  // [n, width]
  const unsigned long long* qplanes;  // [4, width]
  const unsigned int* code_counts;  // [n]
  const float* centroid_dist;       // [n]
  const float* inv_dot;             // [n]  1 / <o_bar, o>
  const float* centroid_dot;        // [n]  (ip / cosine)
  float* dist;                      // [n]
  float* err;                       // [n]
  unsigned int* bit_products;       // [n] optional raw output
  int n, width, metric;
  float t1, t2, t34, q_cdist, q_cdot, sq_cnorm, sqrt_dims, q_norm;
  const float* data_norms;          // [n] (cosine)
};

__global__ void rabitq_estimate_kernel(RabitqParams p) {
  extern __shared__ unsigned long long sq[];  // [4 * width]
  for (int i = threadIdx.x; i < 4 * p.width; i += blockDim.x) sq[i] = p.qplanes[i];
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.n) return;
  const unsigned long long* code = p.codes + static_cast<size_t>(i) * p.width;
  unsigned int s1 = 0, s2 = 0, s4 = 0, s8 = 0;
  for (int w = 0; w < p.width; ++w) {
    const unsigned long long c = code[w];
    s1 += __popcll(c & sq[w]);
    s2 += __popcll(c & sq[p.width + w]);
    s4 += __popcll(c & sq[2 * p.width + w]);
    s8 += __popcll(c & sq[3 * p.width + w]);
  }
  const unsigned int bp = s1 + (s2 << 1) + (s4 << 2) + (s8 << 3);
  if (p.bit_products) p.bit_products[i] = bp;
  if (!p.dist) return;
  const float est = (p.t1 * static_cast<float>(bp) + p.t2 * static_cast<float>(p.code_counts[i]) - p.t34) * p.inv_dot[i];
  const float dcd = p.centroid_dist[i];
  float d, e;
  if (p.metric == 0) {
    const float mult = 2.0f * dcd * p.q_cdist;
    d = dcd * dcd + p.q_cdist * p.q_cdist - mult * est;
    e = mult / p.sqrt_dims;
    if (d < 0.0f) { e = fmaxf(e + d, 0.0f); d = 0.0f; }
  } else {
    const float mult = dcd * p.q_cdist;
    const float ip = mult * est + p.centroid_dot[i] + p.q_cdot - p.sq_cnorm;
    e = mult / p.sqrt_dims;
    if (p.metric == 1) {
      d = -ip;
    } else {
      const float den = p.q_norm * (p.data_norms ? p.data_norms[i] : 1.0f);
      d = den > 0.0f ? 1.0f - ip / den : 1.0f;
      e = den > 0.0f ? e / den : 0.0f;
    }
  }
  p.dist[i] = d;
  if (p.err) p.err[i] = e;
}

}  // namespace afb

extern "C" {

// Sources: n_src lists; list s holds for query q `counts[s][q]` (or fixed_len[s] when counts[s] is null) pairs at
// vals[s] + q*stride[s].  Pointers may be peer-GPU addresses.
int afb_topk_select_x(const float* const* vals, const int* const* idxs, const int* const* counts,
                      const long* stride, const int* fixed_len, int n_src, int n_queries, int k, int max_total,
                      float* out_val, int* out_idx, float* out_thr, int* overflow, void* const* push_val,
                      void* const* push_idx, void* const* push_flag, void* const* push_ready, int n_push,
                      const int* sticky_overflow, const int* wait_ready, int wait_target,
                      const int* const* src_flag, cudaStream_t stream);

int afb_topk_select(const float* const* vals, const int* const* idxs, const int* const* counts, const long* stride,
                    const int* fixed_len, int n_src, int n_queries, int k, int max_total, float* out_val,
                    int* out_idx, float* out_thr, int* overflow, cudaStream_t stream) {
  return afb_topk_select_x(vals, idxs, counts, stride, fixed_len, n_src, n_queries, k, max_total, out_val, out_idx,
                           out_thr, overflow, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, nullptr,
                           stream);
}

// As afb_topk_select, plus the two halves of the cross-GPU merge of a sharded search (see SelectParams):
// n_push > 0 also stores each query's k best into n_push ranks' merge buffers and bumps their arrival counters;
// wait_ready != null first waits, bounded, for this rank's own counter to reach wait_target.  A wait that runs
// out sets the status word (afb_status_read) and the kernel finishes over what is there.
int afb_topk_select_x(const float* const* vals, const int* const* idxs, const int* const* counts,
                      const long* stride, const int* fixed_len, int n_src, int n_queries, int k, int max_total,
                      float* out_val, int* out_idx, float* out_thr, int* overflow, void* const* push_val,
                      void* const* push_idx, void* const* push_flag, void* const* push_ready, int n_push,
                      const int* sticky_overflow, const int* wait_ready, int wait_target,
                      const int* const* src_flag, cudaStream_t stream) {
  using namespace afb;
  if (n_queries <= 0) return 0;
  if (n_push < 0 || n_push > 8) {
    set_last_error("afb_topk_select: at most 8 ranks to push to (got %d)", n_push);
    return -1;
  }
  if (n_src < 1 || n_src > kMaxSources) {
    set_last_error("afb_topk_select: between 1 and %d sources (got %d)", kMaxSources, n_src);
    return -1;
  }
  int cap = 2;
  while (cap < max_total) cap <<= 1;
  if (cap > 16384) {
    set_last_error("afb_topk_select: at most 16384 candidates per query fit the shared-memory sort (asked %d)", max_total);
    return -1;
  }
  SelectParams p = {};
  for (int s = 0; s < n_src; ++s) {
    p.vals[s] = vals[s]; p.idxs[s] = idxs[s]; p.counts[s] = counts ? counts[s] : nullptr;
    p.stride[s] = stride[s]; p.fixed_len[s] = fixed_len[s];
    p.src_flag[s] = src_flag ? src_flag[s] : nullptr;
  }
  for (int o = 0; o < n_push; ++o) {
    p.push_val[o] = reinterpret_cast<float*>(push_val[o]);
    p.push_idx[o] = reinterpret_cast<int*>(push_idx[o]);
    p.push_flag[o] = reinterpret_cast<int*>(push_flag[o]);
    p.push_ready[o] = reinterpret_cast<int*>(push_ready[o]);
  }
  p.n_push = n_push; p.sticky_overflow = sticky_overflow; p.wait_ready = wait_ready; p.wait_target = wait_target;
  p.n_src = n_src; p.k = k; p.sort_cap = cap; p.out_val = out_val; p.out_idx = out_idx; p.out_thr = out_thr;
  p.overflow = overflow;
  const int smem = cap * 8;
  AFB_CONFIGURE_KERNEL(topk_select_kernel, 16384 * 8, 256, 0);
  topk_select_kernel<<<n_queries, 256, smem, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_kmeans_accumulate(const void* x, long ldx, const int* assign, float* sums, int* counts, int M, int D, int K,
                          cudaStream_t stream) {
  using namespace afb;
  if (M <= 0) return 0;
  if (D % 4) {
    set_last_error("afb_kmeans_accumulate: dimension must be a multiple of 4");
    return -1;
  }
  const long threads = static_cast<long>(M) * 32;
  kmeans_accumulate_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, assign, sums, counts, M, D, K);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_kmeans_finalize(const float* sums, const int* counts, float* cent_f32, void* cent_bf16, float* cent_sqnorm,
                        float* shift, int K, int D, int normalize, cudaStream_t stream) {
  using namespace afb;
  if (K <= 0) return 0;
  kmeans_finalize_kernel<<<K, 256, 0, stream>>>(sums, counts, cent_f32, reinterpret_cast<__nv_bfloat16*>(cent_bf16),
                                                cent_sqnorm, shift, D, normalize);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_row_sqnorm(const void* x, long ldx, float* out, int M, int D, cudaStream_t stream) {
  using namespace afb;
  if (M <= 0) return 0;
  const long threads = static_cast<long>(M) * 32;
  row_sqnorm_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, out, M, D);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_gather_rows(const void* x, long ldx, const int* idx, void* out, int n, int D, long rows, cudaStream_t stream) {
  using namespace afb;
  if (n <= 0) return 0;
  if (D % 8) {
    set_last_error("afb_gather_rows: dimension must be a multiple of 8");
    return -1;
  }
  gather_rows_kernel<<<n, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, idx,
                                            reinterpret_cast<__nv_bfloat16*>(out), n, D, rows);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_rabitq_estimate(const void* codes, const void* qplanes, const unsigned int* code_counts,
                        const float* centroid_dist, const float* inv_dot, const float* centroid_dot,
                        const float* data_norms, float* dist, float* err, unsigned int* bit_products, int n, int width,
                        int metric, float t1, float t2, float t34, float q_cdist, float q_cdot, float sq_cnorm,
                        float sqrt_dims, float q_norm, cudaStream_t stream) {
  using namespace afb;
  if (n <= 0) return 0;
  RabitqParams p;
  p.codes = reinterpret_cast<const unsigned long long*>(codes);
  p.qplanes = reinterpret_cast<const unsigned long long*>(qplanes);
  p.code_counts = code_counts; p.centroid_dist = centroid_dist; p.inv_dot = inv_dot; p.centroid_dot = centroid_dot;
  p.data_norms = data_norms; p.dist = dist; p.err = err; p.bit_products = bit_products; p.n = n; p.width = width;
  p.metric = metric; p.t1 = t1; p.t2 = t2; p.t34 = t34; p.q_cdist = q_cdist; p.q_cdot = q_cdot; p.sq_cnorm = sq_cnorm;
  p.sqrt_dims = sqrt_dims; p.q_norm = q_norm;
  rabitq_estimate_kernel<<<(n + 255) / 256, 256, static_cast<size_t>(width) * 32, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
