// Token selection on the device, so logits never travel to the host:
//   * argmax over the vocabulary (greedy decode, speculative verify),
//   * repetition / frequency / presence penalties from a per-sequence token-count table,
//   * temperature -> softmax -> top-k -> top-p -> min-p -> sample, with the thresholds found by radix
//     selection over an order-preserving integer key (4 passes of 256-bin histograms) instead of a sort,
//   * speculative-decoding verify / accept.
//
// Order of operations and the min-p rule (drop p < min_p * p_max) follow the reference's host sampler
// (zig/pkg/inference/src/pipelines/generation.zig:5062-5158); verify/accept follows
// acceptVerifiedDraftTokens (same file, :3228-3340): tokens are accepted while the draft equals the target's
// choice; the first mismatch is replaced by the target's token, and if all match the target's extra position
// supplies a bonus token.
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

__device__ __forceinline__ uint32_t float_key(float f) {
  // Monotonic map float -> uint32 (larger float, larger key).
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(p[i]);
}

// ---------------------------------------------------------------------------------------------------------
// argmax: one CTA per row.  Ties resolve to the lowest index.  `row_stride` lets the caller pick rows out of a
// larger logits buffer; vocab_offset is added to the result (vocabulary-sharded heads).
// ---------------------------------------------------------------------------------------------------------
// Cross-GPU merge of a vocabulary-sharded arg-max (tensor-parallel LM head), fused into the same kernel: each
// rank packs its best (value, global index) into one 64-bit key (order-preserving value bits high, inverted index
// low, so the larger key is the better candidate and ties go to the lower index), stores it into slot
// [my_rank][row] of every rank (8-byte peer stores), then polls its own world slots until all keys have landed,
// takes the maximum and zeroes the slots again (0 is never a valid key).  No flags, no fences, no collective
// library call.  A rank can only reach this kernel again after a cross-rank hand-off of the next step, which the
// slower ranks enter after their own merge, so one set of slots suffices.
struct ArgmaxTp {
  unsigned long long* peer_slots[8];  // rank o's [world][max_rows] key slots
  int world, my_rank, max_rows;
};

template <typename T>
__global__ void argmax_kernel(const T* logits, long row_stride, int V, int* out_idx, float* out_val,
                              int vocab_offset, ArgmaxTp tp) {
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const int row = blockIdx.x;
  griddep_launch();
  griddep_wait();
  const T* lp = logits + static_cast<size_t>(row) * row_stride;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  constexpr int VEC = 16 / sizeof(T);
  if ((reinterpret_cast<uintptr_t>(lp) & 15) == 0) {
    // 16-byte loads; within a thread indices ascend, so a strict > keeps the lowest index on ties.
    const int nvec = V / VEC;
    for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
      const uint4 u = *reinterpret_cast<const uint4*>(lp + static_cast<size_t>(j) * VEC);
      float v[VEC];
      if constexpr (sizeof(T) == 2) {
        const float2 a = unpack_bf16x2(u.x), b2 = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        v[0] = a.x; v[1] = a.y; v[2] = b2.x; v[3] = b2.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
      } else {
        v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        if (v[e] > best) { best = v[e]; bi = j * VEC + e; }
    }
    for (int i = nvec * VEC + threadIdx.x; i < V; i += blockDim.x) {
      const float v = ld_logit<T>(lp, i);
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = ld_logit<T>(lp, i);
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? sval[lane] : -INFINITY;
    bi = lane < nw ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (tp.world > 0) {
      // All lanes hold the local winner; lane o publishes to rank o, then lane s polls slot s.
      const unsigned gidx = static_cast<unsigned>(bi + vocab_offset);
      const unsigned long long key = (static_cast<unsigned long long>(float_key(best)) << 32) | (0xFFFFFFFFu - gidx);
      if (lane < tp.world) {
        unsigned long long* dst = tp.peer_slots[lane] + static_cast<size_t>(tp.my_rank) * tp.max_rows + row;
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(key) : "memory");
      }
      unsigned long long got = 0;
      if (lane < tp.world) {
        unsigned long long* src = tp.peer_slots[tp.my_rank] + static_cast<size_t>(lane) * tp.max_rows + row;
        PeerDeadline dl;
        for (uint32_t it = 0; it < AFB_SPIN_LIMIT; ++it) {
          asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
          if (got != 0ull || dl.expired()) break;
          if (it > 16) __nanosleep(20);
        }
        if (got == 0ull) status_set(kStatusPeerFlagTimeout);
        else *src = 0ull;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, got, o);
        got = other > got ? other : got;
      }
      if (lane == 0) {
        out_idx[row] = static_cast<int>(0xFFFFFFFFu - static_cast<unsigned>(got & 0xFFFFFFFFull));
        if (out_val) out_val[row] = best;
      }
    } else if (lane == 0) {
      out_idx[row] = bi + vocab_offset;
      if (out_val) out_val[row] = best;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Penalties.  counts[b, v] = occurrences of token v in sequence b's context so far (uint16, saturating).
// ---------------------------------------------------------------------------------------------------------
__global__ void count_tokens_kernel(unsigned short* counts, const int* tokens, const int* row_of_token, int n,
                                    int V) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int tok = tokens[i];
  if (tok < 0 || tok >= V) { status_set(kStatusBadIndex); return; }
  unsigned short* c = counts + static_cast<size_t>(row_of_token[i]) * V + tok;
  // 16-bit saturating increment through a 32-bit CAS on the containing word.
  unsigned int* w = reinterpret_cast<unsigned int*>(reinterpret_cast<uintptr_t>(c) & ~uintptr_t(3));
  const int shift = (reinterpret_cast<uintptr_t>(c) & 2) ? 16 : 0;
  unsigned int old = *w, assumed;
  do {
    assumed = old;
    const unsigned int cur = (assumed >> shift) & 0xFFFFu;
    if (cur == 0xFFFFu) break;
    const unsigned int nv = (assumed & ~(0xFFFFu << shift)) | ((cur + 1) << shift);
    old = atomicCAS(w, assumed, nv);
  } while (old != assumed);
}

template <typename T>
__global__ void penalties_kernel(const T* logits, long row_stride, float* out, const unsigned short* counts,
                                 const float* rep, const float* freq, const float* pres, int V) {
  const int row = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= V) return;
  float x = ld_logit<T>(logits + static_cast<size_t>(row) * row_stride, v);
  const unsigned short c = counts ? counts[static_cast<size_t>(row) * V + v] : 0;
  if (c > 0) {
    const float r = rep ? rep[row] : 1.0f;
    if (r != 1.0f) x = x > 0.0f ? x / r : x * r;
    if (freq) x -= freq[row] * static_cast<float>(c);
    if (pres) x -= pres[row];
  }
  out[static_cast<size_t>(row) * V + v] = x;
}

// ---------------------------------------------------------------------------------------------------------
// Sampler: one CTA (1024 threads) per row over fp32 logits.
// ---------------------------------------------------------------------------------------------------------
struct SampleParams {
  const float* logits;  // [B, V]
  int V;
  const float* temperature;  // [B]; <= 0 means greedy
  const int* top_k;          // [B]; <= 0 disables
  const float* top_p;        // [B]; >= 1 disables
  const float* min_p;        // [B]; <= 0 disables
  const float* uniform;      // [B] in [0, 1)
  int* out;                  // [B]
  float* out_prob;           // [B] optional: probability of the chosen token under the filtered distribution
};

__device__ float block_reduce_sum_1024(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[lane];
  t = warp_sum(t);
  return t;
}
__device__ float block_reduce_max_1024(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[lane];
  t = warp_max(t);
  return t;
}

// Finds the largest key K such that weight(key >= K) >= target, where weight is a count (BY_MASS = false) or
// probability mass (BY_MASS = true), among elements with key >= floor_key.  4 passes over the row.
template <bool BY_MASS>
__device__ uint32_t radix_threshold(const float* lp, int V, float m, float inv_t, uint32_t floor_key, float target,
                                    float* hist /* [256] shared */) {
  uint32_t prefix = 0;
  float above = 0.0f;  // weight of keys strictly above the current prefix bucket range
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0.0f;
    __syncthreads();
    const uint32_t mask_hi = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = lp[i];
      const uint32_t key = float_key(x);
      if (key < floor_key) continue;
      if ((key & mask_hi) != (prefix & mask_hi)) continue;
      const float w = BY_MASS ? __expf((x - m) * inv_t) : 1.0f;
      atomicAdd(&hist[(key >> shift) & 0xFF], w);
    }
    __syncthreads();
    // Every thread walks the 256 bins from the top (cheap, avoids another reduction).
    float acc = above;
    int bin = 255;
    for (; bin > 0; --bin) {
      if (acc + hist[bin] >= target) break;
      acc += hist[bin];
    }
    above = acc;
    prefix |= static_cast<uint32_t>(bin) << shift;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(1024) sample_kernel(SampleParams p) {
  __shared__ float red[32];
  __shared__ float hist[256];
  __shared__ float scan[1024];
  __shared__ int s_choice;
  const int row = blockIdx.x;
  const int V = p.V;
  const float* lp = p.logits + static_cast<size_t>(row) * V;
  const float temp = p.temperature ? p.temperature[row] : 1.0f;

  // max (also the greedy answer)
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = lp[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  const float m = block_reduce_max_1024(best, red);
  if (temp <= 0.0f) {
    // greedy: lowest index among the maxima
    int cand = (best == m) ? bi : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int sidx[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sidx[warp] = cand;
    __syncthreads();
    if (warp == 0) {
      cand = sidx[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
      if (lane == 0) {
        p.out[row] = cand;
        if (p.out_prob) p.out_prob[row] = 1.0f;
      }
    }
    return;
  }
  const float inv_t = 1.0f / temp;

  // top-k threshold key
  uint32_t floor_key = 0;
  const int k = p.top_k ? p.top_k[row] : 0;
  if (k > 0 && k < V) floor_key = radix_threshold<false>(lp, V, m, inv_t, 0u, static_cast<float>(k), hist);

  // mass after top-k
  float part = 0.0f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = lp[i];
    if (float_key(x) >= floor_key) part += __expf((x - m) * inv_t);
  }
  float total = block_reduce_sum_1024(part, red);

  // top-p threshold key (smallest set of largest tokens whose mass reaches top_p * total)
  const float tp = p.top_p ? p.top_p[row] : 1.0f;
  if (tp < 1.0f) {
    const uint32_t kp = radix_threshold<true>(lp, V, m, inv_t, floor_key, tp * total, hist);
    floor_key = max(floor_key, kp);
  }
  // min-p: p_i / p_max = exp((x - m)/T) >= min_p
  const float mp = p.min_p ? p.min_p[row] : 0.0f;
  const float min_ratio = mp > 0.0f ? mp : 0.0f;

  // Final pass: contiguous chunk per thread, block scan, pick.
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
  float mine = 0.0f;
  for (int i = lo; i < hi; ++i) {
    const float x = lp[i];
    const float w = __expf((x - m) * inv_t);
    if (float_key(x) >= floor_key && w >= min_ratio) mine += w;
  }
  scan[threadIdx.x] = mine;
  __syncthreads();
  // Hillis-Steele inclusive scan over 1024 entries.
  for (int off = 1; off < 1024; off <<= 1) {
    const float add = threadIdx.x >= off ? scan[threadIdx.x - off] : 0.0f;
    __syncthreads();
    scan[threadIdx.x] += add;
    __syncthreads();
  }
  total = scan[1023];
  const float u = fminf(fmaxf(p.uniform[row], 0.0f), 0.99999994f) * total;
  if (threadIdx.x == 0) s_choice = -1;
  __syncthreads();
  const float before = scan[threadIdx.x] - mine;
  if (mine > 0.0f && u >= before && u < scan[threadIdx.x]) {
    float acc = before;
    int pick = -1;
    float pw = 0.0f;
    for (int i = lo; i < hi; ++i) {
      const float x = lp[i];
      const float w = __expf((x - m) * inv_t);
      if (float_key(x) >= floor_key && w >= min_ratio) {
        pick = i; pw = w;
        acc += w;
        if (u < acc) break;
      }
    }
    s_choice = pick;
    if (p.out_prob) p.out_prob[row] = pw / total;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_choice < 0) {
      // Rounding left u on a boundary no thread claimed: fall back to the arg-max, which is always kept.
      // (best/bi of thread 0 is only its own slice; recompute cheaply.)
      int cand = 0; float bv = -INFINITY;
      for (int i = 0; i < V; ++i) { const float x = lp[i]; if (x > bv) { bv = x; cand = i; } }
      s_choice = cand;
      if (p.out_prob) p.out_prob[row] = 1.0f / total;
    }
    p.out[row] = s_choice;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Speculative verify / accept: draft [B, K], target [B, K+1] -> n_matched [B], next_token [B].
// ---------------------------------------------------------------------------------------------------------
__global__ void spec_verify_kernel(const int* draft, const int* target, int B, int K, int* n_matched, int* next_tok) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int n = 0;
  while (n < K && draft[b * K + n] == target[b * (K + 1) + n]) ++n;
  n_matched[b] = n;
  next_tok[b] = target[b * (K + 1) + n];
}

}  // namespace afb

extern "C" {

int afb_argmax_tp(const void* logits, int is_f32, long row_stride, int rows, int V, int* out_idx, float* out_val,
                  int vocab_offset, void* const* peer_slots, int world, int my_rank, int max_rows,
                  cudaStream_t stream);

int afb_argmax(const void* logits, int is_f32, long row_stride, int rows, int V, int* out_idx, float* out_val,
               int vocab_offset, cudaStream_t stream) {
  return afb_argmax_tp(logits, is_f32, row_stride, rows, V, out_idx, out_val, vocab_offset, nullptr, 0, 0, 0, stream);
}

// Arg-max over a vocabulary shard merged across `world` ranks inside the kernel (see ArgmaxTp): peer_slots[o] is
// rank o's zero-initialised [world][max_rows] array of 64-bit keys.  world = 0: local arg-max only.
int afb_argmax_tp(const void* logits, int is_f32, long row_stride, int rows, int V, int* out_idx, float* out_val,
                  int vocab_offset, void* const* peer_slots, int world, int my_rank, int max_rows,
                  cudaStream_t stream) {
  using namespace afb;
  if (rows <= 0) return 0;
  ArgmaxTp tp = {};
  if (world > 0) {
    if (world > 8 || rows > max_rows || !peer_slots) {
      set_last_error("afb_argmax_tp: at most 8 ranks and rows <= max_rows (rows=%d max_rows=%d)", rows, max_rows);
      return -1;
    }
    tp.world = world; tp.my_rank = my_rank; tp.max_rows = max_rows;
    for (int o = 0; o < world; ++o) tp.peer_slots[o] = reinterpret_cast<unsigned long long*>(peer_slots[o]);
  }
  if (is_f32)
    AFB_CHECK_CUDA(launch_pdl(argmax_kernel<float>, dim3(rows), dim3(1024), 0, stream,
                              reinterpret_cast<const float*>(logits), row_stride, V, out_idx, out_val, vocab_offset,
                              tp));
  else
    AFB_CHECK_CUDA(launch_pdl(argmax_kernel<__nv_bfloat16>, dim3(rows), dim3(1024), 0, stream,
                              reinterpret_cast<const __nv_bfloat16*>(logits), row_stride, V, out_idx, out_val,
                              vocab_offset, tp));
  return 0;
}

int afb_count_tokens(void* counts, const int* tokens, const int* row_of_token, int n, int V, cudaStream_t stream) {
  using namespace afb;
  if (n <= 0) return 0;
  if (V & 1) {
    set_last_error("afb_count_tokens: vocabulary size must be even");
    return -1;
  }
  count_tokens_kernel<<<(n + 255) / 256, 256, 0, stream>>>(reinterpret_cast<unsigned short*>(counts), tokens,
                                                           row_of_token, n, V);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_penalties(const void* logits, int is_f32, long row_stride, float* out, const void* counts, const float* rep,
                  const float* freq, const float* pres, int rows, int V, cudaStream_t stream) {
  using namespace afb;
  if (rows <= 0) return 0;
  dim3 grid((V + 255) / 256, rows);
  if (is_f32)
    penalties_kernel<float><<<grid, 256, 0, stream>>>(reinterpret_cast<const float*>(logits), row_stride, out,
                                                      reinterpret_cast<const unsigned short*>(counts), rep, freq,
                                                      pres, V);
  else
    penalties_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits),
                                                              row_stride, out,
                                                              reinterpret_cast<const unsigned short*>(counts), rep,
                                                              freq, pres, V);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_sample(const float* logits, int rows, int V, const float* temperature, const int* top_k, const float* top_p,
               const float* min_p, const float* uniform, int* out, float* out_prob, cudaStream_t stream) {
  using namespace afb;
  if (rows <= 0) return 0;
  SampleParams p;
  p.logits = logits; p.V = V; p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.min_p = min_p;
  p.uniform = uniform; p.out = out; p.out_prob = out_prob;
  sample_kernel<<<rows, 1024, 0, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_spec_verify(const int* draft, const int* target, int B, int K, int* n_matched, int* next_tok,
                    cudaStream_t stream) {
  using namespace afb;
  if (B <= 0) return 0;
  spec_verify_kernel<<<(B + 127) / 128, 128, 0, stream>>>(draft, target, B, K, n_matched, next_tok);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
