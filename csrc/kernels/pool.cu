// Sequence pooling fused with L2 normalisation: masked mean / CLS / masked max / last active token over a
// packed (varlen) or padded batch of bf16 hidden states, fp32 output.  One CTA per document; each thread owns
// two adjacent hidden columns so token rows are read with coalesced 4-byte accesses.
//
// Semantics follow the reference's pool3D + l2Normalize (zig/pkg/inference/src/pipelines/embedding.zig:322-390,
// zig/lib/linalg/src/mod.zig:298,312): mean over tokens whose mask is > 0, zero vector for an empty mask.
// Also holds the ColBERT late-interaction MaxSim scorer (zig/pkg/inference/src/pipelines/reranking.zig:354-383)
// and the SPLADE log(1+relu) max-pool (zig/pkg/inference/src/pipelines/sparse_embedding.zig:19-21).
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

struct PoolParams {
  const __nv_bfloat16* h;  // token rows, pitch H
  const int* starts;       // [B] first token row of each document
  const int* lens;         // [B] number of token rows
  const int* mask;         // optional per-token-row mask (>0 = active), indexed by token row
  float* out;              // [B, H]
  int B, H;
  int mode;                // 0 mean, 1 cls, 2 max, 3 last
  int normalize;
  // Data-parallel gather fused into the producer: the finished row is also stored into every rank's gathered
  // buffer (peer stores over NVLink) at row `row_offset + b`, and each rank's arrival counter is bumped once per
  // CTA, so the all-gather of per-GPU embedding outputs needs no separate collective.
  float* peer_out[8];
  int* peer_ready[8];
  int n_peers, row_offset;
};

__global__ void pool_kernel(PoolParams p) {
  __shared__ float red[32];
  // Once a cross-GPU wait of this rank has timed out (or the host poisoned the waits) the hand-off counters of
  // the ranks no longer agree: push nothing more, so that rows of a later step can never complete a slower
  // peer's older arrival target.  The peers' own waits then run out and report.
  if (p.n_peers && (status_peek() & kStatusPeerFlagTimeout)) p.n_peers = 0;
  const int b = blockIdx.x;
  const int start = p.starts[b], len = p.lens[b];
  const int H = p.H;
  int last = -1, count = 0;
  if (p.mode == 3 || p.mode == 0) {
    // Active-token count / last active row are the same for every thread; computed redundantly (len <= a few
    // thousand, reads hit L1).
    if (p.mask) {
      for (int t = 0; t < len; ++t)
        if (p.mask[start + t] > 0) { last = t; ++count; }
    } else {
      last = len - 1; count = len;
    }
  }
  float ss = 0.0f;
  for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
    float a0 = 0.0f, a1 = 0.0f;
    if (p.mode == 1) {
      if (len > 0) {
        float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.h + static_cast<size_t>(start) * H + c));
        a0 = v.x; a1 = v.y;
      }
    } else if (p.mode == 3) {
      if (last >= 0) {
        float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.h + static_cast<size_t>(start + last) * H + c));
        a0 = v.x; a1 = v.y;
      }
    } else {
      const bool is_max = p.mode == 2;
      bool any = false;
      if (is_max) { a0 = -3.0e38f; a1 = -3.0e38f; }
      for (int t = 0; t < len; ++t) {
        if (p.mask && p.mask[start + t] <= 0) continue;
        float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.h + static_cast<size_t>(start + t) * H + c));
        if (is_max) { a0 = fmaxf(a0, v.x); a1 = fmaxf(a1, v.y); }
        else { a0 += v.x; a1 += v.y; }
        any = true;
      }
      if (!any) { a0 = 0.0f; a1 = 0.0f; }
      else if (!is_max) { const float inv = 1.0f / static_cast<float>(count); a0 *= inv; a1 *= inv; }
    }
    p.out[static_cast<size_t>(b) * H + c] = a0;
    p.out[static_cast<size_t>(b) * H + c + 1] = a1;
    if (!p.normalize) {
      for (int o = 0; o < p.n_peers; ++o)
        *reinterpret_cast<float2*>(p.peer_out[o] + static_cast<size_t>(p.row_offset + b) * H + c) = make_float2(a0, a1);
    }
    ss += a0 * a0 + a1 * a1;
  }
  if (!p.normalize) {
    if (p.n_peers) {
      __syncthreads();
      if (threadIdx.x == 0)
        for (int o = 0; o < p.n_peers; ++o)
          asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(p.peer_ready[o]) : "memory");
    }
    return;
  }
  ss = warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.0f;
  t = warp_sum(t);
  const float inv = t > 0.0f ? rsqrtf(t) : 0.0f;
  for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
    const float a0 = p.out[static_cast<size_t>(b) * H + c] * inv, a1 = p.out[static_cast<size_t>(b) * H + c + 1] * inv;
    p.out[static_cast<size_t>(b) * H + c] = a0;
    p.out[static_cast<size_t>(b) * H + c + 1] = a1;
    for (int o = 0; o < p.n_peers; ++o)
      *reinterpret_cast<float2*>(p.peer_out[o] + static_cast<size_t>(p.row_offset + b) * H + c) = make_float2(a0, a1);
  }
  if (p.n_peers) {
    __syncthreads();
    if (threadIdx.x == 0)
      for (int o = 0; o < p.n_peers; ++o)
        asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(p.peer_ready[o]) : "memory");
  }
}

// Late-interaction MaxSim: score(d) = sum over query tokens of max over document tokens of cosine(q, t).
// Token embeddings arrive L2-normalised or not; norms are applied here.  One CTA per document, one warp per
// query token (round-robin), lanes stride the embedding dimension.
__global__ void maxsim_kernel(const __nv_bfloat16* q, int nq, const __nv_bfloat16* d, const int* starts,
                              const int* lens, float* out, int D) {
  extern __shared__ float sq[];  // [nq, D] query in fp32 (normalised)
  __shared__ float red[32];
  const int doc = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int i = warp; i < nq; i += nw) {
    float ss = 0.0f;
    for (int c = lane; c < D; c += 32) {
      const float v = __bfloat162float(q[static_cast<size_t>(i) * D + c]);
      sq[i * D + c] = v;
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = ss > 0.0f ? rsqrtf(ss) : 0.0f;
    for (int c = lane; c < D; c += 32) sq[i * D + c] *= inv;
  }
  __syncthreads();
  const int start = starts[doc], len = lens[doc];
  float total = 0.0f;
  for (int i = warp; i < nq; i += nw) {
    float best = -3.0e38f;
    for (int t = 0; t < len; ++t) {
      const __nv_bfloat16* row = d + static_cast<size_t>(start + t) * D;
      float dot = 0.0f, nn = 0.0f;
      for (int c = lane; c < D; c += 32) {
        const float v = __bfloat162float(row[c]);
        dot += v * sq[i * D + c];
        nn += v * v;
      }
      dot = warp_sum(dot);
      nn = warp_sum(nn);
      const float s = nn > 0.0f ? dot * rsqrtf(nn) : 0.0f;
      best = fmaxf(best, s);
    }
    if (len > 0) total += best;
  }
  if (lane == 0) red[warp] = total;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) out[doc] = t;
  }
}

// SPLADE: out[b, v] = max over active tokens of log(1 + relu(logits[t, v])).
__global__ void splade_pool_kernel(const __nv_bfloat16* logits, const int* starts, const int* lens, float* out,
                                   int V) {
  const int b = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= V) return;
  const int start = starts[b], len = lens[b];
  float m = 0.0f;
  for (int t = 0; t < len; ++t) {
    const float x = __bfloat162float(logits[static_cast<size_t>(start + t) * V + v]);
    m = fmaxf(m, x > 0.0f ? log1pf(x) : 0.0f);
  }
  out[static_cast<size_t>(b) * V + v] = m;
}

// Consumer side of a push-style hand-off: returns once `*counter` (bumped by other GPUs with red.release.sys after
// their stores into this GPU's memory) has reached `target`, or records kStatusPeerFlagTimeout after the
// cross-GPU wait limit and returns anyway.  Kernels launched after it on the stream see the pushed data.
__global__ void peer_counter_wait_kernel(const int* counter, int target) {
  if (threadIdx.x == 0) peer_wait_counter(counter, target);
}

}  // namespace afb

extern "C" {

// Stream-ordered bounded wait for an arrival counter in this GPU's memory that peers increment (monotonic,
// wrap-safe compare).  On expiry the status word is set; the call itself always returns 0 once launched.
int afb_peer_counter_wait(const int* counter, int target, cudaStream_t stream) {
  afb::peer_counter_wait_kernel<<<1, 32, 0, stream>>>(counter, target);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_pool_gather(const void* h, const int* starts, const int* lens, const int* mask, float* out, int B, int H,
                    int mode, int normalize, void* const* peer_out, void* const* peer_ready, int n_peers,
                    int row_offset, cudaStream_t stream);

int afb_pool(const void* h, const int* starts, const int* lens, const int* mask, float* out, int B, int H, int mode,
             int normalize, cudaStream_t stream) {
  return afb_pool_gather(h, starts, lens, mask, out, B, H, mode, normalize, nullptr, nullptr, 0, 0, stream);
}

// Pooling whose output rows are also pushed into every rank's gathered buffer (data-parallel embedding gather).
int afb_pool_gather(const void* h, const int* starts, const int* lens, const int* mask, float* out, int B, int H,
                    int mode, int normalize, void* const* peer_out, void* const* peer_ready, int n_peers,
                    int row_offset, cudaStream_t stream) {
  using namespace afb;
  if (B <= 0) return 0;
  if (H % 2 != 0) {
    set_last_error("afb_pool: hidden size must be even (got %d)", H);
    return -1;
  }
  PoolParams p = {};
  if (n_peers < 0 || n_peers > 8) {
    set_last_error("afb_pool_gather: at most 8 ranks");
    return -1;
  }
  p.n_peers = n_peers; p.row_offset = row_offset;
  for (int o = 0; o < n_peers; ++o) {
    p.peer_out[o] = reinterpret_cast<float*>(peer_out[o]);
    p.peer_ready[o] = reinterpret_cast<int*>(peer_ready[o]);
  }
  p.h = reinterpret_cast<const __nv_bfloat16*>(h);
  p.starts = starts; p.lens = lens; p.mask = mask; p.out = out; p.B = B; p.H = H; p.mode = mode;
  p.normalize = normalize;
  int threads = ((H / 2) + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  pool_kernel<<<B, threads, 0, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_maxsim(const void* q, int nq, const void* d, const int* starts, const int* lens, float* out, int n_docs,
               int D, cudaStream_t stream) {
  using namespace afb;
  if (n_docs <= 0) return 0;
  const size_t smem = static_cast<size_t>(nq) * D * 4;
  if (smem > 200 * 1024) {
    set_last_error("afb_maxsim: query of %d tokens x %d dims does not fit in shared memory", nq, D);
    return -1;
  }
  AFB_CONFIGURE_KERNEL(maxsim_kernel, 200 * 1024, 256, 0);
  maxsim_kernel<<<n_docs, 256, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(q), nq,
                                               reinterpret_cast<const __nv_bfloat16*>(d), starts, lens, out, D);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_splade_pool(const void* logits, const int* starts, const int* lens, float* out, int B, int V,
                    cudaStream_t stream) {
  using namespace afb;
  if (B <= 0) return 0;
  dim3 grid((V + 255) / 256, B);
  splade_pool_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), starts, lens, out,
                                               V);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
