// Paged causal attention with the two softmax variants the tensor-core kernels do not carry:
//   * a learned per-head *sink* logit that joins the softmax denominator without contributing a value
//     (the reference's attention-with-sinks contract: zig/pkg/inference/src/graph/backend_contracts.zig:508-542,
//      CPU implementation zig/pkg/inference/src/ops/native_compute.zig:35108-35160), and
//   * a soft cap on the scaled scores, s <- cap * tanh(s / cap) (Gemma-2 style attention logit capping),
//   * a linear position bias, s <- s + slope[head] * (key position - query position) (ALiBi, BLOOM's only position
//     signal; the reference applies it in its decoder attention, zig/pkg/inference/src/architectures/gpt.zig:4894).
// Each is one extra term per score, but they change the normalisation, so they cannot be applied after the fact to
// the output of a kernel that does not also return its log-sum-exp.
//
// Organisation: one warp per (query token, query head).  Keys are visited in chunks of 128: in the score pass every
// lane scores four keys of the chunk (its own rows of K, 16-byte loads; q sits in shared memory as fp32), the chunk
// maximum is reduced with shuffles and the running (max, sum, accumulator) are rescaled; in the value pass lane l
// owns columns l, l + 32, ... of the accumulator and walks the chunk's V rows, which makes every V read a coalesced
// row read.  D <= 256 (eight accumulator registers per lane).  bf16 caches [num_blocks, page, Hkv, D].
//
// Every block id taken from the table is range-checked; a bad one sets kStatusBadIndex and that key is skipped.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../common/status.cuh"
#include "../common/tmap.cuh"

namespace afb {

constexpr int kSinkWarps = 4;
constexpr int kSinkChunk = 128;

struct SinkAttnParams {
  const __nv_bfloat16* q;
  long q_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;
  const int* token_seq;  // [T] sequence of every query row
  const int* q_starts;   // [B]
  const int* q_lens;     // [B]
  const int* kv_lens;    // [B]
  const float* sinks;    // [Hq] or null
  const float* alibi;    // [Hq] slopes or null
  __nv_bfloat16* out;
  long out_stride;
  int max_blocks, page, num_blocks;
  int T, Hq, Hkv, D, window;
  float scale, softcap;
};

__global__ void __launch_bounds__(kSinkWarps * 32) sink_attn_kernel(const SinkAttnParams p) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = p.D;
  float* q_s = smem + warp * (D + kSinkChunk);  // [D]
  float* s_s = q_s + D;                         // [kSinkChunk] probabilities of the current chunk
  const long row = static_cast<long>(blockIdx.x) * kSinkWarps + warp;
  if (row >= static_cast<long>(p.T) * p.Hq) return;
  const int tok = static_cast<int>(row / p.Hq), head = static_cast<int>(row % p.Hq);
  const int b = p.token_seq[tok];
  const int hk = head / (p.Hq / p.Hkv);
  const int q_len = p.q_lens[b], kv_len = p.kv_lens[b];
  const int qi = tok - p.q_starts[b];
  __nv_bfloat16* orow = p.out + static_cast<long>(tok) * p.out_stride + static_cast<long>(head) * D;
  if (qi < 0 || qi >= q_len || kv_len <= 0) {
    for (int d = lane; d < D; d += 32) orow[d] = __float2bfloat16(0.0f);
    return;
  }
  const int qpos = kv_len - q_len + qi;  // absolute position of this query
  int lo = 0;
  if (p.window > 0 && qpos + 1 > p.window) lo = qpos + 1 - p.window;
  const int hi = qpos + 1;  // keys [lo, hi)
  const float slope = p.alibi ? p.alibi[head] : 0.0f;
  const __nv_bfloat16* qrow = p.q + static_cast<long>(tok) * p.q_stride + static_cast<long>(head) * D;
  for (int d = lane; d < D; d += 32) q_s[d] = __bfloat162float(qrow[d]);
  __syncwarp();

  float m_run = p.sinks ? p.sinks[head] : -INFINITY;  // the sink is a key with logit sinks[head] and no value
  float l_run = p.sinks ? 1.0f : 0.0f;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  const int* table = p.block_tables + static_cast<long>(b) * p.max_blocks;
  const long row_elems = static_cast<long>(p.Hkv) * D;

  for (int c0 = lo; c0 < hi; c0 += kSinkChunk) {
    const int n = min(kSinkChunk, hi - c0);
    // score pass: lane scores keys c0 + lane, + 32, + 64, + 96
    float sc[4];
    float cmax = -INFINITY;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int i = lane + 32 * t;
      float s = -INFINITY;
      if (i < n) {
        const int key = c0 + i;
        const int blk_slot = key / p.page;
        const int blk = blk_slot < p.max_blocks ? table[blk_slot] : -1;
        if (blk < 0 || blk >= p.num_blocks) {
          status_set(kStatusBadIndex);
        } else {
          const __nv_bfloat16* kr =
              p.k_cache + (static_cast<long>(blk) * p.page + key % p.page) * row_elems + static_cast<long>(hk) * D;
          float dot = 0.0f;
          for (int d = 0; d < D; d += 8) {  // D is a multiple of 8 and rows are 16-byte aligned (checked on the host)
            const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(h2[j]);
              dot += f.x * q_s[d + 2 * j] + f.y * q_s[d + 2 * j + 1];
            }
          }
          s = dot * p.scale;
          if (p.softcap > 0.0f) s = p.softcap * tanhf(s / p.softcap);
          s += slope * static_cast<float>(key - qpos);
        }
      }
      sc[t] = s;
      cmax = fmaxf(cmax, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
    const float m_new = fmaxf(m_run, cmax);
    if (m_new == -INFINITY) continue;  // nothing visible yet (every key of the chunk was skipped, no sink)
    const float fix = (m_run == -INFINITY) ? 0.0f : __expf(m_run - m_new);
    float csum = 0.0f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float pr = (sc[t] == -INFINITY) ? 0.0f : __expf(sc[t] - m_new);
      s_s[lane + 32 * t] = pr;
      csum += pr;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) csum += __shfl_xor_sync(0xffffffffu, csum, o);
    l_run = l_run * fix + csum;
    m_run = m_new;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= fix;
    __syncwarp();
    // value pass: lane owns columns lane, lane + 32, ...
    for (int i = 0; i < n; ++i) {
      const float pr = s_s[i];
      if (pr == 0.0f) continue;
      const int key = c0 + i;
      const int blk = table[key / p.page];  // range-checked in the score pass (a bad one has pr == 0)
      const __nv_bfloat16* vr =
          p.v_cache + (static_cast<long>(blk) * p.page + key % p.page) * row_elems + static_cast<long>(hk) * D;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (d < D) acc[j] += pr * __bfloat162float(vr[d]);
      }
    }
    __syncwarp();
  }
  const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int d = lane + 32 * j;
    if (d < D) orow[d] = __float2bfloat16(acc[j] * inv);
  }
}

}  // namespace afb

extern "C" {

// Paged causal attention with optional per-head sink logits (sinks: float [Hq] or null), an optional soft cap on
// the scaled scores (softcap <= 0: none) and optional per-head linear position slopes (alibi: float [Hq] or null).  q [T, Hq, D] bf16 (row stride q_stride), caches
// [num_blocks, page, Hkv, D] bf16, token_seq [T] = the sequence of every query row, out [T, Hq, D] bf16.
int afb_attention_sink(const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_tables,
                       int max_blocks, int page, int num_blocks, const int* token_seq, const int* q_starts,
                       const int* q_lens, const int* kv_lens, const float* sinks, const float* alibi, void* out,
                       long out_stride, int B, int T, int Hq, int Hkv, int D, int window, float scale, float softcap,
                       cudaStream_t stream) {
  using namespace afb;
  if (B <= 0 || T <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0 || D <= 0 || D > 256 || (D & 7)) {
    set_last_error("afb_attention_sink: head_dim must be a multiple of 8 up to 256 and Hq a multiple of Hkv "
                   "(D=%d Hq=%d Hkv=%d)", D, Hq, Hkv);
    return -1;
  }
  if (page <= 0 || max_blocks <= 0 || num_blocks <= 0 || !(scale > 0.0f)) {
    set_last_error("afb_attention_sink: bad page / table / scale arguments");
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15)) {
    set_last_error("afb_attention_sink: caches must be 16-byte aligned");
    return -1;
  }
  SinkAttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride = q_stride;
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache); p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = block_tables; p.token_seq = token_seq; p.q_starts = q_starts; p.q_lens = q_lens;
  p.kv_lens = kv_lens; p.sinks = sinks; p.alibi = alibi; p.out = static_cast<__nv_bfloat16*>(out); p.out_stride = out_stride;
  p.max_blocks = max_blocks; p.page = page; p.num_blocks = num_blocks;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.window = window; p.scale = scale; p.softcap = softcap;
  const long rows = static_cast<long>(T) * Hq;
  const int smem = kSinkWarps * (D + kSinkChunk) * static_cast<int>(sizeof(float));
  sink_attn_kernel<<<static_cast<unsigned>((rows + kSinkWarps - 1) / kSinkWarps), kSinkWarps * 32, smem, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
