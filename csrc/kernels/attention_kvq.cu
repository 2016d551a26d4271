// Decode attention over a paged KV cache whose rows are stored in a quantised codec (fp8, int8 per head, int4
// group 32, polar4, turbo3; bf16 for completeness): keys are scored straight from their codes and values are
// dequantised as they are read, so the cache is never expanded in memory.
//
// The reference does this on the CPU and in Metal / WGSL shaders
// (zig/pkg/inference/src/ops/native_compute.zig:35200-35240, web/shaders/gqa_cached_attention_{polar4,turbo3}.wgsl);
// it has no CUDA version.  Row formats and every per-element decode are in csrc/common/kvq_elem.h, which the host
// codec library compiles too, so the arithmetic below is the same code that the CPU tests check.
//
// Work split: one CTA per (sequence, KV head), four warps; a warp takes every fourth key, a lane owns the head
// dimensions d = lane, lane + 32, ...; the G = Hq / Hkv query rows that share the KV head are processed together
// (the key is decoded once for all of them).  Each warp keeps its own running max / sum / accumulator (online
// softmax) and the four are merged through shared memory at the end.  For turbo3 the 32 residual projections of
// each query row are computed once per CTA, and lane p contributes projection p's sign term to the score.
//
// All cache accesses are byte loads (no alignment requirement); block ids from the table are range-checked and a
// bad one records kStatusBadIndex and skips the key instead of reading it.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../common/kvq_elem.h"
#include "../common/status.cuh"
#include "../common/tmap.cuh"

namespace afb {

constexpr int kKvqWarps = 4;
constexpr int kKvqMaxG = 8;

struct KvqParams {
  const __nv_bfloat16* q;   // [B, Hq, D], row stride q_stride elements
  long q_stride;
  const uint8_t* k_cache;   // [num_blocks, page] rows of k_row_bytes
  const uint8_t* v_cache;   // [num_blocks, page] rows of v_row_bytes
  const int* block_tables;  // [B, max_blocks]
  const int* kv_lens;       // [B]
  __nv_bfloat16* out;       // [B, Hq, D], row stride out_stride
  long out_stride;
  long k_row_bytes, v_row_bytes;
  int max_blocks, page, num_blocks;
  int Hq, Hkv, D, G, codec, window;
  float scale, k_scale, v_scale;
};

template <int DP>  // DP = ceil(D / 32): head dimensions per lane
__global__ void __launch_bounds__(kKvqWarps * 32) kvq_decode_attn_kernel(const KvqParams p) {
  extern __shared__ float smem[];
  const int hk = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = p.D, G = p.G;
  float* q_s = smem;                                   // [G][D]
  float* pq_s = q_s + G * D;                           // [G][32]
  float* m_s = pq_s + G * kvq::kTurbo3SketchBits;      // [warps][G]
  float* l_s = m_s + kKvqWarps * G;                    // [warps][G]
  float* acc_s = l_s + kKvqWarps * G;                  // [warps][G][D]

  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    q_s[i] = __bfloat162float(p.q[static_cast<long>(b) * p.q_stride + static_cast<long>(hk * G + g) * D + d]);
  }
  __syncthreads();
  if (p.codec == kvq::kTurbo3) {
    for (int i = threadIdx.x; i < G * kvq::kTurbo3SketchBits; i += blockDim.x) {
      const int g = i / kvq::kTurbo3SketchBits, pr = i % kvq::kTurbo3SketchBits;
      float acc = 0.0f;
      for (int d = 0; d < D; ++d) acc += kvq::random_sign(hk, pr, d) * q_s[g * D + d];
      pq_s[i] = acc;
    }
  }
  __syncthreads();

  const int kv_len = min(p.kv_lens[b], p.max_blocks * p.page);
  const int t0 = p.window > 0 ? max(0, kv_len - p.window) : 0;
  float m[kKvqMaxG], l[kKvqMaxG], acc[kKvqMaxG][DP];
#pragma unroll
  for (int g = 0; g < kKvqMaxG; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.0f;
#pragma unroll
    for (int i = 0; i < DP; ++i) acc[g][i] = 0.0f;
  }
  const float sc = p.scale * p.k_scale;
  for (int t = t0 + warp; t < kv_len; t += kKvqWarps) {
    const int blk = p.block_tables[static_cast<long>(b) * p.max_blocks + t / p.page];
    if (blk < 0 || blk >= p.num_blocks) {
      if (lane == 0) status_set(kStatusBadIndex);
      continue;
    }
    const long row = static_cast<long>(blk) * p.page + t % p.page;
    const uint8_t* kr = p.k_cache + row * p.k_row_bytes;
    const uint8_t* vr = p.v_cache + row * p.v_row_bytes;
    float kd[DP], vd[DP];
#pragma unroll
    for (int i = 0; i < DP; ++i) {
      const int d = lane + 32 * i;
      kd[i] = d < D ? kvq::key_elem(p.codec, kr, p.Hkv, D, hk, d) : 0.0f;
      vd[i] = d < D ? kvq::value_elem(p.codec, vr, p.Hkv, D, hk, d) : 0.0f;
    }
    const bool sk_bit = p.codec == kvq::kTurbo3 ? kvq::turbo3_sketch_bit(kr, p.Hkv, D, hk, lane) : false;
#pragma unroll
    for (int g = 0; g < kKvqMaxG; ++g) {
      if (g < G) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < DP; ++i) {
          const int d = lane + 32 * i;
          if (d < D) s += q_s[g * D + d] * kd[i];
        }
        if (p.codec == kvq::kTurbo3) {
          const float pv = pq_s[g * kvq::kTurbo3SketchBits + lane];
          s += (kvq::kTurbo3ResidualScale / kvq::kTurbo3SketchBits) * (sk_bit ? pv : -pv);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s *= sc;
        const float m_new = fmaxf(m[g], s);
        const float alpha = __expf(m[g] - m_new), pr = __expf(s - m_new);
        l[g] = l[g] * alpha + pr;
        m[g] = m_new;
#pragma unroll
        for (int i = 0; i < DP; ++i) acc[g][i] = acc[g][i] * alpha + pr * vd[i];
      }
    }
  }

  // merge the four warps' partial softmax states
#pragma unroll
  for (int g = 0; g < kKvqMaxG; ++g) {
    if (g < G) {
      if (lane == 0) {
        m_s[warp * G + g] = m[g];
        l_s[warp * G + g] = l[g];
      }
#pragma unroll
      for (int i = 0; i < DP; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc_s[(warp * G + g) * D + d] = acc[g][i];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
    for (int w = 0; w < kKvqWarps; ++w) mm = fmaxf(mm, m_s[w * G + g]);
    float num = 0.0f, den = 0.0f;
    if (mm > -INFINITY) {
      for (int w = 0; w < kKvqWarps; ++w) {
        const float f = __expf(m_s[w * G + g] - mm);  // a warp that saw no key has m = -inf -> factor 0
        num += f * acc_s[(w * G + g) * D + d];
        den += f * l_s[w * G + g];
      }
    }
    p.out[static_cast<long>(b) * p.out_stride + static_cast<long>(hk * G + g) * D + d] =
        __float2bfloat16(den > 0.0f ? num * p.v_scale / den : 0.0f);
  }
}

// Expands cache rows to bf16: out[i, h, d] = element (h, d) of code row row_idx[i], times `scale`.  One CTA per
// row; used to hand a prefill chunk's keys and values to the tensor-core attention kernels (which read bf16) while
// the cache itself stays in its codec.  turbo3 keys expand to their 3-bit base values (the residual sketch only
// enters direct code scoring).  Row ids are range-checked; a bad one records kStatusBadIndex and writes zeros.
__global__ void kvq_expand_rows_kernel(const uint8_t* cache, long row_bytes, const int* row_idx, __nv_bfloat16* out,
                                       int heads, int D, int codec, int is_value, float scale, long num_rows) {
  const long i = blockIdx.x;
  const long row = row_idx[i];
  const int n = heads * D;
  __nv_bfloat16* dst = out + i * n;
  if (row < 0 || row >= num_rows) {
    if (threadIdx.x == 0) status_set(kStatusBadIndex);
    for (int e = threadIdx.x; e < n; e += blockDim.x) dst[e] = __float2bfloat16(0.0f);
    return;
  }
  const uint8_t* src = cache + row * row_bytes;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int h = e / D, d = e % D;
    const float v = is_value ? kvq::value_elem(codec, src, heads, D, h, d) : kvq::key_elem(codec, src, heads, D, h, d);
    dst[e] = __float2bfloat16(v * scale);
  }
}

}  // namespace afb

extern "C" {

// cache: byte rows [num_rows, row_bytes] in `codec`; row_idx int32 [n]; out bf16 [n, heads * D].
int afb_kvq_expand_rows(const void* cache, const int* row_idx, void* out, long n, long num_rows, int heads, int D,
                        int codec, int is_value, float scale, cudaStream_t stream) {
  using namespace afb;
  if (n <= 0) return 0;
  const long rb = is_value ? kvq::value_row_bytes(codec, heads, D) : kvq::key_row_bytes(codec, heads, D);
  if (rb <= 0 || n > 0x7fffffffL) {
    set_last_error("afb_kvq_expand_rows: unsupported codec / head size, or too many rows");
    return -1;
  }
  kvq_expand_rows_kernel<<<static_cast<unsigned>(n), 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(cache), rb, row_idx, reinterpret_cast<__nv_bfloat16*>(out), heads, D, codec,
      is_value, scale, num_rows);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// q [B, Hq, D] bf16 (one decode token per sequence); caches are byte arrays of [num_blocks, page] codec rows.
int afb_kvq_decode_attention(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                             const int* block_tables, int max_blocks, int page, int num_blocks, const int* kv_lens,
                             void* out, long out_stride, int B, int Hq, int Hkv, int D, int codec, int window,
                             float scale, float k_scale, float v_scale, cudaStream_t stream) {
  using namespace afb;
  if (B <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > kKvqMaxG) {
    set_last_error("afb_kvq_decode_attention: needs Hq a multiple of Hkv with at most 8 query heads per KV head");
    return -1;
  }
  KvqParams p;
  p.k_row_bytes = kvq::key_row_bytes(codec, Hkv, D);
  p.v_row_bytes = kvq::value_row_bytes(codec, Hkv, D);
  if (p.k_row_bytes <= 0 || p.v_row_bytes <= 0 || D > 256 || D <= 0 || page <= 0 || max_blocks <= 0 ||
      num_blocks <= 0 || !(scale > 0.0f)) {
    set_last_error("afb_kvq_decode_attention: unsupported codec / head size, or bad page geometry / scale");
    return -1;
  }
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.k_cache = reinterpret_cast<const uint8_t*>(k_cache);
  p.v_cache = reinterpret_cast<const uint8_t*>(v_cache);
  p.block_tables = block_tables;
  p.kv_lens = kv_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.max_blocks = max_blocks; p.page = page; p.num_blocks = num_blocks;
  p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.G = Hq / Hkv; p.codec = codec; p.window = window;
  p.scale = scale; p.k_scale = k_scale; p.v_scale = v_scale;
  const int G = p.G;
  const size_t smem = sizeof(float) * (static_cast<size_t>(G) * D + G * kvq::kTurbo3SketchBits +
                                       2 * kKvqWarps * G + static_cast<size_t>(kKvqWarps) * G * D);
  if (smem > 48 * 1024) {
    set_last_error("afb_kvq_decode_attention: G * D too large for the merge buffer");
    return -1;
  }
  const dim3 grid(Hkv, B), block(kKvqWarps * 32);
  const int dp = (D + 31) / 32;
  if (dp <= 2) kvq_decode_attn_kernel<2><<<grid, block, smem, stream>>>(p);
  else if (dp == 3) kvq_decode_attn_kernel<3><<<grid, block, smem, stream>>>(p);
  else if (dp == 4) kvq_decode_attn_kernel<4><<<grid, block, smem, stream>>>(p);
  else kvq_decode_attn_kernel<8><<<grid, block, smem, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
