// Decoder QKV post-processing in one pass over each token's fused QKV row:
//   reduce fp32 split-K partials (+ optional bias)  ->  optional per-head RMS norm of Q and K (Qwen3 / Gemma)
//   ->  rotary embedding on Q and K  ->  Q to a bf16 activation buffer, K and V into the paged KV cache at the
//   token's slot (bf16, or fp8 e4m3 with a per-tensor scale).
//
// RoPE semantics follow the reference's ropeCore (zig/lib/linalg/src/attention.zig:65-86):
// freq_j = theta^(-2j/rope_dim), angle = position * freq_scale * freq_j, pairs (j, j + rope_dim/2) in the
// half-split (Llama) convention or (2j, 2j+1) in the consecutive convention, dims >= rope_dim untouched.
// The fused head-RMS + RoPE corresponds to the reference's Metal apply_head_rms_rope
// (zig/pkg/inference/src/backends/metal_kernels.m:2575); the KV write to KvPool.writeToken
// (zig/pkg/inference/src/runtime/kv/pool.zig:351).
#include <cuda_fp8.h>

#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

struct RopeKvParams {
  const __nv_bfloat16* qkv;   // [T, row] or null
  const float* partials;      // [S, T, row] or null
  int num_partials;
  long partial_stride;
  const __nv_bfloat16* bias;  // [row] or null
  const int* positions;       // [T]
  const int* slots;           // [T] cache slot (block * page + offset) or < 0 to skip the KV write
  const __nv_bfloat16* q_norm_w;  // [D] or null
  const __nv_bfloat16* k_norm_w;  // [D] or null
  __nv_bfloat16* q_out;       // [T, Hq*D]
  void* k_cache;              // [slots, Hkv, D]
  void* v_cache;
  int T, Hq, Hkv, D;
  int rope_dim, half_split;
  float log2_theta, freq_scale, norm_eps;
  int norm_plus_one;
  int kv_fp8;                 // 1: caches are e4m3 bytes scaled by kv_scale_inv
  float kv_scale_inv;
  long num_slots;
  // Context-extension schemes (llama3, yarn, longrope): a table of rope_dim / 2 frequencies replaces the
  // closed form, and cos / sin are multiplied by the scheme's attention factor.  Null: the closed form.
  const float* inv_freq;
  float rope_mscale;
};

__device__ __forceinline__ float load_val(const RopeKvParams& p, size_t t, int row_width, int col) {
  float v = 0.0f;
  if (p.qkv) v = __bfloat162float(p.qkv[t * row_width + col]);
  for (int s = 0; s < p.num_partials; ++s) v += p.partials[s * p.partial_stride + t * row_width + col];
  if (p.bias) v += __bfloat162float(p.bias[col]);
  return v;
}

__device__ __forceinline__ void store_kv(const RopeKvParams& p, void* cache, size_t idx, float v) {
  if (p.kv_fp8) {
    reinterpret_cast<__nv_fp8_e4m3*>(cache)[idx] = __nv_fp8_e4m3(v * p.kv_scale_inv);
  } else {
    reinterpret_cast<__nv_bfloat16*>(cache)[idx] = __float2bfloat16(v);
  }
}

// gridDim.x = tokens, gridDim.y = groups of heads; each warp takes one head of the group at a time (Hq query
// heads, then Hkv key heads, then Hkv value heads).
__global__ void rope_kv_kernel(RopeKvParams p) {
  const int t = blockIdx.x;
  griddep_launch();
  griddep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x >> 5) * gridDim.y;
  const int D = p.D, half = D / 2;
  const int row_width = (p.Hq + 2 * p.Hkv) * D;
  const float pos = static_cast<float>(p.positions[t]);
  long slot = p.slots ? p.slots[t] : -1;
  if (slot >= p.num_slots) {
    status_set(kStatusBadIndex);
    slot = -1;
  }
  const int rd = p.rope_dim, rh = rd / 2;
  const int total_heads = p.Hq + 2 * p.Hkv;
  for (int hd = blockIdx.y * (blockDim.x >> 5) + warp; hd < total_heads; hd += nw) {
    const int kind = hd < p.Hq ? 0 : (hd < p.Hq + p.Hkv ? 1 : 2);
    const int col0 = hd * D;
    const int hl = kind == 0 ? hd : (kind == 1 ? hd - p.Hq : hd - p.Hq - p.Hkv);
    if (kind == 2) {
      if (slot >= 0) {
        for (int i = lane; i < D; i += 32)
          store_kv(p, p.v_cache, (static_cast<size_t>(slot) * p.Hkv + hl) * D + i, load_val(p, t, row_width, col0 + i));
      }
      continue;
    }
    if (kind == 1 && slot < 0) continue;
    // Each lane owns pair slots j = lane, lane+32, ... < D/2.  Pair slot j < rope_dim/2 is a rotated pair,
    // the rest pass two untouched dims through.
    float a[4], b[4];
    int ia[4], ib[4];
    float ss = 0.0f;
    int cnt = 0;
    for (int j = lane; j < half; j += 32, ++cnt) {
      int i0, i1;
      if (j < rh) {
        if (p.half_split) { i0 = j; i1 = j + rh; } else { i0 = 2 * j; i1 = 2 * j + 1; }
      } else {
        i0 = rd + 2 * (j - rh); i1 = i0 + 1;
      }
      ia[cnt] = i0; ib[cnt] = i1;
      a[cnt] = load_val(p, t, row_width, col0 + i0);
      b[cnt] = load_val(p, t, row_width, col0 + i1);
      ss += a[cnt] * a[cnt] + b[cnt] * b[cnt];
    }
    const __nv_bfloat16* nw_ptr = kind == 0 ? p.q_norm_w : p.k_norm_w;
    if (nw_ptr) {
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / D + p.norm_eps);
      for (int c = 0; c < cnt; ++c) {
        const float wa = __bfloat162float(nw_ptr[ia[c]]) + (p.norm_plus_one ? 1.0f : 0.0f);
        const float wb = __bfloat162float(nw_ptr[ib[c]]) + (p.norm_plus_one ? 1.0f : 0.0f);
        a[c] *= r * wa;
        b[c] *= r * wb;
      }
    }
    cnt = 0;
    for (int j = lane; j < half; j += 32, ++cnt) {
      float x = a[cnt], y = b[cnt];
      if (j < rh) {
        const float freq = p.inv_freq ? p.inv_freq[j]
                                      : exp2f(-2.0f * static_cast<float>(j) / static_cast<float>(rd) * p.log2_theta);
        float sn, cs;
        sincosf(pos * p.freq_scale * freq, &sn, &cs);
        if (p.inv_freq) { sn *= p.rope_mscale; cs *= p.rope_mscale; }
        const float rx = x * cs - y * sn, ry = x * sn + y * cs;
        x = rx; y = ry;
      }
      if (kind == 0) {
        __nv_bfloat16* qo = p.q_out + static_cast<size_t>(t) * p.Hq * D + hl * D;
        qo[ia[cnt]] = __float2bfloat16(x);
        qo[ib[cnt]] = __float2bfloat16(y);
      } else {
        const size_t base = (static_cast<size_t>(slot) * p.Hkv + hl) * D;
        store_kv(p, p.k_cache, base + ia[cnt], x);
        store_kv(p, p.k_cache, base + ib[cnt], y);
      }
    }
  }
}

// Standalone RoPE on a [T, heads, D] bf16 tensor, in place (encoders with rotary positions, tests).  Token rows are
// row_stride elements apart, so the Q and K heads of a fused QKV buffer can be rotated where they lie.
__global__ void rope_inplace_kernel(__nv_bfloat16* x, const int* positions, int heads, int D, int rope_dim,
                                    int half_split, float log2_theta, float freq_scale, long row_stride) {
  const int t = blockIdx.x;
  const float pos = static_cast<float>(positions[t]);
  const int rh = rope_dim / 2;
  for (int idx = threadIdx.x; idx < heads * rh; idx += blockDim.x) {
    const int h = idx / rh, j = idx % rh;
    const int i0 = half_split ? j : 2 * j, i1 = half_split ? j + rh : 2 * j + 1;
    __nv_bfloat16* row = x + static_cast<size_t>(t) * row_stride + static_cast<size_t>(h) * D;
    const float a = __bfloat162float(row[i0]), b = __bfloat162float(row[i1]);
    const float freq = exp2f(-2.0f * static_cast<float>(j) / static_cast<float>(rope_dim) * log2_theta);
    float sn, cs;
    sincosf(pos * freq_scale * freq, &sn, &cs);
    row[i0] = __float2bfloat16(a * cs - b * sn);
    row[i1] = __float2bfloat16(a * sn + b * cs);
  }
}

// Copies whole KV blocks inside the cache (copy-on-write of a shared prefix block, defragmentation).
__global__ void kv_copy_blocks_kernel(uint4* k_cache, uint4* v_cache, const int* src, const int* dst,
                                      long block_u4) {
  const int pair = blockIdx.x;
  const long s = static_cast<long>(src[pair]) * block_u4, d = static_cast<long>(dst[pair]) * block_u4;
  for (long i = threadIdx.x; i < block_u4; i += blockDim.x) {
    k_cache[d + i] = k_cache[s + i];
    v_cache[d + i] = v_cache[s + i];
  }
}

}  // namespace afb

extern "C" {

// As afb_rope_kv_write, with the rotary frequencies taken from a table (inv_freq: rope_dim / 2 floats in device
// memory) and cos / sin scaled by rope_mscale: the frequency-dependent context-extension schemes.
int afb_rope_kv_write_x(const void* qkv, const float* partials, int num_partials, long partial_stride,
                        const void* bias, const int* positions, const int* slots, const void* q_norm_w,
                        const void* k_norm_w, void* q_out, void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D,
                        int rope_dim, int half_split, float theta, float freq_scale, float norm_eps, int norm_plus_one,
                        int kv_fp8, float kv_scale, long num_slots, const float* inv_freq, float rope_mscale,
                        cudaStream_t stream);

int afb_rope_kv_write(const void* qkv, const float* partials, int num_partials, long partial_stride,
                      const void* bias, const int* positions, const int* slots, const void* q_norm_w,
                      const void* k_norm_w, void* q_out, void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D,
                      int rope_dim, int half_split, float theta, float freq_scale, float norm_eps, int norm_plus_one,
                      int kv_fp8, float kv_scale, long num_slots, cudaStream_t stream) {
  return afb_rope_kv_write_x(qkv, partials, num_partials, partial_stride, bias, positions, slots, q_norm_w, k_norm_w,
                             q_out, k_cache, v_cache, T, Hq, Hkv, D, rope_dim, half_split, theta, freq_scale, norm_eps,
                             norm_plus_one, kv_fp8, kv_scale, num_slots, nullptr, 1.0f, stream);
}

int afb_rope_kv_write_x(const void* qkv, const float* partials, int num_partials, long partial_stride,
                        const void* bias, const int* positions, const int* slots, const void* q_norm_w,
                        const void* k_norm_w, void* q_out, void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D,
                        int rope_dim, int half_split, float theta, float freq_scale, float norm_eps, int norm_plus_one,
                        int kv_fp8, float kv_scale, long num_slots, const float* inv_freq, float rope_mscale,
                        cudaStream_t stream) {
  using namespace afb;
  if (T <= 0) return 0;
  if (D > 256 || (D & 1) || rope_dim > D || (rope_dim & 1)) {
    set_last_error("afb_rope_kv_write: head_dim must be even and <= 256, rope_dim even and <= head_dim");
    return -1;
  }
  RopeKvParams p;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.partials = partials; p.num_partials = partials ? num_partials : 0; p.partial_stride = partial_stride;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.positions = positions; p.slots = slots;
  p.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(q_norm_w);
  p.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(k_norm_w);
  p.q_out = reinterpret_cast<__nv_bfloat16*>(q_out);
  p.k_cache = k_cache; p.v_cache = v_cache;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.rope_dim = rope_dim; p.half_split = half_split;
  p.log2_theta = log2f(theta); p.freq_scale = freq_scale; p.norm_eps = norm_eps; p.norm_plus_one = norm_plus_one;
  p.kv_fp8 = kv_fp8; p.kv_scale_inv = kv_scale > 0.0f ? 1.0f / kv_scale : 1.0f; p.num_slots = num_slots;
  p.inv_freq = inv_freq; p.rope_mscale = rope_mscale;
  const int total_heads = Hq + 2 * Hkv;
  // Few tokens (decode): spread the heads of a token over several CTAs; many tokens: one CTA per token.
  int groups = T >= 1024 ? 1 : (total_heads + 7) / 8;
  if (groups < 1) groups = 1;
  dim3 grid(T, groups);
  AFB_CHECK_CUDA(launch_pdl(rope_kv_kernel, grid, dim3(256), 0, stream, p));
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_rope_inplace_strided(void* x, const int* positions, int T, int heads, int D, int rope_dim, int half_split,
                             float theta, float freq_scale, long row_stride, cudaStream_t stream) {
  using namespace afb;
  if (T <= 0) return 0;
  if (row_stride < static_cast<long>(heads) * D || rope_dim > D || rope_dim % 2) {
    set_last_error("afb_rope_inplace: row stride shorter than heads * D, or bad rope_dim");
    return -1;
  }
  rope_inplace_kernel<<<T, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(x), positions, heads, D, rope_dim,
                                             half_split, log2f(theta), freq_scale, row_stride);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_rope_inplace(void* x, const int* positions, int T, int heads, int D, int rope_dim, int half_split, float theta,
                     float freq_scale, cudaStream_t stream) {
  return afb_rope_inplace_strided(x, positions, T, heads, D, rope_dim, half_split, theta, freq_scale,
                                  static_cast<long>(heads) * D, stream);
}

int afb_kv_copy_blocks(void* k_cache, void* v_cache, const int* src, const int* dst, int n_pairs, long block_bytes,
                       cudaStream_t stream) {
  using namespace afb;
  if (n_pairs <= 0) return 0;
  if (block_bytes % 16) {
    set_last_error("afb_kv_copy_blocks: block size must be a multiple of 16 bytes");
    return -1;
  }
  kv_copy_blocks_kernel<<<n_pairs, 256, 0, stream>>>(reinterpret_cast<uint4*>(k_cache),
                                                     reinterpret_cast<uint4*>(v_cache), src, dst, block_bytes / 16);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
