// Row normalisations with everything around them fused: LayerNorm / RMSNorm over bf16 rows with fp32
// statistics, optional residual add (and write-back of the sum), optional bias, and optional reduction of
// fp32 split-K / cross-GPU partial sums produced by the GEMM kernels.  One CTA per row, 16-byte vector
// accesses, the fp32 row staged in shared memory so the input is read from HBM exactly once.
//
// Replaces the reference's one-thread-per-row RMSNorm and 256-thread LayerNorm / add+LayerNorm
// (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:390-499) and the Metal
// rms-norm(+add, +scale) family (zig/pkg/inference/src/backends/metal_kernels.m:2477-2627).
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

struct NormParams {
  const __nv_bfloat16* x;         // [rows, H] or null
  const float* partials;          // [num_partials, rows, H] or null
  const __nv_bfloat16* residual;  // [rows, H] or null
  const __nv_bfloat16* bias;      // [H] or null (added before the norm)
  const __nv_bfloat16* gamma;     // [H]
  const __nv_bfloat16* beta;      // [H] or null
  __nv_bfloat16* sum_out;         // [rows, H] or null: x + partials + residual + bias
  __nv_bfloat16* y;               // [rows, H] or null: normalised output
  float* y_f32;                   // optional fp32 copy of the normalised output
  int rows, H, num_partials;
  long partial_stride;            // elements between partial slices
  int partials_bf16;              // 0: fp32 slices; 1: bf16 slices; 2: bf16 cross-GPU slots handed off Lamport-style
                                  // (poll each element against the sentinel, restore the sentinel after reading)
  float eps;
  int rms;                        // 1: RMSNorm, 0: LayerNorm
  int gamma_plus_one;             // 1: scale by (1 + gamma) (Gemma convention)
  // Optional MX-fp8 copy of the normalised output for the block-scaled GEMM: e4m3 terms [rows, H] and their
  // scale-factor atoms [ceil(rows/128), H/128, 512] (byte (r%32)*16 + (r/32)*4 + kblock).  q1/sf1 null: one term.
  uint8_t* q0;
  uint8_t* q1;
  uint8_t* sf0;
  uint8_t* sf1;
  // ---- tensor-parallel fused collectives (all zero when unused) ----
  // Reduce-scatter side: the partial slices of this rank's rows are pushed into `partials` by every rank's GEMM
  // epilogue; wait until each of the `wait_n` source counters reached `wait_expected`, then reduce.  The last CTA
  // past the wait re-arms the counters.
  int* wait_flags;
  int wait_n, wait_expected;
  int* wait_arrived;
  // All-gather side: the MX output row is written into every rank's activation buffers at row `row_offset + row`
  // (peer stores), then each rank's arrival counter is bumped.
  uint8_t* peer_q0[8];
  uint8_t* peer_q1[8];
  uint8_t* peer_sf0[8];
  uint8_t* peer_sf1[8];
  int* peer_x_ready[8];
  int ag_world, row_offset;
};

__device__ __forceinline__ int norm_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t mx_e8m0_for_amax(float amax) {
  if (!(amax > 0.0f)) return 127u - 8u;
  int e;
  const float m = frexpf(amax, &e);
  int s = e - 9 + ((m > 0.875f) ? 1 : 0);  // smallest power of two with amax / 2^s <= 448
  s = max(-127, min(127, s));
  return static_cast<uint32_t>(s + 127);
}

__device__ __forceinline__ uint32_t mx_pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// Quantises 8 consecutive values held by this thread; the 4 threads that share a 32-element block agree on the
// scale through two shuffles.  Must be called by all 4 threads of the group.
__device__ __forceinline__ void mx_quantize8(const float (&v)[8], uint8_t* q, uint8_t* sf_byte, bool write_sf,
                                             float (&resid)[8], uint2* packed_out = nullptr,
                                             uint32_t* scale_out = nullptr) {
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  // Groups of 4 lanes are active or inactive together (H is a multiple of 32), so the partners exist.
  const unsigned mask = __activemask();
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
  const uint32_t e = mx_e8m0_for_amax(amax);
  const float inv = __uint_as_float((254u - e) << 23);
  const float sc = __uint_as_float(e << 23);
  uint2 p;
  p.x = mx_pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
  p.y = mx_pack_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
  if (q) *reinterpret_cast<uint2*>(q) = p;
  if (write_sf && sf_byte) *sf_byte = static_cast<uint8_t>(e);
  if (packed_out) *packed_out = p;
  if (scale_out) *scale_out = e;
  const uint32_t w[2] = {p.x, p.y};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float2 a = e4m3x2_to_float2(static_cast<uint16_t>(w[h] & 0xFFFF));
    const float2 b = e4m3x2_to_float2(static_cast<uint16_t>(w[h] >> 16));
    resid[4 * h + 0] = v[4 * h + 0] - a.x * sc;
    resid[4 * h + 1] = v[4 * h + 1] - a.y * sc;
    resid[4 * h + 2] = v[4 * h + 2] - b.x * sc;
    resid[4 * h + 3] = v[4 * h + 3] - b.y * sc;
  }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}

__global__ void __launch_bounds__(512) norm_kernel(NormParams p) {
  extern __shared__ float srow[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int H = p.H;
  const size_t base = static_cast<size_t>(row) * H;
  griddep_launch();
  griddep_wait();
  if (p.wait_flags) {
    if (threadIdx.x < p.wait_n) {
      bool ok = false;
      PeerDeadline dl;
      for (uint32_t it = 0; it < AFB_SPIN_LIMIT; ++it) {
        if (norm_ld_acquire_sys(p.wait_flags + threadIdx.x) >= p.wait_expected) { ok = true; break; }
        if (dl.expired()) break;
        __nanosleep(20);
      }
      if (!ok) status_set(kStatusPeerFlagTimeout);
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(p.wait_arrived, 1) == static_cast<int>(gridDim.x) - 1) {
      // Every CTA of this kernel is past its wait and no rank can push again before it has seen this kernel's
      // output, so the counters can be re-armed here.
      *p.wait_arrived = 0;
      for (int s = 0; s < p.wait_n; ++s) atomicExch(p.wait_flags + s, 0);
    }
  }
  float lsum = 0.0f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
    if (p.x) {
      uint4 u = *reinterpret_cast<const uint4*>(p.x + base + i);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
    }
    if (p.partials_bf16 == 2) {
      // One-shot all-reduce, consumer side: the slots of all source ranks are polled together (one round trip
      // when the data is already there), each bounded; then summed in rank order.
      __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(const_cast<float*>(p.partials));
      uint4 u[8];
      unsigned pending = (1u << p.num_partials) - 1u;
      PeerDeadline dl;
      for (uint32_t it = 0; it < AFB_SPIN_LIMIT && pending; ++it) {
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (pending & (1u << s)) u[s] = ld_relaxed_sys_v4(pb + s * p.partial_stride + base + i);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if ((pending & (1u << s)) && !lamport_pending(u[s])) pending &= ~(1u << s);
        if (pending && dl.expired()) break;
        if (pending && it > 16) __nanosleep(20);
      }
      if (pending) status_set(kStatusPeerFlagTimeout);
      const uint4 sentinel = make_uint4(kLamportSentinelX2, kLamportSentinelX2, kLamportSentinelX2, kLamportSentinelX2);
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        if (s < p.num_partials) {
          *reinterpret_cast<uint4*>(pb + s * p.partial_stride + base + i) = sentinel;
          float2 a = unpack_bf16x2(u[s].x), b = unpack_bf16x2(u[s].y), c = unpack_bf16x2(u[s].z), d = unpack_bf16x2(u[s].w);
          v[0] += a.x; v[1] += a.y; v[2] += b.x; v[3] += b.y; v[4] += c.x; v[5] += c.y; v[6] += d.x; v[7] += d.y;
        }
      }
    } else if (p.partials_bf16) {
      const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(p.partials);
      for (int s = 0; s < p.num_partials; ++s) {
        const uint4 u = *reinterpret_cast<const uint4*>(pb + s * p.partial_stride + base + i);
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        v[0] += a.x; v[1] += a.y; v[2] += b.x; v[3] += b.y; v[4] += c.x; v[5] += c.y; v[6] += d.x; v[7] += d.y;
      }
    } else {
      for (int s = 0; s < p.num_partials; ++s) {
        const float4* pp = reinterpret_cast<const float4*>(p.partials + s * p.partial_stride + base + i);
        float4 a = pp[0], b = pp[1];
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w; v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
      }
    }
    if (p.bias) {
      uint4 u = *reinterpret_cast<const uint4*>(p.bias + i);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[0] += a.x; v[1] += a.y; v[2] += b.x; v[3] += b.y; v[4] += c.x; v[5] += c.y; v[6] += d.x; v[7] += d.y;
    }
    if (p.residual) {
      uint4 u = *reinterpret_cast<const uint4*>(p.residual + base + i);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[0] += a.x; v[1] += a.y; v[2] += b.x; v[3] += b.y; v[4] += c.x; v[5] += c.y; v[6] += d.x; v[7] += d.y;
    }
    if (p.sum_out) {
      uint4 u;
      u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
      u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(p.sum_out + base + i) = u;
      // The normalisation below sees exactly what was stored, so a later kernel that re-reads sum_out
      // and one that consumed y agree bit for bit.
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      srow[i + j] = v[j];
      lsum += p.rms ? v[j] * v[j] : v[j];
    }
  }
  if (!p.y && !p.y_f32 && !p.q0 && !p.ag_world) return;
  float mean = 0.0f, rstd;
  if (p.rms) {
    const float ss = block_sum(lsum, red);
    rstd = rsqrtf(ss / H + p.eps);
  } else {
    mean = block_sum(lsum, red) / H;
    float lv = 0.0f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = srow[i + j] - mean;
        lv += d * d;
      }
    }
    const float var = block_sum(lv, red) / H;
    rstd = rsqrtf(var + p.eps);
  }
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 g = *reinterpret_cast<const uint4*>(p.gamma + i);
    float gv[8], bv[8];
    {
      float2 a = unpack_bf16x2(g.x), b = unpack_bf16x2(g.y), c = unpack_bf16x2(g.z), d = unpack_bf16x2(g.w);
      gv[0] = a.x; gv[1] = a.y; gv[2] = b.x; gv[3] = b.y; gv[4] = c.x; gv[5] = c.y; gv[6] = d.x; gv[7] = d.y;
    }
    if (p.beta) {
      uint4 u = *reinterpret_cast<const uint4*>(p.beta + i);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      bv[0] = a.x; bv[1] = a.y; bv[2] = b.x; bv[3] = b.y; bv[4] = c.x; bv[5] = c.y; bv[6] = d.x; bv[7] = d.y;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) bv[j] = 0.0f;
    }
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g1 = p.gamma_plus_one ? gv[j] + 1.0f : gv[j];
      o[j] = (srow[i + j] - mean) * rstd * g1 + bv[j];
    }
    if (p.y) {
      uint4 u;
      u.x = pack_bf16x2(o[0], o[1]); u.y = pack_bf16x2(o[2], o[3]);
      u.z = pack_bf16x2(o[4], o[5]); u.w = pack_bf16x2(o[6], o[7]);
      *reinterpret_cast<uint4*>(p.y + base + i) = u;
    }
    if (p.y_f32) {
      float4* op = reinterpret_cast<float4*>(p.y_f32 + base + i);
      op[0] = make_float4(o[0], o[1], o[2], o[3]);
      op[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
    if (p.q0) {
      // Quantise what a bf16 consumer would have seen, so both paths agree.
      float ob[8], r1[8], r2[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[j] = __bfloat162float(__float2bfloat16(o[j]));
      const int kb = i / 32;
      const size_t sf_off = (static_cast<size_t>(row / 128) * (H / 128) + kb / 4) * 512 + ((row % 128) % 32) * 16 +
                            ((row % 128) / 32) * 4 + (kb % 4);
      const bool lead = (threadIdx.x & 3) == 0;
      mx_quantize8(ob, p.q0 + base + i, p.sf0 + sf_off, lead, r1);
      if (p.q1) mx_quantize8(r1, p.q1 + base + i, p.sf1 + sf_off, lead, r2);
    }
    if (p.ag_world) {
      // All-gather by pushing: quantise once, store the row into every rank's buffers.
      float ob[8], r1[8], r2[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[j] = __bfloat162float(__float2bfloat16(o[j]));
      const int grow = p.row_offset + row;
      const int kb = i / 32;
      const size_t sf_off = (static_cast<size_t>(grow / 128) * (H / 128) + kb / 4) * 512 + ((grow % 128) % 32) * 16 +
                            ((grow % 128) / 32) * 4 + (kb % 4);
      const size_t q_off = static_cast<size_t>(grow) * H + i;
      const bool lead = (threadIdx.x & 3) == 0;
      uint2 pk0, pk1 = make_uint2(0, 0);
      uint32_t e0, e1 = 0;
      mx_quantize8(ob, nullptr, nullptr, false, r1, &pk0, &e0);
      const bool two = p.peer_q1[0] != nullptr;
      if (two) mx_quantize8(r1, nullptr, nullptr, false, r2, &pk1, &e1);
      for (int o_ = 0; o_ < p.ag_world; ++o_) {
        *reinterpret_cast<uint2*>(p.peer_q0[o_] + q_off) = pk0;
        if (lead) p.peer_sf0[o_][sf_off] = static_cast<uint8_t>(e0);
        if (two) {
          *reinterpret_cast<uint2*>(p.peer_q1[o_] + q_off) = pk1;
          if (lead) p.peer_sf1[o_][sf_off] = static_cast<uint8_t>(e1);
        }
      }
    }
  }
  if (p.ag_world) {
    // Block barrier, then one system-scope releasing atomic per rank (cumulative over the block's peer stores).
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int o_ = 0; o_ < p.ag_world; ++o_)
        asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(p.peer_x_ready[o_]) : "memory");
    }
  }
}

// Warp-per-row variant for hidden sizes up to 1024 that are multiples of 256 (the encoder case: tens of
// thousands of short rows).  The row lives in registers, reductions are warp shuffles, there is no shared
// memory and no block barrier, and eight rows share a CTA -- about twice the bandwidth of the CTA-per-row kernel
// on 768-wide rows.  Plain x (+ bias) (+ residual) -> optional sum_out, LayerNorm / RMSNorm -> y.
template <int CHUNKS>
__global__ void __launch_bounds__(256) norm_warp_kernel(NormParams p) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const int lane = threadIdx.x & 31;
  const int H = p.H;
  const size_t base = static_cast<size_t>(row) * H;
  float v[CHUNKS][8];
  float lsum = 0.0f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = c * 256 + lane * 8;
    const uint4 u = *reinterpret_cast<const uint4*>(p.x + base + i);
    const uint32_t* w = &u.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(w[j]); v[c][2 * j] = f.x; v[c][2 * j + 1] = f.y; }
    if (p.bias) {
      const uint4 b = *reinterpret_cast<const uint4*>(p.bias + i);
      const uint32_t* bw = &b.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(bw[j]); v[c][2 * j] += f.x; v[c][2 * j + 1] += f.y; }
    }
    if (p.residual) {
      const uint4 r = *reinterpret_cast<const uint4*>(p.residual + base + i);
      const uint32_t* rw = &r.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(rw[j]); v[c][2 * j] += f.x; v[c][2 * j + 1] += f.y; }
    }
    if (p.sum_out) {
      uint4 o;
      uint32_t* ow = &o.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ow[j] = pack_bf16x2(v[c][2 * j], v[c][2 * j + 1]);
        const float2 f = unpack_bf16x2(ow[j]);
        v[c][2 * j] = f.x; v[c][2 * j + 1] = f.y;
      }
      *reinterpret_cast<uint4*>(p.sum_out + base + i) = o;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) lsum += p.rms ? v[c][j] * v[c][j] : v[c][j];
  }
  if (!p.y) return;
  float mean = 0.0f, rstd;
  if (p.rms) {
    rstd = rsqrtf(warp_sum(lsum) / H + p.eps);
  } else {
    mean = warp_sum(lsum) / H;
    float lv = 0.0f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = v[c][j] - mean; lv += d * d; }
    rstd = rsqrtf(warp_sum(lv) / H + p.eps);
  }
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = c * 256 + lane * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(p.gamma + i);
    uint4 be = make_uint4(0, 0, 0, 0);
    if (p.beta) be = *reinterpret_cast<const uint4*>(p.beta + i);
    const uint32_t* gw = &g.x;
    const uint32_t* bw = &be.x;
    uint4 o;
    uint32_t* ow = &o.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gg = unpack_bf16x2(gw[j]);
      const float2 bb = unpack_bf16x2(bw[j]);
      if (p.gamma_plus_one) { gg.x += 1.0f; gg.y += 1.0f; }
      ow[j] = pack_bf16x2((v[c][2 * j] - mean) * rstd * gg.x + bb.x, (v[c][2 * j + 1] - mean) * rstd * gg.y + bb.y);
    }
    *reinterpret_cast<uint4*>(p.y + base + i) = o;
  }
}

// BERT embeddings: word + position + token-type lookups, summed and LayerNormed in one pass.
struct BertEmbedParams {
  const int* ids;          // [T]
  const int* positions;    // [T]
  const int* type_ids;     // [T] or null (type 0)
  const __nv_bfloat16 *word, *pos, *type;  // tables [*, H]
  const __nv_bfloat16 *gamma, *beta;
  __nv_bfloat16* y;        // [T, H]
  int T, H, vocab, max_pos, n_types;
  float eps;
};

__global__ void bert_embed_ln_kernel(BertEmbedParams p) {
  extern __shared__ float srow[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  int id = p.ids[t], pos = p.positions[t], ty = p.type_ids ? p.type_ids[t] : 0;
  if (id < 0 || id >= p.vocab || pos < 0 || pos >= p.max_pos || ty < 0 || ty >= p.n_types) {
    status_set(kStatusBadIndex);
    id = min(max(id, 0), p.vocab - 1);
    pos = min(max(pos, 0), p.max_pos - 1);
    ty = min(max(ty, 0), p.n_types - 1);
  }
  const int H = p.H;
  float lsum = 0.0f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 a = *reinterpret_cast<const uint4*>(p.word + static_cast<size_t>(id) * H + i);
    uint4 b = *reinterpret_cast<const uint4*>(p.pos + static_cast<size_t>(pos) * H + i);
    uint4 c = *reinterpret_cast<const uint4*>(p.type + static_cast<size_t>(ty) * H + i);
    const uint32_t* au = &a.x; const uint32_t* bu = &b.x; const uint32_t* cu = &c.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = unpack_bf16x2(au[j]), y = unpack_bf16x2(bu[j]), z = unpack_bf16x2(cu[j]);
      const float v0 = x.x + y.x + z.x, v1 = x.y + y.y + z.y;
      srow[i + 2 * j] = v0; srow[i + 2 * j + 1] = v1;
      lsum += v0 + v1;
    }
  }
  const float mean = block_sum(lsum, red) / H;
  float lv = 0.0f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8)
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float d = srow[i + j] - mean; lv += d * d; }
  const float rstd = rsqrtf(block_sum(lv, red) / H + p.eps);
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 g = *reinterpret_cast<const uint4*>(p.gamma + i);
    uint4 be = *reinterpret_cast<const uint4*>(p.beta + i);
    const uint32_t* gu = &g.x; const uint32_t* bu = &be.x;
    uint4 o; uint32_t* ou = &o.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gg = unpack_bf16x2(gu[j]), bb = unpack_bf16x2(bu[j]);
      ou[j] = pack_bf16x2((srow[i + 2 * j] - mean) * rstd * gg.x + bb.x,
                          (srow[i + 2 * j + 1] - mean) * rstd * gg.y + bb.y);
    }
    *reinterpret_cast<uint4*>(p.y + static_cast<size_t>(t) * H + i) = o;
  }
}

// Plain embedding-row gather (decoder token embeddings), optional scale (Gemma multiplies by sqrt(H)).
__global__ void embed_gather_kernel(const int* ids, const __nv_bfloat16* table, __nv_bfloat16* y, int T, int H,
                                    int vocab, float scale) {
  const int t = blockIdx.x;
  griddep_launch();
  griddep_wait();
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    status_set(kStatusBadIndex);
    id = min(max(id, 0), vocab - 1);
  }
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 a = *reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * H + i);
    if (scale != 1.0f) {
      uint32_t* au = &a.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 x = unpack_bf16x2(au[j]);
        au[j] = pack_bf16x2(x.x * scale, x.y * scale);
      }
    }
    *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H + i) = a;
  }
}

static int norm_threads(int H) {
  int t = ((H / 8) + 31) / 32 * 32;
  if (t < 32) t = 32;
  if (t > 512) t = 512;  // norm_kernel is compiled for at most 512 threads (128 registers each)
  return t;
}

}  // namespace afb

extern "C" {

int afb_norm_tp(const void* x, const void* partials, int num_partials, long partial_stride, int partials_bf16,
                const void* residual,
                const void* bias, const void* gamma, const void* beta, void* sum_out, void* y, float* y_f32, int rows,
                int H, float eps, int rms, int gamma_plus_one, void* q0, void* q1, void* sf0, void* sf1,
                int* wait_flags, int wait_n, int wait_expected, int* wait_arrived, void* const* peer_q0,
                void* const* peer_q1, void* const* peer_sf0, void* const* peer_sf1, void* const* peer_x_ready,
                int ag_world, int row_offset, cudaStream_t stream);

int afb_norm(const void* x, const float* partials, int num_partials, long partial_stride, const void* residual,
             const void* bias, const void* gamma, const void* beta, void* sum_out, void* y, float* y_f32, int rows,
             int H, float eps, int rms, int gamma_plus_one, void* q0, void* q1, void* sf0, void* sf1,
             cudaStream_t stream) {
  return afb_norm_tp(x, partials, num_partials, partial_stride, 0, residual, bias, gamma, beta, sum_out, y, y_f32, rows,
                     H, eps, rms, gamma_plus_one, q0, q1, sf0, sf1, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr,
                     nullptr, nullptr, 0, 0, stream);
}

// Tensor-parallel form: optional wait on per-source arrival counters before reducing `partials` (the
// reduce-scatter half), optional push of the MX output row to every rank (the all-gather half).  partials_bf16 = 2:
// `partials` are the per-rank bf16 slots of a one-shot all-reduce, polled and cleared element-wise (no counters).
int afb_norm_tp(const void* x, const void* partials, int num_partials, long partial_stride, int partials_bf16,
                const void* residual,
                const void* bias, const void* gamma, const void* beta, void* sum_out, void* y, float* y_f32, int rows,
                int H, float eps, int rms, int gamma_plus_one, void* q0, void* q1, void* sf0, void* sf1,
                int* wait_flags, int wait_n, int wait_expected, int* wait_arrived, void* const* peer_q0,
                void* const* peer_q1, void* const* peer_sf0, void* const* peer_sf1, void* const* peer_x_ready,
                int ag_world, int row_offset, cudaStream_t stream) {
  using namespace afb;
  if (rows <= 0) return 0;
  if (H % 8 != 0 || H > 16384) {
    set_last_error("afb_norm: hidden size must be a multiple of 8 and <= 16384 (got %d)", H);
    return -1;
  }
  NormParams p = {};
  if (ag_world < 0 || ag_world > 8 || wait_n > 32) {
    set_last_error("afb_norm_tp: at most 8 ranks and 32 source counters");
    return -1;
  }
  p.wait_flags = wait_flags; p.wait_n = wait_n; p.wait_expected = wait_expected; p.wait_arrived = wait_arrived;
  p.ag_world = ag_world; p.row_offset = row_offset;
  for (int o = 0; o < ag_world; ++o) {
    p.peer_q0[o] = reinterpret_cast<uint8_t*>(peer_q0[o]);
    p.peer_q1[o] = peer_q1 ? reinterpret_cast<uint8_t*>(peer_q1[o]) : nullptr;
    p.peer_sf0[o] = reinterpret_cast<uint8_t*>(peer_sf0[o]);
    p.peer_sf1[o] = peer_sf1 ? reinterpret_cast<uint8_t*>(peer_sf1[o]) : nullptr;
    p.peer_x_ready[o] = reinterpret_cast<int*>(peer_x_ready[o]);
  }
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.partials = reinterpret_cast<const float*>(partials); p.num_partials = partials ? num_partials : 0;
  p.partial_stride = partial_stride; p.partials_bf16 = partials_bf16;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  p.beta = reinterpret_cast<const __nv_bfloat16*>(beta);
  p.sum_out = reinterpret_cast<__nv_bfloat16*>(sum_out);
  p.y = reinterpret_cast<__nv_bfloat16*>(y);
  p.y_f32 = y_f32;
  p.rows = rows; p.H = H; p.eps = eps; p.rms = rms; p.gamma_plus_one = gamma_plus_one;
  p.q0 = reinterpret_cast<uint8_t*>(q0); p.q1 = reinterpret_cast<uint8_t*>(q1);
  p.sf0 = reinterpret_cast<uint8_t*>(sf0); p.sf1 = reinterpret_cast<uint8_t*>(sf1);
  if ((q0 || ag_world) && (H % 128)) {
    set_last_error("afb_norm: MX output needs a hidden size that is a multiple of 128 (got %d)", H);
    return -1;
  }
  const size_t smem = static_cast<size_t>(H) * 4;
  AFB_CONFIGURE_KERNEL(norm_kernel, 16384 * 4, 256, 0);
  const bool plain = x && !p.num_partials && !y_f32 && !q0 && !ag_world && !wait_flags && (y || sum_out);
  if (plain && rows >= 512 && H % 256 == 0 && H <= 1024) {
    const int grid = (rows + 7) / 8;
    switch (H / 256) {
      case 1: norm_warp_kernel<1><<<grid, 256, 0, stream>>>(p); break;
      case 2: norm_warp_kernel<2><<<grid, 256, 0, stream>>>(p); break;
      case 3: norm_warp_kernel<3><<<grid, 256, 0, stream>>>(p); break;
      default: norm_warp_kernel<4><<<grid, 256, 0, stream>>>(p); break;
    }
    AFB_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  AFB_CHECK_CUDA(launch_pdl(norm_kernel, dim3(rows), dim3(norm_threads(H)), smem, stream, p));
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_bert_embed_ln(const int* ids, const int* positions, const int* type_ids, const void* word, const void* pos,
                      const void* type, const void* gamma, const void* beta, void* y, int T, int H, int vocab,
                      int max_pos, int n_types, float eps, cudaStream_t stream) {
  using namespace afb;
  if (T <= 0) return 0;
  if (H % 8 != 0 || H > 12288) {
    set_last_error("afb_bert_embed_ln: hidden size must be a multiple of 8 and <= 12288 (got %d)", H);
    return -1;
  }
  BertEmbedParams p;
  p.ids = ids; p.positions = positions; p.type_ids = type_ids;
  p.word = reinterpret_cast<const __nv_bfloat16*>(word);
  p.pos = reinterpret_cast<const __nv_bfloat16*>(pos);
  p.type = reinterpret_cast<const __nv_bfloat16*>(type);
  p.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  p.beta = reinterpret_cast<const __nv_bfloat16*>(beta);
  p.y = reinterpret_cast<__nv_bfloat16*>(y);
  p.T = T; p.H = H; p.vocab = vocab; p.max_pos = max_pos; p.n_types = n_types; p.eps = eps;
  bert_embed_ln_kernel<<<T, norm_threads(H), static_cast<size_t>(H) * 4, stream>>>(p);
  AFB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int afb_embed_gather(const int* ids, const void* table, void* y, int T, int H, int vocab, float scale,
                     cudaStream_t stream) {
  using namespace afb;
  if (T <= 0) return 0;
  if (H % 8 != 0) {
    set_last_error("afb_embed_gather: hidden size must be a multiple of 8 (got %d)", H);
    return -1;
  }
  AFB_CHECK_CUDA(launch_pdl(embed_gather_kernel, dim3(T), dim3(norm_threads(H)), 0, stream, ids,
                            reinterpret_cast<const __nv_bfloat16*>(table), reinterpret_cast<__nv_bfloat16*>(y), T, H,
                            vocab, scale));
  return 0;
}

}  // extern "C"
