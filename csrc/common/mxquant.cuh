// MX (OCP microscaling) fp8 activation quantisation shared by the kernels that emit GEMM-ready activations:
// e4m3 payload bytes [T, K] plus one e8m0 scale per 32-element block, stored in the 512-byte scale-factor atoms
// that tcgen05 block-scaled MMA reads ([ceil(T/128), K/128] atoms; byte (r % 32) * 16 + (r / 32) * 4 + kblock of
// an atom belongs to row r of the 128-row group and K block kblock of the 128-wide K chunk).
// The optional second term quantises the residual of the first, which makes the pair about bf16-exact.
#pragma once
#include "ptx.cuh"

namespace afb {

// Smallest power of two s with amax / s <= 448 (the e4m3 maximum, 1.75 * 2^8), as a biased e8m0 byte.
__device__ __forceinline__ uint32_t e8m0_for_amax(float amax) {
  if (!(amax > 0.0f)) return 127u - 8u;
  int e;
  const float m = frexpf(amax, &e);  // amax = m * 2^e, m in [0.5, 1)
  int s = e - 9 + ((m > 0.875f) ? 1 : 0);  // 448 = 0.875 * 2^9
  s = max(-127, min(127, s));
  return static_cast<uint32_t>(s + 127);
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ void unpack_e4m3x4(uint32_t v, float (&o)[4]) {
  const float2 a = e4m3x2_to_float2(static_cast<uint16_t>(v & 0xFFFF));
  const float2 b = e4m3x2_to_float2(static_cast<uint16_t>(v >> 16));
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

__device__ __forceinline__ size_t mx_sf_offset(int t, int k_chunks, int col) {
  const int kb = col >> 5, chunk = kb >> 2, j = kb & 3, r = t & 127;
  return (static_cast<size_t>(t >> 7) * k_chunks + chunk) * 512 + (r & 31) * 16 + (r >> 5) * 4 + j;
}

// Quantises the 4 consecutive values v of row t at columns [col, col + 4), col a multiple of 4.  The 8 lanes that
// hold one 32-element block (an aligned lane octet with consecutive col) must call this together; `store` = false
// lets a lane take part in the shuffles without writing (padding rows).  q1 / sf1 null: single term.
__device__ __forceinline__ void mx_quantize4_store(const float (&v)[4], int t, int col, int K, uint8_t* q0,
                                                   uint8_t* q1, uint8_t* sf0, uint8_t* sf1, bool store) {
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const uint32_t e0 = e8m0_for_amax(amax);
  const float inv0 = __uint_as_float((254u - e0) << 23);  // 2^-(e0 - 127)
  const uint32_t p0 = pack_e4m3x4(v[0] * inv0, v[1] * inv0, v[2] * inv0, v[3] * inv0);
  const size_t sf_off = mx_sf_offset(t, K >> 7, col);
  const bool lead = (col & 31) == 0;
  if (store) {
    *reinterpret_cast<uint32_t*>(q0 + static_cast<size_t>(t) * K + col) = p0;
    if (lead) sf0[sf_off] = static_cast<uint8_t>(e0);
  }
  if (q1) {
    float d[4];
    unpack_e4m3x4(p0, d);
    const float s0 = __uint_as_float(e0 << 23);
    float r[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) r[c] = v[c] - d[c] * s0;
    float rmax = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    const uint32_t e1 = e8m0_for_amax(rmax);
    const float inv1 = __uint_as_float((254u - e1) << 23);
    if (store) {
      *reinterpret_cast<uint32_t*>(q1 + static_cast<size_t>(t) * K + col) =
          pack_e4m3x4(r[0] * inv1, r[1] * inv1, r[2] * inv1, r[3] * inv1);
      if (lead) sf1[sf_off] = static_cast<uint8_t>(e1);
    }
  }
}

}  // namespace afb
