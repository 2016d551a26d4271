// Per-element decoders of GGUF block formats, compiled for both the host and the device: value `j` of one block.
// The device kernel (csrc/kernels/gguf_dequant.cu) runs one of these per output element; the host entry point
// afb_gguf_element() exposes the very same code so it can be checked on a machine without a GPU against the
// block-at-a-time decoders in csrc/host/codecs.cpp.  Block layouts as in ggml (ids: 2 Q4_0, 8 Q8_0, 12 Q4_K,
// 13 Q5_K, 14 Q6_K, 39 MXFP4).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define AFB_HD __host__ __device__ __forceinline__
#else
#define AFB_HD inline
#endif

namespace afb {
namespace gguf {

AFB_HD float half_bits_to_float(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: normalise
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  union { uint32_t u; float f; } cv;
  cv.u = bits;
  return cv.f;
}

AFB_HD float load_half(const uint8_t* p) {
  return half_bits_to_float(static_cast<uint16_t>(p[0] | (static_cast<uint16_t>(p[1]) << 8)));
}

// (scale, min) number `j` of the 8 six-bit pairs packed in 12 bytes (Q4_K / Q5_K).
AFB_HD void k4_scale_min(int j, const uint8_t* q, int* sc, int* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

AFB_HD float e2m1_value(int code) {
  // 0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives
  const int m = code & 7;
  const float mag = m < 4 ? 0.5f * m : (m == 4 ? 2.0f : (m == 5 ? 3.0f : (m == 6 ? 4.0f : 6.0f)));
  return (code & 8) ? -mag : mag;
}

AFB_HD long block_values(int type) {
  switch (type) {
    case 2: case 8: case 39: return 32;
    case 12: case 13: case 14: return 256;
    default: return -1;
  }
}
AFB_HD long block_bytes(int type) {
  switch (type) {
    case 2: return 18; case 8: return 34; case 39: return 17;
    case 12: return 144; case 13: return 176; case 14: return 210;
    default: return -1;
  }
}

// Value j (0 <= j < block_values(type)) of the block at p.
AFB_HD float element(int type, const uint8_t* p, int j) {
  switch (type) {
    case 8:  // Q8_0: fp16 d, 32 int8
      return load_half(p) * static_cast<float>(static_cast<int8_t>(p[2 + j]));
    case 2: {  // Q4_0: fp16 d, 16 bytes; low nibbles are values 0..15, high nibbles 16..31; offset 8
      const uint8_t b = p[2 + (j & 15)];
      return load_half(p) * static_cast<float>(static_cast<int>(j < 16 ? (b & 0xF) : (b >> 4)) - 8);
    }
    case 39: {  // MXFP4: e8m0 scale byte, 16 bytes of e2m1 nibbles, same nibble order as Q4_0
      const uint8_t b = p[1 + (j & 15)];
      union { uint32_t u; float f; } sc;
      sc.u = p[0] ? (static_cast<uint32_t>(p[0]) << 23) : 0x00400000u;
      return e2m1_value(j < 16 ? (b & 0xF) : (b >> 4)) * sc.f;
    }
    case 12: {  // Q4_K: fp16 d, fp16 dmin, 12 scale bytes, 128 nibble bytes; 64-value groups share 32 bytes
      const int group = j >> 6, within = j & 63, hi = within >> 5, l = within & 31;
      int sc, mn;
      k4_scale_min(2 * group + hi, p + 4, &sc, &mn);
      const uint8_t b = p[16 + group * 32 + l];
      return load_half(p) * sc * static_cast<float>(hi ? (b >> 4) : (b & 0xF)) - load_half(p + 2) * mn;
    }
    case 13: {  // Q5_K: as Q4_K plus 32 bytes of fifth bits (bit 2 * group + hi of byte l)
      const int group = j >> 6, within = j & 63, hi = within >> 5, l = within & 31;
      int sc, mn;
      k4_scale_min(2 * group + hi, p + 4, &sc, &mn);
      const uint8_t b = p[48 + group * 32 + l];
      const int fifth = (p[16 + l] >> (2 * group + hi)) & 1;
      const int q = (hi ? (b >> 4) : (b & 0xF)) + (fifth << 4);
      return load_half(p) * sc * static_cast<float>(q) - load_half(p + 2) * mn;
    }
    case 14: {  // Q6_K: 128 low-nibble bytes, 64 bytes of 2-bit highs, 16 int8 scales, fp16 d
      const int half = j >> 7, within = j & 127, quarter = within >> 5, l = within & 31;
      const uint8_t* ql = p + half * 64;
      const uint8_t* qh = p + 128 + half * 32;
      const int8_t* sc = reinterpret_cast<const int8_t*>(p + 192) + half * 8;
      const uint8_t lo = ql[l + ((quarter & 1) ? 32 : 0)];
      const int nib = (quarter & 2) ? (lo >> 4) : (lo & 0xF);
      const int q = (nib | (((qh[l] >> (2 * quarter)) & 3) << 4)) - 32;
      return load_half(p + 208) * sc[(l >> 4) + 2 * quarter] * static_cast<float>(q);
    }
    default:
      return 0.0f;
  }
}

// Values [32 * sub, 32 * sub + 32) of the block at p, decoded together: the per-sub-block scale / offset is worked
// out once and every packed byte is read once.  Same values as element(type, p, 32 * sub + i).
// The fused matrix-vector kernel (kernels/gemm_gguf.cu) calls this with a compile-time `type`.
AFB_HD void decode32(int type, const uint8_t* p, int sub, float* out) {
  switch (type) {
    case 8: {  // Q8_0
      const float d = load_half(p);
      for (int i = 0; i < 32; ++i) out[i] = d * static_cast<float>(static_cast<int8_t>(p[2 + i]));
      return;
    }
    case 2: {  // Q4_0
      const float d = load_half(p);
      for (int i = 0; i < 16; ++i) {
        const uint8_t b = p[2 + i];
        out[i] = d * static_cast<float>(static_cast<int>(b & 0xF) - 8);
        out[i + 16] = d * static_cast<float>(static_cast<int>(b >> 4) - 8);
      }
      return;
    }
    case 39: {  // MXFP4
      union { uint32_t u; float f; } sc;
      sc.u = p[0] ? (static_cast<uint32_t>(p[0]) << 23) : 0x00400000u;
      for (int i = 0; i < 16; ++i) {
        const uint8_t b = p[1 + i];
        out[i] = e2m1_value(b & 0xF) * sc.f;
        out[i + 16] = e2m1_value(b >> 4) * sc.f;
      }
      return;
    }
    case 12: {  // Q4_K: sub-block = (group, half): 32 nibbles of the group's 32 bytes
      const int group = sub >> 1, hi = sub & 1;
      int sc, mn;
      k4_scale_min(sub, p + 4, &sc, &mn);
      const float d = load_half(p) * sc, m = load_half(p + 2) * mn;
      const uint8_t* q = p + 16 + group * 32;
      for (int i = 0; i < 32; ++i) out[i] = d * static_cast<float>(hi ? (q[i] >> 4) : (q[i] & 0xF)) - m;
      return;
    }
    case 13: {  // Q5_K
      const int group = sub >> 1, hi = sub & 1;
      int sc, mn;
      k4_scale_min(sub, p + 4, &sc, &mn);
      const float d = load_half(p) * sc, m = load_half(p + 2) * mn;
      const uint8_t* q = p + 48 + group * 32;
      for (int i = 0; i < 32; ++i) {
        const int v = (hi ? (q[i] >> 4) : (q[i] & 0xF)) + (((p[16 + i] >> sub) & 1) << 4);
        out[i] = d * static_cast<float>(v) - m;
      }
      return;
    }
    case 14: {  // Q6_K: sub-block = (half, quarter)
      const int half = sub >> 2, quarter = sub & 3;
      const uint8_t* ql = p + half * 64 + ((quarter & 1) ? 32 : 0);
      const uint8_t* qh = p + 128 + half * 32;
      const int8_t* sc = reinterpret_cast<const int8_t*>(p + 192) + half * 8 + 2 * quarter;
      const float d = load_half(p + 208);
      const float d0 = d * sc[0], d1 = d * sc[1];
      for (int i = 0; i < 32; ++i) {
        const int nib = (quarter & 2) ? (ql[i] >> 4) : (ql[i] & 0xF);
        const int v = (nib | (((qh[i] >> (2 * quarter)) & 3) << 4)) - 32;
        out[i] = (i < 16 ? d0 : d1) * static_cast<float>(v);
      }
      return;
    }
    default:
      for (int i = 0; i < 32; ++i) out[i] = 0.0f;
  }
}

}  // namespace gguf
}  // namespace afb
