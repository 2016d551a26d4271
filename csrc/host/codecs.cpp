// CPU codecs for quantised artifact formats (the numerical authority the GPU paths are tested against):
// GGUF block dequantisation (legacy Q4/Q5/Q8, the K-quants Q2_K..Q6_K and Q8_K, IQ4_NL / IQ4_XS, ternary TQ1_0 /
// TQ2_0, MXFP4, NVFP4), fp16 / bf16 widening, fp8 E4M3 encode / decode and the
// int8 / int4 KV-cache encodings.
//
// Block geometry and decode rules follow the reference's gguf/tensor_types.zig:160-214 and gguf/quant_codec.zig
// (Q4_0 uses the ggml nibble order: low nibbles are elements 0..15, high nibbles 16..31; Q4_K packs eight 6-bit
// (scale, min) pairs in 12 bytes; MXFP4 is one e8m0 scale byte + 16 nibble bytes of e2m1 values), and the KV
// encodings follow zig/pkg/inference/KVCACHE.md:114-140 / runtime/kv/pool.zig:614-700 (fp8 = E4M3 bias 7, clamp
// +-448, no inf/NaN; int8 = per-head fp32 scale; int4 = groups of 32, fp16 scale + 16 packed bytes, low nibble first).
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../common/gguf_elem.h"

namespace {

inline float half_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400));
      bits = sign | ((127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000;
  int32_t exp = ((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFF;
  if (exp >= 31) return sign | 0x7C00 | (((x & 0x7FFFFFFF) > 0x7F800000) ? 0x200 : 0);
  if (exp <= 0) {
    if (exp < -10) return sign;
    man |= 0x800000;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return sign | h;
  }
  uint32_t h = (exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1FFF;
  if (rem > 0x1000 || (rem == 0x1000 && (h & 1))) ++h;
  return sign | h;
}

inline float e8m0_to_float(uint8_t e) {
  uint32_t bits = e ? (static_cast<uint32_t>(e) << 23) : 0x00400000u;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

inline void q4k_scale_min(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

inline float load_half(const uint8_t* p) {
  uint16_t h;
  memcpy(&h, p, 2);
  return half_to_float(h);
}

// Unsigned e4m3 (4 exponent bits, bias 7, 3 mantissa bits, no sign): the NVFP4 sub-block scale.
inline float ue4m3_to_float(uint8_t v) {
  const int exp = (v >> 3) & 0xF, man = v & 7;
  if (exp == 0) return man / 8.0f * 0.015625f;
  if (exp == 15 && man == 7) return 0.0f;
  return (1.0f + man / 8.0f) * ldexpf(1.0f, exp - 7);
}

const int8_t kIq4nlValues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

const float kMxfp4Values[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

}  // namespace

extern "C" {

// IQ codebook formats, Q8_1, Q1_0 and the plain integer / f64 types live in gguf_iq.cpp.
long afb_gguf_iq_block_bytes(int type);
long afb_gguf_iq_block_values(int type);
int afb_gguf_iq_dequantize(int type, const uint8_t* src, float* dst, long n_values);

// type ids (ggml numbering): 0 F32, 1 F16, 2 Q4_0, 3 Q4_1, 6 Q5_0, 7 Q5_1, 8 Q8_0, 10 Q2_K, 11 Q3_K, 12 Q4_K,
// 13 Q5_K, 14 Q6_K, 15 Q8_K, 20 IQ4_NL, 23 IQ4_XS, 30 BF16, 34 TQ1_0, 35 TQ2_0, 39 MXFP4, 40 NVFP4.
long afb_gguf_block_bytes(int type) {
  switch (type) {
    case 0: return 4; case 1: return 2; case 30: return 2;
    case 2: return 18; case 3: return 20; case 6: return 22; case 7: return 24; case 8: return 34;
    case 10: return 84; case 11: return 110; case 12: return 144; case 13: return 176; case 14: return 210;
    case 15: return 292; case 20: return 18; case 23: return 136; case 34: return 54; case 35: return 66;
    case 39: return 17; case 40: return 36;
    case 36: return 32; case 37: return 1;
    default: return afb_gguf_iq_block_bytes(type);
  }
}
long afb_gguf_block_values(int type) {
  switch (type) {
    case 0: case 1: case 30: case 37: return 1;
    case 36: return 128;
    case 2: case 3: case 6: case 7: case 8: case 20: case 39: return 32;
    case 40: return 64;
    case 10: case 11: case 12: case 13: case 14: case 15: case 23: case 34: case 35: return 256;
    default: return afb_gguf_iq_block_values(type);
  }
}

// Dequantises n_values (a multiple of the block size) from src to fp32 dst.  Returns 0, or -1 for an unknown type.
int afb_gguf_dequantize(int type, const uint8_t* src, float* dst, long n_values) {
  switch (type) {
    case 0: memcpy(dst, src, n_values * 4); return 0;
    case 1: { const uint16_t* h = reinterpret_cast<const uint16_t*>(src);
              for (long i = 0; i < n_values; ++i) dst[i] = half_to_float(h[i]); return 0; }
    case 30: { const uint16_t* h = reinterpret_cast<const uint16_t*>(src);
               for (long i = 0; i < n_values; ++i) { uint32_t b = static_cast<uint32_t>(h[i]) << 16; memcpy(&dst[i], &b, 4); }
               return 0; }
    case 36: {  // I2_S (BitNet): 32 bytes carry 128 ternary values; byte g holds values g, g + 32, g + 64, g + 96
                //  in bits 7-6, 5-4, 3-2, 1-0; codes 0 / 1 / 2 are -1 / 0 / +1.  The tensor's scale follows the blocks.
      static const float kMap[4] = {-1.0f, 0.0f, 1.0f, 0.0f};
      for (long b = 0; b < n_values / 128; ++b) {
        const uint8_t* p = src + b * 32;
        for (int g = 0; g < 32; ++g)
          for (int lane = 0; lane < 4; ++lane) dst[b * 128 + lane * 32 + g] = kMap[(p[g] >> (6 - 2 * lane)) & 3];
      }
      return 0;
    }
    case 37: {  // I8_S: signed bytes
      const int8_t* q = reinterpret_cast<const int8_t*>(src);
      for (long i = 0; i < n_values; ++i) dst[i] = static_cast<float>(q[i]);
      return 0;
    }
    case 8: {
      for (long b = 0; b < n_values / 32; ++b) {
        const uint8_t* p = src + b * 34;
        uint16_t dh; memcpy(&dh, p, 2);
        const float d = half_to_float(dh);
        const int8_t* q = reinterpret_cast<const int8_t*>(p + 2);
        for (int j = 0; j < 32; ++j) dst[b * 32 + j] = d * q[j];
      }
      return 0;
    }
    case 2: {
      for (long b = 0; b < n_values / 32; ++b) {
        const uint8_t* p = src + b * 18;
        uint16_t dh; memcpy(&dh, p, 2);
        const float d = half_to_float(dh);
        const uint8_t* q = p + 2;
        for (int j = 0; j < 16; ++j) {
          dst[b * 32 + j] = d * (static_cast<int>(q[j] & 0xF) - 8);
          dst[b * 32 + j + 16] = d * (static_cast<int>(q[j] >> 4) - 8);
        }
      }
      return 0;
    }
    case 12: {
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 144;
        uint16_t dh, mh; memcpy(&dh, p, 2); memcpy(&mh, p + 2, 2);
        const float d = half_to_float(dh), dmin = half_to_float(mh);
        const uint8_t* sc = p + 4;
        const uint8_t* q = p + 16;
        float* y = dst + b * 256;
        int is = 0;
        for (int j = 0; j < 256; j += 64) {
          uint8_t s1, m1, s2, m2;
          q4k_scale_min(is, sc, &s1, &m1);
          q4k_scale_min(is + 1, sc, &s2, &m2);
          const float d1 = d * s1, mm1 = dmin * m1, d2 = d * s2, mm2 = dmin * m2;
          for (int l = 0; l < 32; ++l) y[j + l] = d1 * (q[l] & 0xF) - mm1;
          for (int l = 0; l < 32; ++l) y[j + 32 + l] = d2 * (q[l] >> 4) - mm2;
          q += 32;
          is += 2;
        }
      }
      return 0;
    }
    case 39: {
      for (long b = 0; b < n_values / 32; ++b) {
        const uint8_t* p = src + b * 17;
        const float d = e8m0_to_float(p[0]);
        for (int j = 0; j < 16; ++j) {
          dst[b * 32 + j] = kMxfp4Values[p[1 + j] & 0xF] * d;
          dst[b * 32 + j + 16] = kMxfp4Values[p[1 + j] >> 4] * d;
        }
      }
      return 0;
    }
    case 3: {  // Q4_1: fp16 d, fp16 m, 16 nibble bytes; x = d * q + m
      for (long b = 0; b < n_values / 32; ++b) {
        const uint8_t* p = src + b * 20;
        const float d = load_half(p), m = load_half(p + 2);
        const uint8_t* q = p + 4;
        for (int j = 0; j < 16; ++j) {
          dst[b * 32 + j] = d * (q[j] & 0xF) + m;
          dst[b * 32 + j + 16] = d * (q[j] >> 4) + m;
        }
      }
      return 0;
    }
    case 6: case 7: {  // Q5_0 (fp16 d, offset 16) / Q5_1 (fp16 d, fp16 m): 32 fifth bits, then 16 nibble bytes
      const bool has_min = type == 7;
      const int bytes = has_min ? 24 : 22;
      for (long b = 0; b < n_values / 32; ++b) {
        const uint8_t* p = src + b * bytes;
        const float d = load_half(p), m = has_min ? load_half(p + 2) : 0.0f;
        uint32_t qh; memcpy(&qh, p + (has_min ? 4 : 2), 4);
        const uint8_t* q = p + (has_min ? 8 : 6);
        for (int j = 0; j < 16; ++j) {
          const int lo = (q[j] & 0xF) | (((qh >> j) & 1u) << 4);
          const int hi = (q[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4);
          dst[b * 32 + j] = has_min ? d * lo + m : d * (lo - 16);
          dst[b * 32 + j + 16] = has_min ? d * hi + m : d * (hi - 16);
        }
      }
      return 0;
    }
    case 10: {  // Q2_K: 16 x (4-bit scale | 4-bit min), 64 bytes of 2-bit values, fp16 d, fp16 dmin
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 84;
        const uint8_t* scales = p;
        const uint8_t* q = p + 16;
        const float d = load_half(p + 80), dmin = load_half(p + 82);
        float* y = dst + b * 256;
        int is = 0;
        for (int n = 0; n < 256; n += 128) {
          for (int shift = 0; shift < 8; shift += 2) {
            for (int half = 0; half < 2; ++half) {
              const uint8_t sc = scales[is++];
              const float dl = d * (sc & 0xF), ml = dmin * (sc >> 4);
              for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l + 16 * half] >> shift) & 3) - ml;
            }
          }
          q += 32;
        }
      }
      return 0;
    }
    case 11: {  // Q3_K: 32 bytes of high bits, 64 bytes of low 2-bit values, 16 six-bit scales in 12 bytes, fp16 d
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 110;
        const uint8_t* hm = p;
        const uint8_t* q = p + 32;
        const float d_all = load_half(p + 108);
        uint32_t aux[4] = {0, 0, 0, 0};
        memcpy(aux, p + 96, 12);
        const uint32_t k1 = 0x03030303u, k2 = 0x0f0f0f0fu, tmp = aux[2];
        aux[2] = ((aux[0] >> 4) & k2) | (((tmp >> 4) & k1) << 4);
        aux[3] = ((aux[1] >> 4) & k2) | (((tmp >> 6) & k1) << 4);
        aux[0] = (aux[0] & k2) | (((tmp >> 0) & k1) << 4);
        aux[1] = (aux[1] & k2) | (((tmp >> 2) & k1) << 4);
        int8_t scales[16];
        memcpy(scales, aux, 16);
        float* y = dst + b * 256;
        int is = 0;
        uint8_t m = 1;
        for (int n = 0; n < 256; n += 128) {
          for (int shift = 0; shift < 8; shift += 2) {
            for (int half = 0; half < 2; ++half) {
              const float dl = d_all * (scales[is++] - 32);
              for (int l = 0; l < 16; ++l) {
                const int lo = (q[l + 16 * half] >> shift) & 3;
                *y++ = dl * (lo - ((hm[l + 16 * half] & m) ? 0 : 4));
              }
            }
            m <<= 1;
          }
          q += 32;
        }
      }
      return 0;
    }
    case 13: {  // Q5_K: fp16 d, fp16 dmin, 12 scale bytes (as Q4_K), 32 bytes of fifth bits, 128 nibble bytes
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 176;
        const float d = load_half(p), dmin = load_half(p + 2);
        const uint8_t* sc = p + 4;
        const uint8_t* qh = p + 16;
        const uint8_t* ql = p + 48;
        float* y = dst + b * 256;
        int is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (int j = 0; j < 256; j += 64) {
          uint8_t s1, m1, s2, m2;
          q4k_scale_min(is, sc, &s1, &m1);
          q4k_scale_min(is + 1, sc, &s2, &m2);
          const float d1 = d * s1, mm1 = dmin * m1, d2 = d * s2, mm2 = dmin * m2;
          for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - mm1;
          for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - mm2;
          ql += 32;
          is += 2;
          u1 <<= 2;
          u2 <<= 2;
        }
      }
      return 0;
    }
    case 14: {  // Q6_K: 128 bytes of low nibbles, 64 bytes of high 2-bit pairs, 16 int8 scales, fp16 d
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 210;
        const uint8_t* ql = p;
        const uint8_t* qh = p + 128;
        const int8_t* sc = reinterpret_cast<const int8_t*>(p + 192);
        const float d = load_half(p + 208);
        float* y = dst + b * 256;
        for (int n = 0; n < 256; n += 128) {
          for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const int q1 = static_cast<int>((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int q2 = static_cast<int>((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int q3 = static_cast<int>((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int q4 = static_cast<int>((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            y[l] = d * sc[is] * q1;
            y[l + 32] = d * sc[is + 2] * q2;
            y[l + 64] = d * sc[is + 4] * q3;
            y[l + 96] = d * sc[is + 6] * q4;
          }
          y += 128; ql += 64; qh += 32; sc += 8;
        }
      }
      return 0;
    }
    case 15: {  // Q8_K: fp32 d, 256 int8 values, 16 int16 block sums (unused when decoding)
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 292;
        float d; memcpy(&d, p, 4);
        const int8_t* q = reinterpret_cast<const int8_t*>(p + 4);
        for (int j = 0; j < 256; ++j) dst[b * 256 + j] = d * q[j];
      }
      return 0;
    }
    case 20: {  // IQ4_NL: fp16 d, 16 nibble bytes indexing a fixed non-linear 16-entry table
      for (long b = 0; b < n_values / 32; ++b) {
        const uint8_t* p = src + b * 18;
        const float d = load_half(p);
        for (int j = 0; j < 16; ++j) {
          dst[b * 32 + j] = d * kIq4nlValues[p[2 + j] & 0xF];
          dst[b * 32 + j + 16] = d * kIq4nlValues[p[2 + j] >> 4];
        }
      }
      return 0;
    }
    case 23: {  // IQ4_XS: fp16 d, 8 six-bit sub-block scales (2 high bits in a u16, 4 low bits in nibbles), 128 nibble bytes
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 136;
        const float d = load_half(p);
        uint16_t sh; memcpy(&sh, p + 2, 2);
        const uint8_t* sl = p + 4;
        const uint8_t* q = p + 8;
        float* y = dst + b * 256;
        for (int ib = 0; ib < 8; ++ib) {
          const int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
          const float dl = d * (ls - 32);
          for (int j = 0; j < 16; ++j) {
            y[j] = dl * kIq4nlValues[q[j] & 0xF];
            y[j + 16] = dl * kIq4nlValues[q[j] >> 4];
          }
          y += 32; q += 16;
        }
      }
      return 0;
    }
    case 34: {  // TQ1_0: ternary digits packed five per byte (base 3, fixed-point), 48 + 4 bytes, fp16 d
      static const uint8_t pow3[6] = {1, 3, 9, 27, 81, 243};
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 54;
        const uint8_t* qs = p;
        const uint8_t* qh = p + 48;
        const float d = load_half(p + 52);
        float* y = dst + b * 256;
        auto digit = [](uint8_t byte, uint8_t mul) -> int {
          const uint8_t q = static_cast<uint8_t>(byte * mul);
          return static_cast<int>((static_cast<uint16_t>(q) * 3) >> 8);
        };
        for (int n = 0; n < 5; ++n)
          for (int m = 0; m < 32; ++m) *y++ = (digit(qs[m], pow3[n]) - 1) * d;
        for (int n = 0; n < 5; ++n)
          for (int m = 0; m < 16; ++m) *y++ = (digit(qs[32 + m], pow3[n]) - 1) * d;
        for (int n = 0; n < 4; ++n)
          for (int j = 0; j < 4; ++j) *y++ = (digit(qh[j], pow3[n]) - 1) * d;
      }
      return 0;
    }
    case 35: {  // TQ2_0: ternary values in 2 bits, 64 bytes, fp16 d
      for (long b = 0; b < n_values / 256; ++b) {
        const uint8_t* p = src + b * 66;
        const float d = load_half(p + 64);
        float* y = dst + b * 256;
        for (int j = 0; j < 64; j += 32)
          for (int l = 0; l < 4; ++l)
            for (int m = 0; m < 32; ++m) *y++ = (static_cast<int>((p[j + m] >> (l * 2)) & 3) - 1) * d;
      }
      return 0;
    }
    case 40: {  // NVFP4: four unsigned-e4m3 scales, then four 16-value sub-blocks of e2m1 nibbles (8 bytes each)
      for (long b = 0; b < n_values / 64; ++b) {
        const uint8_t* p = src + b * 36;
        for (int sub = 0; sub < 4; ++sub) {
          const float d = ue4m3_to_float(p[sub]);
          const uint8_t* q = p + 4 + sub * 8;
          float* y = dst + b * 64 + sub * 16;
          for (int j = 0; j < 8; ++j) {
            y[j] = kMxfp4Values[q[j] & 0xF] * d;
            y[j + 8] = kMxfp4Values[q[j] >> 4] * d;
          }
        }
      }
      return 0;
    }
    default: return afb_gguf_iq_dequantize(type, src, dst, n_values);
  }
}

// Value j of one block through the host/device per-element decoder (the code the GPU kernel runs).
float afb_gguf_element(int type, const uint8_t* block, int j) { return afb::gguf::element(type, block, j); }
long afb_gguf_element_block_values(int type) { return afb::gguf::block_values(type); }

// Quantisers (used by tests and the export tool).
int afb_gguf_quantize_q8_0(const float* src, uint8_t* dst, long n_values) {
  for (long b = 0; b < n_values / 32; ++b) {
    float amax = 0;
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(src[b * 32 + j]));
    const float d = amax / 127.0f, id = d > 0 ? 1.0f / d : 0.0f;
    const uint16_t dh = float_to_half(d);
    uint8_t* p = dst + b * 34;
    memcpy(p, &dh, 2);
    for (int j = 0; j < 32; ++j) reinterpret_cast<int8_t*>(p + 2)[j] = static_cast<int8_t>(lrintf(src[b * 32 + j] * id));
  }
  return 0;
}

int afb_gguf_quantize_q4_0(const float* src, uint8_t* dst, long n_values) {
  for (long b = 0; b < n_values / 32; ++b) {
    float amax = 0, mx = 0;
    for (int j = 0; j < 32; ++j) { const float v = src[b * 32 + j]; if (fabsf(v) > amax) { amax = fabsf(v); mx = v; } }
    const float d = mx / -8.0f, id = d != 0 ? 1.0f / d : 0.0f;
    const uint16_t dh = float_to_half(d);
    uint8_t* p = dst + b * 18;
    memcpy(p, &dh, 2);
    for (int j = 0; j < 16; ++j) {
      int a = static_cast<int>(src[b * 32 + j] * id + 8.5f), c = static_cast<int>(src[b * 32 + j + 16] * id + 8.5f);
      a = a < 0 ? 0 : (a > 15 ? 15 : a); c = c < 0 ? 0 : (c > 15 ? 15 : c);
      p[2 + j] = static_cast<uint8_t>(a | (c << 4));
    }
  }
  return 0;
}

// fp8 E4M3 (bias 7, max 448, no inf; NaN inputs map to 0) for the KV cache.
uint8_t afb_f32_to_e4m3(float f) {
  if (f != f) return 0;
  uint8_t sign = f < 0 ? 0x80 : 0;
  float a = fabsf(f);
  if (a >= 448.0f) return sign | 0x7E;
  if (a < 0.0009765625f) return sign;  // below half the smallest subnormal (2^-10)
  int e;
  float m = frexpf(a, &e);  // a = m * 2^e, m in [0.5, 1)
  int exp = e - 1 + 7;      // biased exponent of 1.xxx * 2^(e-1)
  if (exp <= 0) {
    // subnormal: value = man/8 * 2^-6
    int man = static_cast<int>(lrintf(a * 512.0f));  // a / 2^-9
    if (man >= 8) return sign | 0x08;
    return sign | static_cast<uint8_t>(man);
  }
  int man = static_cast<int>(lrintf((m * 2.0f - 1.0f) * 8.0f));
  if (man == 8) { man = 0; ++exp; }
  if (exp > 15 || (exp == 15 && man > 6)) return sign | 0x7E;
  return sign | static_cast<uint8_t>((exp << 3) | man);
}

float afb_e4m3_to_f32(uint8_t v) {
  const float sign = (v & 0x80) ? -1.0f : 1.0f;
  const int exp = (v >> 3) & 0xF, man = v & 7;
  if (exp == 0) return sign * man / 8.0f * 0.015625f;
  if (exp == 15 && man == 7) return 0.0f;  // the NaN encoding is never produced; decode it as 0
  return sign * (1.0f + man / 8.0f) * ldexpf(1.0f, exp - 7);
}

void afb_e4m3_lut(float* out256) {
  for (int i = 0; i < 256; ++i) out256[i] = afb_e4m3_to_f32(static_cast<uint8_t>(i));
}

// int8 KV: one fp32 scale per head vector.  Returns the scale.
float afb_kv_encode_int8(const float* src, int8_t* dst, int n) {
  float amax = 0;
  for (int i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(src[i]));
  const float scale = amax / 127.0f, inv = scale > 0 ? 1.0f / scale : 0.0f;
  for (int i = 0; i < n; ++i) dst[i] = static_cast<int8_t>(lrintf(src[i] * inv));
  return scale;
}

// int4 KV: groups of 32 -> fp16 scale + 16 bytes, low nibble first, values offset by 8.
void afb_kv_encode_int4(const float* src, uint8_t* dst, int n) {
  for (int g = 0; g < n / 32; ++g) {
    float amax = 0;
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(src[g * 32 + j]));
    const float scale = amax / 7.0f, inv = scale > 0 ? 1.0f / scale : 0.0f;
    const uint16_t sh = float_to_half(scale);
    uint8_t* p = dst + g * 18;
    memcpy(p, &sh, 2);
    for (int j = 0; j < 16; ++j) {
      int a = static_cast<int>(lrintf(src[g * 32 + 2 * j] * inv)) + 8, b = static_cast<int>(lrintf(src[g * 32 + 2 * j + 1] * inv)) + 8;
      a = a < 0 ? 0 : (a > 15 ? 15 : a); b = b < 0 ? 0 : (b > 15 ? 15 : b);
      p[2 + j] = static_cast<uint8_t>(a | (b << 4));
    }
  }
}

void afb_kv_decode_int4(const uint8_t* src, float* dst, int n) {
  for (int g = 0; g < n / 32; ++g) {
    const uint8_t* p = src + g * 18;
    uint16_t sh; memcpy(&sh, p, 2);
    const float scale = half_to_float(sh);
    for (int j = 0; j < 16; ++j) {
      dst[g * 32 + 2 * j] = scale * (static_cast<int>(p[2 + j] & 0xF) - 8);
      dst[g * 32 + 2 * j + 1] = scale * (static_cast<int>(p[2 + j] >> 4) - 8);
    }
  }
}

// Values [32 * sub, 32 * sub + 32) of one GGUF block through the decoder the fused matrix-vector kernel uses.
void afb_gguf_decode32(int type, const uint8_t* block, int sub, float* out) {
  afb::gguf::decode32(type, block, sub, out);
}

// The fused GGUF matrix-vector kernel's work split (kernels/gemm_gguf.cu) replayed on the host with the same index
// arithmetic: CTA -> 4 warps -> 2 rows each; K in chunks of 1024 values, lane l of a chunk owns sub-block l; per-lane
// partial sums are added lane by lane.  x [M, ldx] and out [M, N] are fp32 here.  Returns the number of
// (row, sub-block) units visited, or -1 for a type without a fused kernel.
long afb_gguf_mul_mv_host(int type, const uint8_t* W, const float* X, float* out, int M, int N, int K, long ldx) {
  const long bv = afb::gguf::block_values(type), bb = afb::gguf::block_bytes(type);
  if (bv < 0 || K % bv) return -1;
  const int kWarps = 4, kRows = 2, kChunk = 1024;
  const long row_bytes = static_cast<long>(K / bv) * bb;
  const int ctas = (N + kWarps * kRows - 1) / (kWarps * kRows);
  long units = 0;
  for (int cta = 0; cta < ctas; ++cta)
    for (int warp = 0; warp < kWarps; ++warp) {
      const int n0 = (cta * kWarps + warp) * kRows;
      for (int r = 0; r < kRows; ++r) {
        const int n = n0 + r;
        if (n >= N) continue;
        for (int m = 0; m < M; ++m) {
          float lanes[32] = {0};
          for (int kc = 0; kc < K; kc += kChunk)
            for (int lane = 0; lane < 32; ++lane) {
              const int k0 = kc + lane * 32;
              if (k0 >= K) continue;
              const long blk = k0 / bv;
              const int sub = static_cast<int>((k0 % bv) / 32);
              float wv[32];
              afb::gguf::decode32(type, W + n * row_bytes + blk * bb, sub, wv);
              float s = 0.0f;
              for (int i = 0; i < 32; ++i) s = fmaf(wv[i], X[m * ldx + k0 + i], s);
              lanes[lane] += s;
              if (m == 0) ++units;
            }
          float v = 0.0f;
          for (int lane = 0; lane < 32; ++lane) v += lanes[lane];
          out[static_cast<long>(m) * N + n] = v;
        }
      }
    }
  return units;
}

}  // extern "C"
