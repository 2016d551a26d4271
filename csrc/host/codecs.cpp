// CPU codecs for quantised artifact formats (the numerical authority the GPU paths are tested against):
// GGUF Q8_0 / Q4_0 / Q4_K / MXFP4 block dequantisation, fp16 / bf16 widening, fp8 E4M3 encode / decode and the
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

const float kMxfp4Values[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

}  // namespace

extern "C" {

// type ids: 0 F32, 1 F16, 2 Q4_0, 8 Q8_0, 12 Q4_K, 30 BF16, 39 MXFP4 (ggml numbering).
long afb_gguf_block_bytes(int type) {
  switch (type) {
    case 0: return 4; case 1: return 2; case 30: return 2;
    case 2: return 18; case 8: return 34; case 12: return 144; case 39: return 17;
    default: return -1;
  }
}
long afb_gguf_block_values(int type) {
  switch (type) {
    case 0: case 1: case 30: return 1;
    case 2: case 8: case 39: return 32;
    case 12: return 256;
    default: return -1;
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
    default: return -1;
  }
}

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

}  // extern "C"
