// GGUF "IQ" codebook formats and the remaining simple tensor types, decoded to fp32.
//
// Block layouts (all little-endian; QK = 256 values per block unless noted), as fixed by the GGUF / ggml format and
// listed by the reference (zig/pkg/inference/src/gguf/tensor_types.zig:17-214; decoders in gguf/quant_codec.zig):
//
//   IQ2_XXS  66 B: f16 d | 8 x (u32 grid bytes, u32 signs+scale): four 8-value rows of the 256-row grid per group
//            of 32, each with a 7-bit sign index; 4-bit scale in the top bits: x = d (0.5 + s) 0.25 * grid * sign
//   IQ2_XS   74 B: f16 d | 32 x u16 (9-bit grid row, 7-bit sign index) | 8 scale bytes (two 4-bit scales)
//   IQ2_S    82 B: f16 d | 32 grid low bytes | 32 sign bytes | 8 bytes of 2-bit grid high bits | 8 scale bytes
//   IQ3_XXS  98 B: f16 d | 64 grid bytes (rows of 4 values) | 8 x u32 signs+scale: x = d (0.5 + s) 0.5 * grid * sign
//   IQ3_S   110 B: f16 d | 64 grid low bytes | 8 bytes of ninth bits | 32 sign bytes | 4 scale bytes: d (1 + 2 s)
//   IQ1_S    50 B: f16 d | 32 grid low bytes | 16 x u16 (4 x 3-bit grid high, 3-bit scale, delta sign)
//            x = d (2 s + 1) (grid +- 0.125), grid values in {-1, 0, 1}
//   IQ1_M    56 B: 32 grid low bytes | 16 bytes (two 3-bit grid high + delta-sign nibbles) | 4 x u16 scales whose
//            top nibbles spell the block's f16 d; a 3-bit scale per 16 values
//   Q8_1     36 B (32 values): f16 d, f16 sum, 32 int8          x = d * q
//   Q1_0     18 B (128 values): f16 d, 16 bytes of sign bits    x = +d where the bit is set, -d otherwise
//   I8 / I16 / I32 / I64 / F64: plain element conversions.
#include <stdint.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "../common/gguf_iq_grids.h"

namespace {

inline float h2f(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) { bits = sign; }
    else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) { bits = sign | 0x7F800000u | (man << 13); }
  else { bits = sign | ((exp + 112u) << 23) | (man << 13); }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline uint16_t rd16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
inline uint32_t rd32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }

struct Grids {
  std::vector<float> iq2xxs, iq2xs, iq2s, iq3xxs, iq3s, iq1s;
  uint8_t ksigns[128];
};

template <int NV>
std::vector<float> expand(const char* digits, int rows, int width, const signed char (&values)[NV]) {
  std::vector<float> g(static_cast<size_t>(rows) * width);
  for (size_t i = 0; i < g.size(); ++i) {
    const char c = digits[i];
    const int idx = c <= '9' ? c - '0' : c - 'a' + 10;
    g[i] = static_cast<float>(values[idx]);
  }
  return g;
}

const Grids& grids() {
  static Grids g;
  static std::once_flag once;
  std::call_once(once, [] {
    using namespace afb::iq;
    g.iq2xxs = expand(kIq2xxsDigits, kIq2xxsRows, kIq2xxsWidth, kIq2xxsValues);
    g.iq2xs = expand(kIq2xsDigits, kIq2xsRows, kIq2xsWidth, kIq2xsValues);
    g.iq2s = expand(kIq2sDigits, kIq2sRows, kIq2sWidth, kIq2sValues);
    g.iq3xxs = expand(kIq3xxsDigits, kIq3xxsRows, kIq3xxsWidth, kIq3xxsValues);
    g.iq3s = expand(kIq3sDigits, kIq3sRows, kIq3sWidth, kIq3sValues);
    g.iq1s = expand(kIq1sDigits, kIq1sRows, kIq1sWidth, kIq1sValues);
    // 7-bit sign index -> 8 sign bits: the eighth bit makes the number of minus signs even
    for (int i = 0; i < 128; ++i) g.ksigns[i] = static_cast<uint8_t>(i | ((__builtin_popcount(i) & 1) << 7));
  });
  return g;
}

inline void put8(float* dst, const float* row, float scale, uint8_t signs) {
  for (int j = 0; j < 8; ++j) dst[j] = scale * row[j] * ((signs >> j) & 1 ? -1.0f : 1.0f);
}
inline void put4(float* dst, const float* row, float scale, uint8_t signs4) {
  for (int j = 0; j < 4; ++j) dst[j] = scale * row[j] * ((signs4 >> j) & 1 ? -1.0f : 1.0f);
}

}  // namespace

extern "C" {

long afb_gguf_iq_block_bytes(int type) {
  switch (type) {
    case 9: return 36; case 16: return 66; case 17: return 74; case 18: return 98; case 19: return 50;
    case 21: return 110; case 22: return 82; case 29: return 56; case 41: return 18;
    case 24: return 1; case 25: return 2; case 26: return 4; case 27: return 8; case 28: return 8;
    default: return -1;
  }
}
long afb_gguf_iq_block_values(int type) {
  switch (type) {
    case 9: return 32; case 41: return 128;
    case 16: case 17: case 18: case 19: case 21: case 22: case 29: return 256;
    case 24: case 25: case 26: case 27: case 28: return 1;
    default: return -1;
  }
}

// Dequantises n_values (a multiple of the block size) of the types listed above.  Returns 0, -1 for another type.
int afb_gguf_iq_dequantize(int type, const uint8_t* src, float* dst, long n_values) {
  const long bv = afb_gguf_iq_block_values(type), bb = afb_gguf_iq_block_bytes(type);
  if (bv <= 0 || n_values % bv != 0) return -1;
  const Grids& G = grids();
  const long nb = n_values / bv;
  switch (type) {
    case 24: { const int8_t* p = reinterpret_cast<const int8_t*>(src); for (long i = 0; i < n_values; ++i) dst[i] = p[i]; return 0; }
    case 25: { for (long i = 0; i < n_values; ++i) dst[i] = static_cast<int16_t>(rd16(src + 2 * i)); return 0; }
    case 26: { for (long i = 0; i < n_values; ++i) dst[i] = static_cast<float>(static_cast<int32_t>(rd32(src + 4 * i))); return 0; }
    case 27: { for (long i = 0; i < n_values; ++i) { int64_t v; memcpy(&v, src + 8 * i, 8); dst[i] = static_cast<float>(v); } return 0; }
    case 28: { for (long i = 0; i < n_values; ++i) { double v; memcpy(&v, src + 8 * i, 8); dst[i] = static_cast<float>(v); } return 0; }
    case 9: {
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        for (int i = 0; i < 32; ++i) dst[b * 32 + i] = d * static_cast<int8_t>(p[4 + i]);
      }
      return 0;
    }
    case 41: {
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        for (int i = 0; i < 128; ++i) dst[b * 128 + i] = (p[2 + i / 8] >> (i % 8)) & 1 ? d : -d;
      }
      return 0;
    }
    case 16: {  // IQ2_XXS
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        for (int g = 0; g < 8; ++g) {
          const uint8_t* q = p + 2 + 8 * g;
          const uint32_t aux = rd32(q + 4);
          const float db = d * (0.5f + static_cast<float>(aux >> 28)) * 0.25f;
          for (int r = 0; r < 4; ++r)
            put8(dst + b * 256 + g * 32 + r * 8, &G.iq2xxs[static_cast<size_t>(q[r]) * 8], db,
                 G.ksigns[(aux >> (7 * r)) & 0x7F]);
        }
      }
      return 0;
    }
    case 17: {  // IQ2_XS
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        const uint8_t* sc = p + 2 + 64;
        for (int i = 0; i < 32; ++i) {          // 32 rows of 8 values; a 4-bit scale per 16 values
          const uint16_t q = rd16(p + 2 + 2 * i);
          const int s = (sc[i / 4] >> (4 * ((i / 2) & 1))) & 0xF;
          const float db = d * (0.5f + static_cast<float>(s)) * 0.25f;
          put8(dst + b * 256 + i * 8, &G.iq2xs[static_cast<size_t>(q & 511) * 8], db, G.ksigns[q >> 9]);
        }
      }
      return 0;
    }
    case 22: {  // IQ2_S
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        const uint8_t *qs = p + 2, *sg = p + 2 + 32, *qh = p + 2 + 64, *sc = p + 2 + 72;
        for (int i = 0; i < 32; ++i) {
          const int hi = (qh[i / 4] >> (2 * (i % 4))) & 3;
          const int s = (sc[i / 4] >> (4 * ((i / 2) & 1))) & 0xF;
          const float db = d * (0.5f + static_cast<float>(s)) * 0.25f;
          put8(dst + b * 256 + i * 8, &G.iq2s[static_cast<size_t>(qs[i] | (hi << 8)) * 8], db, sg[i]);
        }
      }
      return 0;
    }
    case 18: {  // IQ3_XXS
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        const uint8_t *qs = p + 2, *sa = p + 2 + 64;
        for (int g = 0; g < 8; ++g) {             // groups of 32 values: 8 grid rows of 4, one u32 of signs + scale
          const uint32_t aux = rd32(sa + 4 * g);
          const float db = d * (0.5f + static_cast<float>(aux >> 28)) * 0.5f;
          for (int r = 0; r < 4; ++r) {
            const uint8_t signs = G.ksigns[(aux >> (7 * r)) & 0x7F];
            put4(dst + b * 256 + g * 32 + r * 8, &G.iq3xxs[static_cast<size_t>(qs[g * 8 + 2 * r]) * 4], db, signs & 0xF);
            put4(dst + b * 256 + g * 32 + r * 8 + 4, &G.iq3xxs[static_cast<size_t>(qs[g * 8 + 2 * r + 1]) * 4], db, signs >> 4);
          }
        }
      }
      return 0;
    }
    case 21: {  // IQ3_S
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        const uint8_t *qs = p + 2, *qh = p + 2 + 64, *sg = p + 2 + 72, *sc = p + 2 + 104;
        for (int i = 0; i < 64; ++i) {            // 64 rows of 4 values; a 4-bit scale per 32 values
          const int hi = (qh[i / 8] >> (i % 8)) & 1;
          const int s = (sc[i / 16] >> (4 * ((i / 8) & 1))) & 0xF;
          const float db = d * static_cast<float>(1 + 2 * s);
          const uint8_t signs = sg[i / 2];
          put4(dst + b * 256 + i * 4, &G.iq3s[static_cast<size_t>(qs[i] | (hi << 8)) * 4], db,
               (i & 1) ? signs >> 4 : signs & 0xF);
        }
      }
      return 0;
    }
    case 19: {  // IQ1_S
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const float d = h2f(rd16(p));
        const uint8_t *qs = p + 2, *qhp = p + 2 + 32;
        for (int g = 0; g < 8; ++g) {             // groups of 32 values: 4 grid rows of 8
          const uint16_t qh = rd16(qhp + 2 * g);
          const float dl = d * static_cast<float>(2 * ((qh >> 12) & 7) + 1);
          const float delta = (qh & 0x8000) ? -0.125f : 0.125f;
          for (int r = 0; r < 4; ++r) {
            const float* row = &G.iq1s[static_cast<size_t>(qs[g * 4 + r] | (((qh >> (3 * r)) & 7) << 8)) * 8];
            for (int j = 0; j < 8; ++j) dst[b * 256 + g * 32 + r * 8 + j] = dl * (row[j] + delta);
          }
        }
      }
      return 0;
    }
    case 29: {  // IQ1_M
      for (long b = 0; b < nb; ++b) {
        const uint8_t* p = src + b * bb;
        const uint8_t *qs = p, *qh = p + 32, *scp = p + 48;
        uint16_t sc[4];
        for (int i = 0; i < 4; ++i) sc[i] = rd16(scp + 2 * i);
        const uint16_t dbits = static_cast<uint16_t>((sc[0] >> 12) | ((sc[1] >> 8) & 0x00F0) | ((sc[2] >> 4) & 0x0F00) |
                                                     (sc[3] & 0xF000));
        const float d = h2f(dbits);
        for (int i = 0; i < 32; ++i) {            // 32 rows of 8 values; a 3-bit scale per 16 values
          const int nib = (qh[i / 2] >> (4 * (i & 1))) & 0xF;
          const int s = (sc[i / 8] >> (3 * ((i / 2) & 3))) & 7;
          const float dl = d * static_cast<float>(2 * s + 1);
          const float delta = (nib & 8) ? -0.125f : 0.125f;
          const float* row = &G.iq1s[static_cast<size_t>(qs[i] | ((nib & 7) << 8)) * 8];
          for (int j = 0; j < 8; ++j) dst[b * 256 + i * 8 + j] = dl * (row[j] + delta);
        }
      }
      return 0;
    }
    default: return -1;
  }
}

}  // extern "C"
