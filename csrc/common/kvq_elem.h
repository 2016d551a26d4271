// Quantised KV-cache row formats, compiled for both the host and the device.
//
// One cache row holds one token: all KV heads of the key (or of the value).  Codecs and their row layouts follow
// the reference's KV pool (zig/pkg/inference/src/runtime/kv/pool.zig:30-130, 610-890) and its 4-bit / 3-bit key
// codecs (zig/pkg/inference/src/runtime/kv/turboquant.zig:30-330):
//
//   bf16    heads * D bf16 values
//   fp8     heads * D e4m3 bytes
//   int8    per head: one f32 scale (max|x| / 127, 1 when the head is all zero), then D int8 codes
//   int4    over the flattened row, groups of 32: one f16 scale (max|x| / 7), then 16 bytes of two signed nibbles
//           (element 2i in the low nibble)
//   polar4  keys: two 4-bit codes per byte on the fixed grid c / 7.5 - 1 in [-1, 1]; values: the int8 layout
//   turbo3  keys: 3-bit codes packed little-endian bit by bit on the grid c / 3.5 - 1, followed by a 32-bit sign
//           sketch per head of the residual under pseudo-random +-1 projections; values: the int8 layout
//
// The attention kernels (csrc/kernels/attention_kvq.cu) and the host codecs (csrc/host/kv_codecs.cpp) both go
// through the element accessors below, so the device arithmetic can be checked on a machine without a GPU.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define AFB_KVQ_HD __host__ __device__ __forceinline__
#else
#define AFB_KVQ_HD inline
#endif

namespace afb {
namespace kvq {

enum Codec { kBf16 = 0, kFp8 = 1, kInt8 = 2, kInt4 = 3, kPolar4 = 4, kTurbo3 = 5 };

constexpr int kInt4Group = 32;
constexpr int kInt4GroupBytes = 2 + kInt4Group / 2;
constexpr int kTurbo3SketchBits = 32;
constexpr float kTurbo3ResidualScale = 0.125f;

AFB_KVQ_HD float bits_to_float(uint32_t u) {
  union { uint32_t u; float f; } cv;
  cv.u = u;
  return cv.f;
}

AFB_KVQ_HD uint32_t float_to_bits(float f) {
  union { uint32_t u; float f; } cv;
  cv.f = f;
  return cv.u;
}

AFB_KVQ_HD float half_to_float(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  if (exp == 0) {
    if (man == 0) return bits_to_float(sign);
    int e = -1;
    do { man <<= 1; ++e; } while (!(man & 0x400u));
    return bits_to_float(sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13));
  }
  if (exp == 31) return bits_to_float(sign | 0x7F800000u | (man << 13));
  return bits_to_float(sign | ((exp + 112u) << 23) | (man << 13));
}

AFB_KVQ_HD float fp8_e4m3_to_float(uint8_t b) {
  const uint32_t sign = static_cast<uint32_t>(b & 0x80u) << 24;
  const uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
  if (e == 0) {  // subnormal: m * 2^-9
    const float v = static_cast<float>(m) * 0.001953125f;
    return (b & 0x80u) ? -v : v;
  }
  if (e == 15 && m == 7) return bits_to_float(sign | 0x7FC00000u);  // the single NaN pattern
  return bits_to_float(sign | ((e + 120u) << 23) | (m << 20));
}

// Round to nearest even, saturating at +-448 (0x7E); NaN maps to 0x7F.
AFB_KVQ_HD uint8_t float_to_fp8_e4m3(float f) {
  const uint32_t u = float_to_bits(f);
  const uint8_t sign = static_cast<uint8_t>((u >> 24) & 0x80u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return sign | 0x7F;
  if (a >= 0x43E80000u) return sign | 0x7E;  // >= 464 rounds past 448: saturate (and so does infinity)
  const int e = static_cast<int>(a >> 23) - 127;
  if (e < -6) {  // subnormal range: units of 2^-9
    const float q = bits_to_float(a) * 512.0f;  // exact scaling
    int r = static_cast<int>(q);
    const float frac = q - static_cast<float>(r);
    if (frac > 0.5f || (frac == 0.5f && (r & 1))) ++r;
    return sign | static_cast<uint8_t>(r);  // r == 8 is the smallest normal, whose encoding is 0x08
  }
  uint32_t m = a & 0x7FFFFFu;
  uint32_t keep = m >> 20;
  const uint32_t rest = m & 0xFFFFFu;
  uint32_t ee = static_cast<uint32_t>(e + 7);
  if (rest > 0x80000u || (rest == 0x80000u && (keep & 1u))) {
    if (++keep == 8u) { keep = 0; ++ee; }
  }
  if (ee > 15u || (ee == 15u && keep == 7u)) return sign | 0x7E;
  return sign | static_cast<uint8_t>((ee << 3) | keep);
}

AFB_KVQ_HD float bf16_to_float(uint16_t h) { return bits_to_float(static_cast<uint32_t>(h) << 16); }

AFB_KVQ_HD bool head_dim_supported(int D) { return D == 64 || D == 80 || D == 128 || D == 256; }

AFB_KVQ_HD long int8_row_bytes(int heads, int D) { return static_cast<long>(heads) * (4 + D); }

AFB_KVQ_HD long int4_row_bytes(long values) { return ((values + kInt4Group - 1) / kInt4Group) * kInt4GroupBytes; }

AFB_KVQ_HD long turbo3_base_bytes(int heads, int D) { return (static_cast<long>(heads) * D * 3 + 7) / 8; }

AFB_KVQ_HD long turbo3_sketch_bytes(int heads) { return (static_cast<long>(heads) * kTurbo3SketchBits + 7) / 8; }

// Bytes of one token's key row; 0 for a codec / head size that is not supported.
AFB_KVQ_HD long key_row_bytes(int codec, int heads, int D) {
  const long values = static_cast<long>(heads) * D;
  switch (codec) {
    case kBf16: return values * 2;
    case kFp8: return values;
    case kInt8: return int8_row_bytes(heads, D);
    case kInt4: return int4_row_bytes(values);
    case kPolar4: return head_dim_supported(D) ? (values + 1) / 2 : 0;
    case kTurbo3: return head_dim_supported(D) ? turbo3_base_bytes(heads, D) + turbo3_sketch_bytes(heads) : 0;
    default: return 0;
  }
}

AFB_KVQ_HD long value_row_bytes(int codec, int heads, int D) {
  if (codec == kPolar4 || codec == kTurbo3) return head_dim_supported(D) ? int8_row_bytes(heads, D) : 0;
  return key_row_bytes(codec, heads, D);
}

AFB_KVQ_HD float load_f32(const uint8_t* p) {
  return bits_to_float(static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) |
                       (static_cast<uint32_t>(p[2]) << 16) | (static_cast<uint32_t>(p[3]) << 24));
}

AFB_KVQ_HD float int8_elem(const uint8_t* row, int D, int head, int d) {
  const uint8_t* h = row + static_cast<long>(head) * (4 + D);
  return static_cast<float>(static_cast<int8_t>(h[4 + d])) * load_f32(h);
}

AFB_KVQ_HD float int4_elem(const uint8_t* row, long idx) {
  const uint8_t* g = row + (idx / kInt4Group) * kInt4GroupBytes;
  const int j = static_cast<int>(idx % kInt4Group);
  const float scale = half_to_float(static_cast<uint16_t>(g[0] | (static_cast<uint16_t>(g[1]) << 8)));
  const uint8_t b = g[2 + j / 2];
  int n = (j & 1) ? (b >> 4) : (b & 0xF);
  if (n & 8) n -= 16;
  return static_cast<float>(n) * scale;
}

AFB_KVQ_HD int packed3_get(const uint8_t* src, long idx) {
  const long bit = idx * 3;
  const long byte = bit >> 3;
  const int shift = static_cast<int>(bit & 7);
  uint32_t bits = static_cast<uint32_t>(src[byte]) >> shift;
  if (shift > 5) bits |= static_cast<uint32_t>(src[byte + 1]) << (8 - shift);
  return static_cast<int>(bits & 7u);
}

AFB_KVQ_HD float polar4_value(int code) { return static_cast<float>(code & 15) / 7.5f - 1.0f; }

AFB_KVQ_HD float turbo3_value(int code) { return static_cast<float>(code & 7) / 3.5f - 1.0f; }

// Element d of head `head` of a key row (for turbo3: the 3-bit base value, without the sketch correction).
AFB_KVQ_HD float key_elem(int codec, const uint8_t* row, int heads, int D, int head, int d) {
  const long idx = static_cast<long>(head) * D + d;
  switch (codec) {
    case kBf16: return bf16_to_float(static_cast<uint16_t>(row[2 * idx] | (static_cast<uint16_t>(row[2 * idx + 1]) << 8)));
    case kFp8: return fp8_e4m3_to_float(row[idx]);
    case kInt8: return int8_elem(row, D, head, d);
    case kInt4: return int4_elem(row, idx);
    case kPolar4: {
      const uint8_t b = row[idx >> 1];
      return polar4_value((idx & 1) ? (b >> 4) : (b & 0xF));
    }
    case kTurbo3: return turbo3_value(packed3_get(row, idx));
    default: return 0.0f;
  }
  (void)heads;
}

AFB_KVQ_HD float value_elem(int codec, const uint8_t* row, int heads, int D, int head, int d) {
  if (codec == kPolar4 || codec == kTurbo3) return int8_elem(row, D, head, d);
  return key_elem(codec, row, heads, D, head, d);
}

// Pseudo-random sign of projection `projection` at dimension `dim` for KV head `head` (a 64-bit mix).
AFB_KVQ_HD float random_sign(uint64_t head, uint64_t projection, uint64_t dim) {
  uint64_t x = (head + 1) * 0x9e3779b97f4a7c15ull;
  x ^= (projection + 1) * 0xbf58476d1ce4e5b9ull;
  x ^= (dim + 1) * 0x94d049bb133111ebull;
  x ^= x >> 30;
  x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27;
  x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return (x & 1) ? -1.0f : 1.0f;
}

// Bit `projection` of head `head`'s residual sketch inside a turbo3 key row.
AFB_KVQ_HD bool turbo3_sketch_bit(const uint8_t* row, int heads, int D, int head, int projection) {
  const uint8_t* sk = row + turbo3_base_bytes(heads, D);
  const long bit = static_cast<long>(head) * kTurbo3SketchBits + projection;
  return (sk[bit >> 3] >> (bit & 7)) & 1;
}

// Score correction of a turbo3 key for a query whose 32 projections are `pq`: mean of sign * projection,
// times the fixed residual scale.
AFB_KVQ_HD float turbo3_residual_score(const float* pq, const uint8_t* row, int heads, int D, int head) {
  float acc = 0.0f;
  for (int p = 0; p < kTurbo3SketchBits; ++p) acc += turbo3_sketch_bit(row, heads, D, head, p) ? pq[p] : -pq[p];
  return kTurbo3ResidualScale * acc / static_cast<float>(kTurbo3SketchBits);
}

}  // namespace kvq
}  // namespace afb
