// GGUF block quantisers for the export tool: Q4_1, Q5_0, Q5_1, Q8_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_K (Q4_0 and Q8_0
// live with the decoders in codecs.cpp).  Each is the inverse of the block decoder of the same type in codecs.cpp, so
// the layouts are stated there; what is decided here is only how scales are chosen:
//
//   * asymmetric types (x = d * q + m or x = d * sc * q - dmin * mn): the range [min(x, 0) .. max(x)] of a (sub-)block
//     is spread over the code range; the K-quants then quantise the sub-block scales and offsets themselves (6 or 4
//     bits against a per-super-block fp16 d / dmin) and RE-QUANTISE the values against the scales as they will be
//     decoded, so the rounding of the scales does not add to the rounding of the values;
//   * symmetric types (x = d * sc * (q - bias)): the sub-block scale follows the value of largest magnitude, signed,
//     so that it lands on the most negative code and the full range is used.
//
// The reference's exporter offers the same set (zig/pkg/inference/src/native_export_gguf.zig:4814 --format list;
// quantisers in zig/pkg/inference/src/gguf/quant_codec.zig:586-1260).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>

extern "C" int afb_gguf_quantize_q8_0(const float* src, uint8_t* dst, long n_values);
extern "C" int afb_gguf_quantize_q4_0(const float* src, uint8_t* dst, long n_values);

namespace {

uint16_t to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return static_cast<uint16_t>(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (h & 1))) ++h;
    return static_cast<uint16_t>(sign | h);
  }
  uint32_t h = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return static_cast<uint16_t>(sign | h);
}

float from_half(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FFu, out;
  if (exp == 0) {
    if (man == 0) {
      out = sign;
    } else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      out = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    out = sign | 0x7F800000u | (man << 13);
  } else {
    out = sign | ((exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

// the value an fp16 field will read back as
float half_round(float f, uint16_t* bits) {
  *bits = to_half(f);
  return from_half(*bits);
}

int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
int nearest(float v) { return static_cast<int>(lrintf(v)); }

// range of a run of values with the minimum not above zero (offsets are stored unsigned)
void range_of(const float* x, int n, float* lo, float* hi) {
  float a = 0.0f, b = x[0];
  for (int i = 0; i < n; ++i) {
    a = std::min(a, x[i]);
    b = std::max(b, x[i]);
  }
  *lo = a;
  *hi = std::max(b, a);
}

void put_half(uint8_t* p, uint16_t h) { std::memcpy(p, &h, 2); }

// ---- 32-value blocks with an fp16 scale (and offset) ---------------------------------------------------------
void q4_1_block(const float* x, uint8_t* p) {
  float lo = x[0], hi = x[0];
  for (int i = 1; i < 32; ++i) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); }
  uint16_t dh, mh;
  const float d = half_round((hi - lo) / 15.0f, &dh), m = half_round(lo, &mh);
  const float id = d > 0 ? 1.0f / d : 0.0f;
  put_half(p, dh); put_half(p + 2, mh);
  for (int j = 0; j < 16; ++j) {
    const int a = clampi(nearest((x[j] - m) * id), 0, 15), b = clampi(nearest((x[j + 16] - m) * id), 0, 15);
    p[4 + j] = static_cast<uint8_t>(a | (b << 4));
  }
}

void q5_block(const float* x, uint8_t* p, bool with_min) {
  uint16_t dh, mh = 0;
  float d, m = 0.0f;
  if (with_min) {
    float lo = x[0], hi = x[0];
    for (int i = 1; i < 32; ++i) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); }
    d = half_round((hi - lo) / 31.0f, &dh);
    m = half_round(lo, &mh);
  } else {
    float amax = 0.0f, mx = 0.0f;
    for (int i = 0; i < 32; ++i) if (std::fabs(x[i]) > amax) { amax = std::fabs(x[i]); mx = x[i]; }
    d = half_round(mx / -16.0f, &dh);
  }
  const float id = d != 0 ? 1.0f / d : 0.0f;
  uint32_t qh = 0;
  uint8_t* q = p + (with_min ? 8 : 6);
  for (int j = 0; j < 16; ++j) {
    int a, b;
    if (with_min) {
      a = clampi(nearest((x[j] - m) * id), 0, 31);
      b = clampi(nearest((x[j + 16] - m) * id), 0, 31);
    } else {
      a = clampi(static_cast<int>(x[j] * id + 16.5f), 0, 31);
      b = clampi(static_cast<int>(x[j + 16] * id + 16.5f), 0, 31);
    }
    q[j] = static_cast<uint8_t>((a & 0xF) | ((b & 0xF) << 4));
    qh |= static_cast<uint32_t>(a >> 4) << j;
    qh |= static_cast<uint32_t>(b >> 4) << (j + 16);
  }
  put_half(p, dh);
  if (with_min) put_half(p + 2, mh);
  std::memcpy(p + (with_min ? 4 : 2), &qh, 4);
}

void q8_1_block(const float* x, uint8_t* p) {       // fp16 d, fp16 s = d * sum(q), 32 int8
  float amax = 0.0f;
  for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[i]));
  uint16_t dh, sh;
  const float d = half_round(amax / 127.0f, &dh), id = d > 0 ? 1.0f / d : 0.0f;
  int sum = 0;
  for (int i = 0; i < 32; ++i) {
    const int q = clampi(nearest(x[i] * id), -127, 127);
    reinterpret_cast<int8_t*>(p + 4)[i] = static_cast<int8_t>(q);
    sum += q;
  }
  half_round(d * static_cast<float>(sum), &sh);
  put_half(p, dh); put_half(p + 2, sh);
}

// ---- K-quants: 256-value super-blocks --------------------------------------------------------------------------
// eight 6-bit (scale, offset) pairs in 12 bytes, the packing q4k_scale_min reads
void pack_scales_k4(const uint8_t* sc, const uint8_t* mn, uint8_t* out) {
  for (int j = 0; j < 4; ++j) {
    out[j] = static_cast<uint8_t>((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
    out[j + 4] = static_cast<uint8_t>((mn[j] & 63) | ((mn[j + 4] >> 4) << 6));
    out[j + 8] = static_cast<uint8_t>((sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4));
  }
}

// Q4_K (bits = 4) and Q5_K (bits = 5): x = d * sc * q - dmin * mn per 32-value sub-block
void q45_k_block(const float* x, uint8_t* p, int bits) {
  const int qmax = (1 << bits) - 1;
  float scale[8], off[8];
  float max_scale = 0.0f, max_off = 0.0f;
  for (int s = 0; s < 8; ++s) {
    float lo, hi;
    range_of(x + 32 * s, 32, &lo, &hi);
    scale[s] = (hi - lo) / static_cast<float>(qmax);
    off[s] = -lo;
    max_scale = std::max(max_scale, scale[s]);
    max_off = std::max(max_off, off[s]);
  }
  uint16_t dh, mh;
  const float d = half_round(max_scale / 63.0f, &dh), dmin = half_round(max_off / 63.0f, &mh);
  const float id = d > 0 ? 1.0f / d : 0.0f, imin = dmin > 0 ? 1.0f / dmin : 0.0f;
  uint8_t sc[8], mn[8];
  for (int s = 0; s < 8; ++s) {
    sc[s] = static_cast<uint8_t>(clampi(nearest(scale[s] * id), 0, 63));
    mn[s] = static_cast<uint8_t>(clampi(nearest(off[s] * imin), 0, 63));
  }
  put_half(p, dh); put_half(p + 2, mh);
  pack_scales_k4(sc, mn, p + 4);
  uint8_t* qh = bits == 5 ? p + 16 : nullptr;
  uint8_t* ql = p + (bits == 5 ? 48 : 16);
  if (qh) std::memset(qh, 0, 32);
  int q[256];
  for (int s = 0; s < 8; ++s) {
    const float ds = d * sc[s], ms = dmin * mn[s], ids = ds > 0 ? 1.0f / ds : 0.0f;
    for (int l = 0; l < 32; ++l) q[32 * s + l] = clampi(nearest((x[32 * s + l] + ms) * ids), 0, qmax);
  }
  for (int pair = 0; pair < 4; ++pair) {          // sub-blocks 2 * pair (low nibbles) and 2 * pair + 1 (high nibbles)
    for (int l = 0; l < 32; ++l) {
      const int a = q[64 * pair + l], b = q[64 * pair + 32 + l];
      ql[32 * pair + l] = static_cast<uint8_t>((a & 0xF) | ((b & 0xF) << 4));
      if (qh) {
        if (a >> 4) qh[l] |= static_cast<uint8_t>(1u << (2 * pair));
        if (b >> 4) qh[l] |= static_cast<uint8_t>(2u << (2 * pair));
      }
    }
  }
}

// Q6_K: x = d * sc * (q - 32), int8 scale per 16 values, q in 0..63
void q6_k_block(const float* x, uint8_t* p) {
  float s[16], max_abs = 0.0f;
  for (int j = 0; j < 16; ++j) {
    float amax = 0.0f, mx = 0.0f;
    for (int l = 0; l < 16; ++l) if (std::fabs(x[16 * j + l]) > amax) { amax = std::fabs(x[16 * j + l]); mx = x[16 * j + l]; }
    s[j] = mx / -32.0f;                                  // the largest value lands on code 0 (= -32)
    max_abs = std::max(max_abs, std::fabs(s[j]));
  }
  uint16_t dh;
  const float d = half_round(max_abs / 127.0f, &dh), id = d > 0 ? 1.0f / d : 0.0f;
  int8_t* scales = reinterpret_cast<int8_t*>(p + 192);
  int q[256];
  for (int j = 0; j < 16; ++j) {
    scales[j] = static_cast<int8_t>(clampi(nearest(s[j] * id), -128, 127));
    const float ds = d * scales[j], ids = ds != 0 ? 1.0f / ds : 0.0f;
    for (int l = 0; l < 16; ++l) q[16 * j + l] = clampi(nearest(x[16 * j + l] * ids) + 32, 0, 63);
  }
  put_half(p + 208, dh);
  uint8_t* ql = p;
  uint8_t* qh = p + 128;
  for (int n = 0; n < 2; ++n) {                   // halves of 128 values; within a half four runs of 32
    const int* v = q + 128 * n;
    for (int l = 0; l < 32; ++l) {
      const int q1 = v[l], q2 = v[l + 32], q3 = v[l + 64], q4 = v[l + 96];
      ql[64 * n + l] = static_cast<uint8_t>((q1 & 0xF) | ((q3 & 0xF) << 4));
      ql[64 * n + l + 32] = static_cast<uint8_t>((q2 & 0xF) | ((q4 & 0xF) << 4));
      qh[32 * n + l] = static_cast<uint8_t>((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
    }
  }
}

// Q2_K: x = d * (sc & 15) * q - dmin * (sc >> 4) per 16 values, q in 0..3
void q2_k_block(const float* x, uint8_t* p) {
  float scale[16], off[16], max_scale = 0.0f, max_off = 0.0f;
  for (int j = 0; j < 16; ++j) {
    float lo, hi;
    range_of(x + 16 * j, 16, &lo, &hi);
    scale[j] = (hi - lo) / 3.0f;
    off[j] = -lo;
    max_scale = std::max(max_scale, scale[j]);
    max_off = std::max(max_off, off[j]);
  }
  uint16_t dh, mh;
  const float d = half_round(max_scale / 15.0f, &dh), dmin = half_round(max_off / 15.0f, &mh);
  const float id = d > 0 ? 1.0f / d : 0.0f, imin = dmin > 0 ? 1.0f / dmin : 0.0f;
  uint8_t* scales = p;
  uint8_t* qs = p + 16;
  std::memset(qs, 0, 64);
  put_half(p + 80, dh); put_half(p + 82, mh);
  int q[256];
  for (int j = 0; j < 16; ++j) {
    const int sc = clampi(nearest(scale[j] * id), 0, 15), mn = clampi(nearest(off[j] * imin), 0, 15);
    scales[j] = static_cast<uint8_t>(sc | (mn << 4));
    const float ds = d * sc, ms = dmin * mn, ids = ds > 0 ? 1.0f / ds : 0.0f;
    for (int l = 0; l < 16; ++l) q[16 * j + l] = clampi(nearest((x[16 * j + l] + ms) * ids), 0, 3);
  }
  // decoder order: for each half of 128: shift 0, 2, 4, 6; within a shift two runs of 16 (bytes l and l + 16)
  int is = 0;
  for (int n = 0; n < 2; ++n)
    for (int shift = 0; shift < 8; shift += 2)
      for (int half = 0; half < 2; ++half, ++is)
        for (int l = 0; l < 16; ++l) qs[32 * n + l + 16 * half] |= static_cast<uint8_t>(q[16 * is + l] << shift);
}

// Q3_K: x = d * (sc - 32) * (q - 4), six-bit scale per 16 values, q in 0..7 (two low bits + one high bit)
void q3_k_block(const float* x, uint8_t* p) {
  float s[16], max_abs = 0.0f;
  for (int j = 0; j < 16; ++j) {
    float amax = 0.0f, mx = 0.0f;
    for (int l = 0; l < 16; ++l) if (std::fabs(x[16 * j + l]) > amax) { amax = std::fabs(x[16 * j + l]); mx = x[16 * j + l]; }
    s[j] = mx / -4.0f;
    max_abs = std::max(max_abs, std::fabs(s[j]));
  }
  uint16_t dh;
  const float d = half_round(max_abs / 31.0f, &dh), id = d > 0 ? 1.0f / d : 0.0f;
  int sc[16], q[256];
  for (int j = 0; j < 16; ++j) {
    sc[j] = clampi(nearest(s[j] * id), -32, 31);
    const float ds = d * sc[j], ids = ds != 0 ? 1.0f / ds : 0.0f;
    for (int l = 0; l < 16; ++l) q[16 * j + l] = clampi(nearest(x[16 * j + l] * ids) + 4, 0, 7);
  }
  uint8_t* hm = p;
  uint8_t* qs = p + 32;
  std::memset(p, 0, 96);
  // scales: value + 32 in six bits; low nibbles in bytes 0..7 (j and j + 8), the two high bits of scale j in byte
  // 8 + j % 4 at bit pair j / 4 -- the layout the decoder unpacks through its four 32-bit words
  uint8_t* sb = p + 96;
  std::memset(sb, 0, 12);
  for (int j = 0; j < 16; ++j) {
    const int v = sc[j] + 32;
    if (j < 8) sb[j] |= static_cast<uint8_t>(v & 0xF);
    else sb[j - 8] |= static_cast<uint8_t>((v & 0xF) << 4);
    sb[8 + j % 4] |= static_cast<uint8_t>((v >> 4) << (2 * (j / 4)));
  }
  put_half(p + 108, dh);
  int is = 0;
  uint8_t m = 1;
  for (int n = 0; n < 2; ++n) {
    for (int shift = 0; shift < 8; shift += 2) {
      for (int half = 0; half < 2; ++half, ++is)
        for (int l = 0; l < 16; ++l) {
          const int v = q[16 * is + l];
          qs[32 * n + l + 16 * half] |= static_cast<uint8_t>((v & 3) << shift);
          if (v & 4) hm[l + 16 * half] |= m;
        }
      m = static_cast<uint8_t>(m << 1);
    }
  }
}

// Q8_K: fp32 d, 256 int8, 16 int16 sums of 16
void q8_k_block(const float* x, uint8_t* p) {
  float amax = 0.0f, mx = 0.0f;
  for (int i = 0; i < 256; ++i) if (std::fabs(x[i]) > amax) { amax = std::fabs(x[i]); mx = x[i]; }
  const float iscale = amax > 0 ? -128.0f / mx : 0.0f, d = amax > 0 ? 1.0f / iscale : 0.0f;
  std::memcpy(p, &d, 4);
  int8_t* q = reinterpret_cast<int8_t*>(p + 4);
  for (int i = 0; i < 256; ++i) q[i] = static_cast<int8_t>(clampi(nearest(iscale * x[i]), -128, 127));
  for (int j = 0; j < 16; ++j) {
    int16_t sum = 0;
    for (int l = 0; l < 16; ++l) sum = static_cast<int16_t>(sum + q[16 * j + l]);
    std::memcpy(p + 4 + 256 + 2 * j, &sum, 2);
  }
}

}  // namespace

extern "C" {

// Quantise n_values fp32 values (a multiple of the type's block length) into `type` (ggml numbering).  Returns 0,
// -1 for a type without a quantiser here, -2 when n_values is not a whole number of blocks.
int afb_gguf_quantize(int type, const float* src, uint8_t* dst, long n_values) {
  struct Geo { int values, bytes; };
  Geo g;
  switch (type) {
    case 2: g = {32, 18}; break;
    case 3: g = {32, 20}; break;
    case 6: g = {32, 22}; break;
    case 7: g = {32, 24}; break;
    case 8: g = {32, 34}; break;
    case 9: g = {32, 36}; break;
    case 10: g = {256, 84}; break;
    case 11: g = {256, 110}; break;
    case 12: g = {256, 144}; break;
    case 13: g = {256, 176}; break;
    case 14: g = {256, 210}; break;
    case 15: g = {256, 292}; break;
    default: return -1;
  }
  if (n_values % g.values) return -2;
  if (type == 2) return afb_gguf_quantize_q4_0(src, dst, n_values);
  if (type == 8) return afb_gguf_quantize_q8_0(src, dst, n_values);
  for (long b = 0; b < n_values / g.values; ++b) {
    const float* x = src + b * g.values;
    uint8_t* p = dst + b * g.bytes;
    switch (type) {
      case 3: q4_1_block(x, p); break;
      case 6: q5_block(x, p, false); break;
      case 7: q5_block(x, p, true); break;
      case 9: q8_1_block(x, p); break;
      case 10: q2_k_block(x, p); break;
      case 11: q3_k_block(x, p); break;
      case 12: q45_k_block(x, p, 4); break;
      case 13: q45_k_block(x, p, 5); break;
      case 14: q6_k_block(x, p); break;
      case 15: q8_k_block(x, p); break;
    }
  }
  return 0;
}

}  // extern "C"
