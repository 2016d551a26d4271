// Host side of the quantised KV-cache codecs: row encoders, row decoders, and a decode attention that scores a query
// straight against the compressed key rows (no dequantised key buffer) and dequantises values as it reads them.
//
// Formats and the element accessors are in csrc/common/kvq_elem.h (shared with the CUDA kernel); this file adds
// what only the writer needs: choosing scales and packing codes.  Behaviour follows the reference's KV pool and key
// codecs (zig/pkg/inference/src/runtime/kv/pool.zig:351-530, 704-885; runtime/kv/turboquant.zig:47-204) and its
// compressed-key attention loop (zig/pkg/inference/src/ops/native_compute.zig:35200-35240).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../common/kvq_elem.h"

namespace {

using namespace afb::kvq;

uint16_t float_to_half(float f) {
  const uint32_t u = float_to_bits(f);
  const uint16_t sign = static_cast<uint16_t>((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return sign | (a > 0x7F800000u ? 0x7E00 : 0x7C00);
  if (a >= 0x477FF000u) return sign | 0x7C00;  // rounds to infinity
  if (a < 0x33000001u) return sign;            // below half of the smallest subnormal
  const int e = static_cast<int>(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) {  // subnormal half
    shift = 13 + (-14 - e);
    base = 0;
  } else {
    shift = 13;
    base = static_cast<uint32_t>(e + 15) << 10;
    m &= 0x7FFFFFu;
  }
  uint32_t keep = m >> shift;
  const uint32_t rest = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rest > half || (rest == half && (keep & 1u))) ++keep;
  return sign | static_cast<uint16_t>(base + keep);  // a mantissa carry moves into the exponent correctly
}

uint16_t float_to_bf16(float f) {
  uint32_t u = float_to_bits(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

void encode_int8(const float* src, uint8_t* dst, int heads, int D) {
  for (int h = 0; h < heads; ++h) {
    const float* x = src + static_cast<long>(h) * D;
    float mx = 0.0f;
    for (int d = 0; d < D; ++d) mx = std::max(mx, std::fabs(x[d]));
    const float scale = mx == 0.0f ? 1.0f : mx / 127.0f;
    uint8_t* o = dst + static_cast<long>(h) * (4 + D);
    std::memcpy(o, &scale, 4);
    const float inv = 1.0f / scale;
    for (int d = 0; d < D; ++d) {
      const float r = std::round(x[d] * inv);
      o[4 + d] = static_cast<uint8_t>(static_cast<int8_t>(std::min(127.0f, std::max(-127.0f, r))));
    }
  }
}

void encode_int4(const float* src, uint8_t* dst, long values) {
  for (long g0 = 0; g0 < values; g0 += kInt4Group) {
    const long n = std::min<long>(kInt4Group, values - g0);
    float mx = 0.0f;
    for (long i = 0; i < n; ++i) mx = std::max(mx, std::fabs(src[g0 + i]));
    const uint16_t hs = float_to_half(mx == 0.0f ? 1.0f : mx / 7.0f);
    uint8_t* o = dst + (g0 / kInt4Group) * kInt4GroupBytes;
    o[0] = static_cast<uint8_t>(hs & 0xFF);
    o[1] = static_cast<uint8_t>(hs >> 8);
    const float inv = 1.0f / half_to_float(hs);
    for (int i = 0; i < kInt4Group; i += 2) {
      auto code = [&](long j) -> uint8_t {
        if (j >= n) return 0;
        const float r = std::min(7.0f, std::max(-7.0f, std::round(src[g0 + j] * inv)));
        return static_cast<uint8_t>(static_cast<int8_t>(r)) & 0xF;
      };
      o[2 + i / 2] = static_cast<uint8_t>(code(i) | (code(i + 1) << 4));
    }
  }
}

inline int grid_code(float v, float half_levels, int max_code) {
  const float c = std::min(1.0f, std::max(-1.0f, v));
  // round half away from zero on a non-negative argument = floor(x + 0.5)
  const int q = static_cast<int>(std::floor((c + 1.0f) * half_levels + 0.5f));
  return std::min(max_code, std::max(0, q));
}

void encode_polar4(const float* src, uint8_t* dst, long values) {
  for (long i = 0; i < values; i += 2) {
    const int lo = grid_code(src[i], 7.5f, 15);
    const int hi = i + 1 < values ? grid_code(src[i + 1], 7.5f, 15) : 0;
    dst[i / 2] = static_cast<uint8_t>(lo | (hi << 4));
  }
}

void packed3_set(uint8_t* dst, long idx, int code) {
  const long bit = idx * 3, byte = bit >> 3;
  const int shift = static_cast<int>(bit & 7);
  const uint32_t bits = static_cast<uint32_t>(code & 7) << shift;
  dst[byte] |= static_cast<uint8_t>(bits & 0xFF);
  if (shift > 5) dst[byte + 1] |= static_cast<uint8_t>(bits >> 8);
}

void encode_turbo3(const float* src, uint8_t* dst, int heads, int D) {
  const long values = static_cast<long>(heads) * D;
  const long base = turbo3_base_bytes(heads, D), sk = turbo3_sketch_bytes(heads);
  std::memset(dst, 0, static_cast<size_t>(base + sk));
  for (long i = 0; i < values; ++i) packed3_set(dst, i, grid_code(src[i], 3.5f, 7));
  uint8_t* sketch = dst + base;
  for (int h = 0; h < heads; ++h) {
    for (int p = 0; p < kTurbo3SketchBits; ++p) {
      float acc = 0.0f;
      for (int d = 0; d < D; ++d) {
        const long i = static_cast<long>(h) * D + d;
        acc += random_sign(h, p, d) * (src[i] - turbo3_value(packed3_get(dst, i)));
      }
      if (acc >= 0.0f) {
        const long bit = static_cast<long>(h) * kTurbo3SketchBits + p;
        sketch[bit >> 3] |= static_cast<uint8_t>(1u << (bit & 7));
      }
    }
  }
}

}  // namespace

extern "C" {

long afb_kvq_row_bytes(int codec, int heads, int D, int is_value) {
  return is_value ? value_row_bytes(codec, heads, D) : key_row_bytes(codec, heads, D);
}

// src: [n_rows, heads * D] fp32; dst: n_rows rows of afb_kvq_row_bytes bytes.
int afb_kvq_encode_rows(int codec, int is_value, const float* src, uint8_t* dst, long n_rows, int heads, int D) {
  const long rb = afb_kvq_row_bytes(codec, heads, D, is_value);
  if (rb <= 0) return -1;
  const long values = static_cast<long>(heads) * D;
  const int eff = (is_value && (codec == kPolar4 || codec == kTurbo3)) ? static_cast<int>(kInt8) : codec;
  for (long r = 0; r < n_rows; ++r) {
    const float* x = src + r * values;
    uint8_t* o = dst + r * rb;
    switch (eff) {
      case kBf16:
        for (long i = 0; i < values; ++i) {
          const uint16_t h = float_to_bf16(x[i]);
          o[2 * i] = static_cast<uint8_t>(h & 0xFF);
          o[2 * i + 1] = static_cast<uint8_t>(h >> 8);
        }
        break;
      case kFp8:
        for (long i = 0; i < values; ++i) o[i] = float_to_fp8_e4m3(x[i]);
        break;
      case kInt8: encode_int8(x, o, heads, D); break;
      case kInt4: encode_int4(x, o, values); break;
      case kPolar4: encode_polar4(x, o, values); break;
      case kTurbo3: encode_turbo3(x, o, heads, D); break;
      default: return -1;
    }
  }
  return 0;
}

int afb_kvq_decode_rows(int codec, int is_value, const uint8_t* src, float* dst, long n_rows, int heads, int D) {
  const long rb = afb_kvq_row_bytes(codec, heads, D, is_value);
  if (rb <= 0) return -1;
  for (long r = 0; r < n_rows; ++r)
    for (int h = 0; h < heads; ++h)
      for (int d = 0; d < D; ++d)
        dst[(r * heads + h) * D + d] = is_value ? value_elem(codec, src + r * rb, heads, D, h, d)
                                                : key_elem(codec, src + r * rb, heads, D, h, d);
  return 0;
}

// The 32 sign projections of one query head for KV head `kv_head` (turbo3 residual scoring).
void afb_kvq_project_query(const float* q, int D, int kv_head, float* out32) {
  for (int p = 0; p < kTurbo3SketchBits; ++p) {
    float acc = 0.0f;
    for (int d = 0; d < D; ++d) acc += random_sign(kv_head, p, d) * q[d];
    out32[p] = acc;
  }
}

// One decode step of one sequence: q [Hq, D] fp32 against n_tokens cache rows (token-major), online softmax in
// fp32.  Keys at positions <= n_tokens - 1 - window are skipped when window > 0.  k_scale / v_scale multiply the
// decoded keys / values (per-tensor scales of an fp8 cache; 1 otherwise).
int afb_kvq_attention_host(int codec, const float* q, const uint8_t* k_rows, const uint8_t* v_rows, long n_tokens,
                           int Hq, int Hkv, int D, float scale, float k_scale, float v_scale, int window,
                           float* out) {
  const long krb = key_row_bytes(codec, Hkv, D), vrb = value_row_bytes(codec, Hkv, D);
  if (krb <= 0 || vrb <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  const int G = Hq / Hkv;
  const long t0 = window > 0 ? std::max<long>(0, n_tokens - window) : 0;
  std::vector<float> acc(D), pq(kTurbo3SketchBits);
  for (int hq = 0; hq < Hq; ++hq) {
    const int hk = hq / G;
    const float* qh = q + static_cast<long>(hq) * D;
    if (codec == kTurbo3) afb_kvq_project_query(qh, D, hk, pq.data());
    float m = -INFINITY, l = 0.0f;
    std::fill(acc.begin(), acc.end(), 0.0f);
    for (long t = t0; t < n_tokens; ++t) {
      const uint8_t* kr = k_rows + t * krb;
      float s = 0.0f;
      for (int d = 0; d < D; ++d) s += qh[d] * key_elem(codec, kr, Hkv, D, hk, d);
      if (codec == kTurbo3) s += turbo3_residual_score(pq.data(), kr, Hkv, D, hk);
      s *= scale * k_scale;
      const float m_new = std::max(m, s);
      const float alpha = std::exp(m - m_new), p = std::exp(s - m_new);
      l = l * alpha + p;
      const uint8_t* vr = v_rows + t * vrb;
      for (int d = 0; d < D; ++d) acc[d] = acc[d] * alpha + p * value_elem(codec, vr, Hkv, D, hk, d);
      m = m_new;
    }
    for (int d = 0; d < D; ++d) out[static_cast<long>(hq) * D + d] = l > 0.0f ? acc[d] * v_scale / l : 0.0f;
  }
  return 0;
}

}  // extern "C"
