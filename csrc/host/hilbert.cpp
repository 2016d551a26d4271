// Hilbert-curve keys for float vectors (bulk index builds sort by them so that leaves hold nearby vectors).
// The key of a vector is the Hilbert index of the point whose integer coordinates are the raw IEEE-754 bit patterns
// of its components (32 bits per dimension), written most significant bit first: 4 * dims bytes that compare
// lexicographically in curve order.  The axes -> transposed-index step is Skilling's in-place transform
// ("Programming the Hilbert curve", 2004); the layout matches the reference's zig/lib/vector/src/vector.zig:42-140
// (bit `b` of every coordinate, most significant first, coordinates in order).
#include <stdint.h>
#include <string.h>

#include <vector>

namespace {

void axes_to_transpose(uint32_t* x, int n) {
  const uint32_t m = 1u << 31;
  for (uint32_t q = m; q > 1; q >>= 1) {  // inverse undo of the excess work
    const uint32_t p = q - 1;
    for (int i = 0; i < n; ++i) {
      if (x[i] & q) {
        x[0] ^= p;
      } else {
        const uint32_t t = (x[0] ^ x[i]) & p;
        x[0] ^= t;
        x[i] ^= t;
      }
    }
  }
  for (int i = 1; i < n; ++i) x[i] ^= x[i - 1];  // Gray encode
  uint32_t t = 0;
  for (uint32_t q = m; q > 1; q >>= 1)
    if (x[n - 1] & q) t ^= q - 1;
  for (int i = 0; i < n; ++i) x[i] ^= t;
}

}  // namespace

extern "C" {

// vectors: [n, dims] fp32; keys: [n, 4 * dims] bytes.  Returns 0, or -1 for bad arguments.
int afb_hilbert_keys(const float* vectors, long n, int dims, uint8_t* keys) {
  if (!vectors || !keys || n < 0 || dims <= 0) return -1;
  const int key_len = 4 * dims;
  std::vector<uint32_t> x(dims);
  for (long r = 0; r < n; ++r) {
    memcpy(x.data(), vectors + r * dims, sizeof(uint32_t) * dims);
    axes_to_transpose(x.data(), dims);
    uint8_t* out = keys + r * key_len;
    memset(out, 0, key_len);
    // bit plane by bit plane (most significant first), coordinates in order: output bit index counts from the front
    long bit_out = 0;
    for (int b = 31; b >= 0; --b) {
      for (int i = 0; i < dims; ++i, ++bit_out) {
        if ((x[i] >> b) & 1u) out[bit_out >> 3] |= static_cast<uint8_t>(0x80u >> (bit_out & 7));
      }
    }
  }
  return 0;
}

}  // extern "C"
