// CPU fp32 reference path, restated from the reference's native CPU maths (zig/lib/linalg/src/gemm.zig tiled
// SGEMM, attention.zig softmax attention, mod.zig:298-312 meanPool / l2Normalize, zig/lib/vector/src/vector.zig
// distance + top-k): a BERT-style post-LN encoder forward, masked mean pooling + L2 normalisation, and exact
// top-k search.  It is the timed CPU baseline of the plumbing benchmark and an independent oracle for the GPU
// pipeline (no PyTorch involved).  Threads split rows of the big loops; inner loops are written so the compiler
// vectorises them (-O3 -march=x86-64-v3).
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

namespace {

int g_threads = 0;

int n_threads() {
  if (g_threads > 0) return g_threads;
  unsigned h = std::thread::hardware_concurrency();
  return h ? static_cast<int>(h) : 4;
}

template <class F>
void parallel_rows(int rows, F fn) {
  const int nt = std::min(n_threads(), std::max(rows, 1));
  if (nt <= 1) { fn(0, rows); return; }
  std::vector<std::thread> th;
  const int per = (rows + nt - 1) / nt;
  for (int t = 0; t < nt; ++t) {
    const int lo = t * per, hi = std::min(rows, lo + per);
    if (lo >= hi) break;
    th.emplace_back([=] { fn(lo, hi); });
  }
  for (auto& t : th) t.join();
}

// y[m, n] = sum_k x[m, k] * w[n, k] + b[n]; 4x4 register tile over (m, n), k innermost and contiguous in both.
void linear(const float* x, const float* w, const float* b, float* y, int M, int N, int K) {
  parallel_rows(M, [&](int lo, int hi) {
    for (int m = lo; m < hi; m += 4) {
      const int mm = std::min(4, hi - m);
      for (int n = 0; n < N; n += 4) {
        const int nn = std::min(4, N - n);
        float acc[4][4] = {{0}};
        for (int i = 0; i < mm; ++i)
          for (int j = 0; j < nn; ++j) {
            const float* xr = x + static_cast<size_t>(m + i) * K;
            const float* wr = w + static_cast<size_t>(n + j) * K;
            float s = 0;
#pragma omp simd reduction(+ : s)
            for (int k = 0; k < K; ++k) s += xr[k] * wr[k];
            acc[i][j] = s;
          }
        for (int i = 0; i < mm; ++i)
          for (int j = 0; j < nn; ++j) y[static_cast<size_t>(m + i) * N + n + j] = acc[i][j] + (b ? b[n + j] : 0.0f);
      }
    }
  });
}

void layer_norm(float* x, const float* g, const float* b, int rows, int H, float eps) {
  parallel_rows(rows, [&](int lo, int hi) {
    for (int r = lo; r < hi; ++r) {
      float* v = x + static_cast<size_t>(r) * H;
      float mean = 0;
      for (int i = 0; i < H; ++i) mean += v[i];
      mean /= H;
      float var = 0;
      for (int i = 0; i < H; ++i) { const float d = v[i] - mean; var += d * d; }
      const float rstd = 1.0f / sqrtf(var / H + eps);
      for (int i = 0; i < H; ++i) v[i] = (v[i] - mean) * rstd * g[i] + b[i];
    }
  });
}

inline float gelu(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

struct Layer {
  const float *qkv_w, *qkv_b, *o_w, *o_b, *ln1_g, *ln1_b, *ff1_w, *ff1_b, *ff2_w, *ff2_b, *ln2_g, *ln2_b;
};

}  // namespace

extern "C" {

void afb_cpu_set_threads(int n) { g_threads = n; }

// Weights arrive as one array of pointers: [word, pos, type, emb_ln_g, emb_ln_b, then 12 pointers per layer in the
// order of struct Layer].  ids/type_ids/mask are [B, S] (mask > 0 = real token).  out: [B, H] pooled, L2-normalised.
int afb_cpu_bert_embed(const float* const* w, int n_layers, int H, int heads, int F, float eps, const int* ids,
                       const int* type_ids, const int* mask, int B, int S, float* out) {
  const int T = B * S, D = H / heads;
  std::vector<float> x(static_cast<size_t>(T) * H), qkv(static_cast<size_t>(T) * 3 * H), ctx(static_cast<size_t>(T) * H),
      tmp(static_cast<size_t>(T) * H), ff(static_cast<size_t>(T) * F);
  const float *word = w[0], *pos = w[1], *type = w[2];
  for (int t = 0; t < T; ++t) {
    const int s = t % S, ty = type_ids ? type_ids[t] : 0;
    for (int i = 0; i < H; ++i)
      x[static_cast<size_t>(t) * H + i] = word[static_cast<size_t>(ids[t]) * H + i] + pos[static_cast<size_t>(s) * H + i] +
                                          type[static_cast<size_t>(ty) * H + i];
  }
  layer_norm(x.data(), w[3], w[4], T, H, eps);
  const float scale = 1.0f / sqrtf(static_cast<float>(D));
  for (int l = 0; l < n_layers; ++l) {
    Layer L;
    memcpy(&L, w + 5 + l * 12, sizeof(Layer));
    linear(x.data(), L.qkv_w, L.qkv_b, qkv.data(), T, 3 * H, H);
    parallel_rows(B * heads, [&](int lo, int hi) {
      std::vector<float> sc(S);
      for (int bh = lo; bh < hi; ++bh) {
        const int b = bh / heads, h = bh % heads;
        for (int i = 0; i < S; ++i) {
          const float* q = &qkv[(static_cast<size_t>(b) * S + i) * 3 * H + h * D];
          float mx = -INFINITY;
          for (int j = 0; j < S; ++j) {
            if (mask && mask[b * S + j] <= 0) { sc[j] = -INFINITY; continue; }
            const float* k = &qkv[(static_cast<size_t>(b) * S + j) * 3 * H + H + h * D];
            float s = 0;
#pragma omp simd reduction(+ : s)
            for (int d = 0; d < D; ++d) s += q[d] * k[d];
            sc[j] = s * scale;
            mx = fmaxf(mx, sc[j]);
          }
          float den = 0;
          for (int j = 0; j < S; ++j) { sc[j] = (sc[j] == -INFINITY) ? 0.0f : expf(sc[j] - mx); den += sc[j]; }
          float* o = &ctx[(static_cast<size_t>(b) * S + i) * H + h * D];
          for (int d = 0; d < D; ++d) o[d] = 0;
          for (int j = 0; j < S; ++j) {
            if (sc[j] == 0.0f) continue;
            const float p = sc[j] / den;
            const float* v = &qkv[(static_cast<size_t>(b) * S + j) * 3 * H + 2 * H + h * D];
#pragma omp simd
            for (int d = 0; d < D; ++d) o[d] += p * v[d];
          }
        }
      }
    });
    linear(ctx.data(), L.o_w, L.o_b, tmp.data(), T, H, H);
    for (size_t i = 0; i < tmp.size(); ++i) x[i] += tmp[i];
    layer_norm(x.data(), L.ln1_g, L.ln1_b, T, H, eps);
    linear(x.data(), L.ff1_w, L.ff1_b, ff.data(), T, F, H);
    parallel_rows(T, [&](int lo, int hi) {
      for (size_t i = static_cast<size_t>(lo) * F; i < static_cast<size_t>(hi) * F; ++i) ff[i] = gelu(ff[i]);
    });
    linear(ff.data(), L.ff2_w, L.ff2_b, tmp.data(), T, H, F);
    for (size_t i = 0; i < tmp.size(); ++i) x[i] += tmp[i];
    layer_norm(x.data(), L.ln2_g, L.ln2_b, T, H, eps);
  }
  for (int b = 0; b < B; ++b) {
    float* o = out + static_cast<size_t>(b) * H;
    for (int i = 0; i < H; ++i) o[i] = 0;
    int cnt = 0;
    for (int s = 0; s < S; ++s) {
      if (mask && mask[b * S + s] <= 0) continue;
      ++cnt;
      for (int i = 0; i < H; ++i) o[i] += x[(static_cast<size_t>(b) * S + s) * H + i];
    }
    float ss = 0;
    for (int i = 0; i < H; ++i) { if (cnt) o[i] /= cnt; ss += o[i] * o[i]; }
    const float inv = ss > 0 ? 1.0f / sqrtf(ss) : 0.0f;
    for (int i = 0; i < H; ++i) o[i] *= inv;
  }
  return 0;
}

// Exact top-k.  metric: 0 l2_squared, 1 inner_product, 2 cosine (lower is closer).  out_idx / out_dist: [Q, k].
int afb_cpu_topk(const float* q, const float* x, int Q, long N, int D, int k, int metric, int* out_idx,
                 float* out_dist) {
  std::vector<float> xn(N);
  parallel_rows(static_cast<int>(N), [&](int lo, int hi) {
    for (long n = lo; n < hi; ++n) {
      float s = 0;
      const float* r = x + n * D;
      for (int d = 0; d < D; ++d) s += r[d] * r[d];
      xn[n] = s;
    }
  });
  parallel_rows(Q, [&](int lo, int hi) {
    std::vector<std::pair<float, int>> heap;
    for (int qi = lo; qi < hi; ++qi) {
      const float* qv = q + static_cast<size_t>(qi) * D;
      float qn = 0;
      for (int d = 0; d < D; ++d) qn += qv[d] * qv[d];
      heap.clear();
      for (long n = 0; n < N; ++n) {
        const float* r = x + n * D;
        float dot = 0;
#pragma omp simd reduction(+ : dot)
        for (int d = 0; d < D; ++d) dot += qv[d] * r[d];
        float dist;
        if (metric == 0) dist = fmaxf(0.0f, qn + xn[n] - 2.0f * dot);
        else if (metric == 1) dist = -dot;
        else { const float den = sqrtf(qn) * sqrtf(xn[n]); dist = den > 0 ? 1.0f - dot / den : 1.0f; }
        if (static_cast<int>(heap.size()) < k) {
          heap.emplace_back(dist, static_cast<int>(n));
          std::push_heap(heap.begin(), heap.end());
        } else if (dist < heap.front().first) {
          std::pop_heap(heap.begin(), heap.end());
          heap.back() = {dist, static_cast<int>(n)};
          std::push_heap(heap.begin(), heap.end());
        }
      }
      std::sort_heap(heap.begin(), heap.end());
      for (int i = 0; i < k; ++i) {
        const bool ok = i < static_cast<int>(heap.size());
        out_idx[static_cast<size_t>(qi) * k + i] = ok ? heap[i].second : -1;
        out_dist[static_cast<size_t>(qi) * k + i] = ok ? heap[i].first : INFINITY;
      }
    }
  });
  return 0;
}

}  // extern "C"
