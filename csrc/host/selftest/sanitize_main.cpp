// Stress driver for the host runtime, meant to be built with -fsanitize=address,undefined (memory errors, leaks,
// undefined behaviour) and with -fsanitize=thread (data races in the threaded paths).  It links the host sources
// directly and drives their C entry points with seeded random workloads; it checks a few invariants itself and
// leaves the rest to the sanitizer runtime.  Exit code 0 = clean.
//
// Usage: sanitize_main [asan|tsan] [seed]
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <random>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void* afb_kv_create(int num_blocks, int page);
void afb_kv_destroy(void* h);
int afb_kv_free_blocks(void* h);
int afb_kv_attach(void* h, int64_t seq);
int afb_kv_attach_shared(void* h, int64_t seq, int64_t parent, int prefix_tokens);
int afb_kv_take_cow(void* h, int* src, int* dst, int max);
int afb_kv_append(void* h, int64_t seq, int n_tokens, int* out_slots);
int afb_kv_truncate(void* h, int64_t seq, int new_len);
int afb_kv_trim_window(void* h, int64_t seq, int window);
int afb_kv_len(void* h, int64_t seq);
int afb_kv_block_table(void* h, int64_t seq, int* out, int max);
int afb_kv_detach(void* h, int64_t seq);
int afb_kv_refcount(void* h, int block);

void* afb_sched_create(int max_items, int max_query_tokens, int prefill_chunk, int min_chunk, int decode_streak,
                       int max_kv_blocks, int page, int max_queue);
void afb_sched_destroy(void* h);
int afb_sched_admit(void* h, int64_t id, int prompt_len, int max_new_tokens);
int afb_sched_claim_step(void* h, int64_t* ids, int* modes, int* q_lens, int* kv_before, int max_out);
int afb_sched_complete_step(void* h, int n, const int64_t* ids, const int* tokens_out, const int* finished);
int afb_sched_fail_step(void* h);
int afb_sched_cancel(void* h, int64_t id);

void* afb_grammar_json_new(int root_object_only);
void* afb_grammar_gbnf_new(const char* text, const char* root);
void afb_grammar_free(void* h);
void afb_grammar_reset(void* h);
int afb_grammar_set_vocab(void* h, const uint8_t* bytes, const int64_t* offsets, int n_tokens);
int afb_grammar_mask(void* h, uint8_t* allowed);
int afb_grammar_accept_bytes(void* h, const uint8_t* bytes, int n);
int afb_grammar_complete(void* h);

long afb_kvq_row_bytes(int codec, int heads, int D, int is_value);
int afb_kvq_encode_rows(int codec, int is_value, const float* src, uint8_t* dst, long n_rows, int heads, int D);
int afb_kvq_decode_rows(int codec, int is_value, const uint8_t* src, float* dst, long n_rows, int heads, int D);
int afb_kvq_attention_host(int codec, const float* q, const uint8_t* k_rows, const uint8_t* v_rows, long n_tokens,
                           int Hq, int Hkv, int D, float scale, float k_scale, float v_scale, int window, float* out);

long afb_gguf_block_bytes(int type);
long afb_gguf_block_values(int type);
int afb_gguf_dequantize(int type, const uint8_t* src, float* dst, long n_values);
float afb_gguf_element(int type, const uint8_t* block, int j);
long afb_gguf_element_block_values(int type);
int afb_image_preprocess_host(const uint8_t* img, int src_w, int src_h, int channels, float crop_x, float crop_y,
                              float crop_w, float crop_h, int out_w, int out_h, int mode, float rescale,
                              const float* mean3, const float* std3, float* out_chw);
int afb_hilbert_keys(const float* vectors, long n, int dims, uint8_t* keys);
void afb_cpu_set_threads(int n);
int afb_cpu_topk(const float* q, const float* x, int Q, long N, int D, int k, int metric, int* out_idx,
                 float* out_dist);
}

static int g_fail = 0;
#define CHECK(c)                                                        \
  do {                                                                  \
    if (!(c)) {                                                         \
      std::fprintf(stderr, "CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #c); \
      ++g_fail;                                                         \
    }                                                                   \
  } while (0)

static void kv_pool_workload(unsigned seed, int iters) {
  std::mt19937 rng(seed);
  const int blocks = 64, page = 16;
  void* kv = afb_kv_create(blocks, page);
  std::map<int64_t, int> len;
  int64_t next = 1;
  std::vector<int> slots(512), tab(64), src(64), dst(64);
  for (int it = 0; it < iters; ++it) {
    const int op = static_cast<int>(rng() % 8);
    if (op == 0 || len.empty()) {
      if (afb_kv_attach(kv, next) == 0) len[next] = 0;
      ++next;
    } else {
      auto pick = len.begin();
      std::advance(pick, rng() % len.size());
      const int64_t s = pick->first;
      if (op <= 3) {
        const int n = 1 + static_cast<int>(rng() % 40);
        if (afb_kv_append(kv, s, n, slots.data()) == 0) {
          pick->second += n;
          for (int i = 0; i < n; ++i) CHECK(slots[i] >= 0 && slots[i] < blocks * page);
        }
        afb_kv_take_cow(kv, src.data(), dst.data(), 64);
      } else if (op == 4 && pick->second > 0) {
        const int nl = static_cast<int>(rng() % (pick->second + 1));
        if (afb_kv_truncate(kv, s, nl) == 0) pick->second = nl;
      } else if (op == 5 && pick->second > 0) {
        const int pre = static_cast<int>(rng() % (pick->second + 1));
        if (afb_kv_attach_shared(kv, next, s, pre) == 0) len[next] = pre;
        ++next;
      } else if (op == 6) {
        afb_kv_trim_window(kv, s, 8 + static_cast<int>(rng() % 64));
      } else {
        CHECK(afb_kv_detach(kv, s) == 0);
        len.erase(pick);
        continue;
      }
      CHECK(afb_kv_len(kv, s) == pick->second);
      const int nb = afb_kv_block_table(kv, s, tab.data(), 64);
      CHECK(nb >= 0 && nb <= 64);
    }
  }
  for (auto& kvp : len) afb_kv_detach(kv, kvp.first);
  CHECK(afb_kv_free_blocks(kv) == blocks);
  for (int b = 0; b < blocks; ++b) CHECK(afb_kv_refcount(kv, b) == 0);
  afb_kv_destroy(kv);
}

static void scheduler_workload(unsigned seed, int iters) {
  std::mt19937 rng(seed);
  void* s = afb_sched_create(16, 512, 256, 32, 4, 256, 16, 64);
  int64_t next = 1;
  std::vector<int64_t> ids(16);
  std::vector<int> modes(16), ql(16), kvb(16), toks(16), fin(16);
  for (int it = 0; it < iters; ++it) {
    if (rng() % 3 == 0) afb_sched_admit(s, next++, 1 + static_cast<int>(rng() % 700), 1 + static_cast<int>(rng() % 20));
    if (rng() % 17 == 0 && next > 1) afb_sched_cancel(s, 1 + static_cast<int64_t>(rng() % (next - 1)));
    const int n = afb_sched_claim_step(s, ids.data(), modes.data(), ql.data(), kvb.data(), 16);
    CHECK(n >= 0 && n <= 16);
    if (n == 0) continue;
    int total = 0;
    for (int i = 0; i < n; ++i) total += ql[i];
    CHECK(total <= 512);
    if (rng() % 11 == 0) {
      afb_sched_fail_step(s);
      continue;
    }
    for (int i = 0; i < n; ++i) {
      toks[i] = static_cast<int>(rng() % 1000);
      fin[i] = rng() % 13 == 0;
    }
    afb_sched_complete_step(s, n, ids.data(), toks.data(), fin.data());
  }
  afb_sched_destroy(s);
}

static void grammar_workload(unsigned seed) {
  std::mt19937 rng(seed);
  // byte-level vocabulary plus a few multi-byte tokens
  std::vector<uint8_t> bytes;
  std::vector<int64_t> off{0};
  for (int b = 0; b < 256; ++b) {
    bytes.push_back(static_cast<uint8_t>(b));
    off.push_back(static_cast<int64_t>(bytes.size()));
  }
  for (const char* t : {"{\"", "\":", "true", "false", "null", "\", \"", "}}", "[1,", "0.5e3"}) {
    for (const char* c = t; *c; ++c) bytes.push_back(static_cast<uint8_t>(*c));
    off.push_back(static_cast<int64_t>(bytes.size()));
  }
  const int V = static_cast<int>(off.size()) - 1;
  std::vector<uint8_t> allowed(V);
  void* gs[2] = {afb_grammar_json_new(1),
                 afb_grammar_gbnf_new("root ::= item (\",\" item)*\nitem ::= [a-z]+ | \"(\" root \")\" | num\nnum ::= "
                                      "\"-\"? [0-9]+ (\".\" [0-9]+)?\n", "root")};
  for (void* g : gs) {
    CHECK(g != nullptr);
    if (!g) continue;
    CHECK(afb_grammar_set_vocab(g, bytes.data(), off.data(), V) == 0);
    for (int round = 0; round < 20; ++round) {
      afb_grammar_reset(g);
      for (int step = 0; step < 200; ++step) {
        const int n_ok = afb_grammar_mask(g, allowed.data());
        if (n_ok <= 0) break;
        std::vector<int> ok;
        for (int t = 0; t < V; ++t)
          if (allowed[t]) ok.push_back(t);
        if (ok.empty()) break;
        const int t = ok[rng() % ok.size()];
        CHECK(afb_grammar_accept_bytes(g, bytes.data() + off[t], static_cast<int>(off[t + 1] - off[t])) == 1);
        if (afb_grammar_complete(g) && rng() % 4 == 0) break;
      }
    }
    afb_grammar_free(g);
  }
  // malformed grammars must be rejected, not crash
  for (const char* bad : {"root ::= (", "root ::= [a-", "root ::= missing", "", "root ::= \"a\" |"}) {
    void* g = afb_grammar_gbnf_new(bad, "root");
    if (g) afb_grammar_free(g);
  }
}

static void kv_codec_workload(unsigned seed) {
  std::mt19937 rng(seed);
  std::normal_distribution<float> nd(0.0f, 0.6f);
  const int dims[] = {64, 80, 128, 256};
  for (int codec = 0; codec < 6; ++codec) {
    for (int D : dims) {
      for (int heads : {1, 3}) {
        const long T = 19;
        const long kb = afb_kvq_row_bytes(codec, heads, D, 0), vb = afb_kvq_row_bytes(codec, heads, D, 1);
        CHECK(kb > 0 && vb > 0);
        std::vector<float> k(T * heads * D), v(T * heads * D), back(T * heads * D), q(2 * heads * D), out(2 * heads * D);
        for (auto& x : k) x = nd(rng);
        for (auto& x : v) x = nd(rng);
        for (auto& x : q) x = nd(rng);
        std::vector<uint8_t> kr(T * kb), vr(T * vb);   // exactly sized: an overrun is an ASan report
        CHECK(afb_kvq_encode_rows(codec, 0, k.data(), kr.data(), T, heads, D) == 0);
        CHECK(afb_kvq_encode_rows(codec, 1, v.data(), vr.data(), T, heads, D) == 0);
        CHECK(afb_kvq_decode_rows(codec, 0, kr.data(), back.data(), T, heads, D) == 0);
        CHECK(afb_kvq_decode_rows(codec, 1, vr.data(), back.data(), T, heads, D) == 0);
        CHECK(afb_kvq_attention_host(codec, q.data(), kr.data(), vr.data(), T, 2 * heads, heads, D, 0.1f, 1.0f, 1.0f,
                                     rng() % 2 ? 7 : 0, out.data()) == 0);
        for (float x : out) CHECK(x == x);
      }
    }
  }
  CHECK(afb_kvq_row_bytes(4, 2, 96, 0) == 0);
}

static void gguf_and_image_workload(unsigned seed) {
  std::mt19937 rng(seed);
  // every block decoder over random bytes in buffers of exactly the block size (an overrun is an ASan report)
  for (int type = 0; type < 64; ++type) {
    const long bb = afb_gguf_block_bytes(type), bv = afb_gguf_block_values(type);
    if (bb <= 0 || bv <= 0) continue;
    const long blocks = 7;
    std::vector<uint8_t> src(blocks * bb);
    for (auto& b : src) b = static_cast<uint8_t>(rng());
    std::vector<float> dst(blocks * bv);
    CHECK(afb_gguf_dequantize(type, src.data(), dst.data(), blocks * bv) == 0);
    const long ev = afb_gguf_element_block_values(type);
    if (ev > 0) {
      for (long b = 0; b < blocks; ++b)
        for (long j = 0; j < ev; ++j) {
          const float e = afb_gguf_element(type, src.data() + b * bb, static_cast<int>(j));
          const float d = dst[b * bv + j];
          CHECK(e == d || (e != e && d != d));     // the per-element decoder and the block decoder agree
        }
    }
  }
  // image preprocessing at awkward geometries: 1-pixel sources, crops at the border, up- and down-scaling
  const float mean[3] = {0.48f, 0.45f, 0.40f}, sd[3] = {0.26f, 0.26f, 0.27f};
  const int geo[][4] = {{1, 1, 8, 8}, {2, 3, 5, 7}, {37, 19, 16, 16}, {64, 64, 3, 1}, {5, 200, 9, 2}};
  for (auto& g : geo) {
    for (int ch : {3, 4}) {
      for (int mode = 0; mode < 3; ++mode) {
        std::vector<uint8_t> img(static_cast<size_t>(g[0]) * g[1] * ch);
        for (auto& b : img) b = static_cast<uint8_t>(rng());
        std::vector<float> out(3u * g[2] * g[3]);
        CHECK(afb_image_preprocess_host(img.data(), g[0], g[1], ch, 0.0f, 0.0f, static_cast<float>(g[0]),
                                        static_cast<float>(g[1]), g[2], g[3], mode, 1.0f / 255, mean, sd,
                                        out.data()) == 0);
        // a crop hanging off the bottom-right corner
        CHECK(afb_image_preprocess_host(img.data(), g[0], g[1], ch, g[0] * 0.5f, g[1] * 0.5f, g[0] * 0.5f + 0.49f,
                                        g[1] * 0.5f + 0.49f, g[2], g[3], mode, 1.0f / 255, mean, sd, out.data()) == 0);
        for (float v : out) CHECK(v == v);
      }
    }
  }
  std::vector<float> pts(257 * 24);
  for (auto& v : pts) v = static_cast<float>(rng() % 2000) / 1000.0f - 1.0f;
  std::vector<uint8_t> keys(257 * 4 * 24, 0);   // exactly 4 bytes per dimension
  afb_hilbert_keys(pts.data(), 257, 24, keys.data());
}

static void threaded_workload(unsigned seed) {
  std::mt19937 rng(seed);
  std::normal_distribution<float> nd;
  const int Q = 24, D = 48, k = 5;
  const long N = 3000;
  std::vector<float> q(Q * D), x(N * D);
  for (auto& v : q) v = nd(rng);
  for (auto& v : x) v = nd(rng);
  afb_cpu_set_threads(4);
  std::vector<int> idx(Q * k);
  std::vector<float> dist(Q * k);
  for (int metric = 0; metric < 3; ++metric) {
    CHECK(afb_cpu_topk(q.data(), x.data(), Q, N, D, k, metric, idx.data(), dist.data()) == 0);
    for (int i = 0; i < Q * k; ++i) CHECK(idx[i] >= 0 && idx[i] < N);
  }
  std::vector<uint8_t> keys(N * ((D + 7) / 8 * 8));
  (void)keys;
  // the block pool and the scheduler are shared between the HTTP threads and the engine thread
  void* kv = afb_kv_create(256, 16);
  std::vector<std::thread> th;
  for (int t = 0; t < 4; ++t) {
    th.emplace_back([kv, t, seed] {
      std::mt19937 r(seed + 17 * t);
      std::vector<int> slots(64);
      for (int i = 0; i < 300; ++i) {
        const int64_t s = 1000 * (t + 1) + i;
        if (afb_kv_attach(kv, s) != 0) continue;
        afb_kv_append(kv, s, 1 + static_cast<int>(r() % 48), slots.data());
        afb_kv_truncate(kv, s, static_cast<int>(r() % 8));
        afb_kv_detach(kv, s);
      }
    });
  }
  for (auto& t : th) t.join();
  CHECK(afb_kv_free_blocks(kv) == 256);
  afb_kv_destroy(kv);
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "asan";
  const unsigned seed = argc > 2 ? static_cast<unsigned>(std::atoi(argv[2])) : 1u;
  if (mode == "tsan") {
    threaded_workload(seed);
  } else {
    kv_pool_workload(seed, 6000);
    scheduler_workload(seed + 1, 4000);
    grammar_workload(seed + 2);
    kv_codec_workload(seed + 3);
    gguf_and_image_workload(seed + 5);
    threaded_workload(seed + 4);
  }
  std::printf("sanitize_main %s seed=%u failures=%d\n", mode.c_str(), seed, g_fail);
  return g_fail ? 1 : 0;
}
