// Hierarchical navigable small-world graph index (host side): insert, delete with local repair, filtered search,
// save / load.  It is the counterpart of the reference's graph index
// (go/pkg/antfly/lib/vectorindex/hnsw.go:221-255 configuration, :1277-1627 insertion, :1658-1802 search with a
// metadata-prefix filter and the direct-scan rule for selective filters, :1804-2100 deletion and entry-point
// repair), whose nodes live as key/value records in an LSM store and are walked through an LRU node cache.
//
// This one keeps the whole graph in flat arrays: vectors [slots, dim] fp32, layer-0 adjacency as fixed slabs of
// (count, M0 neighbours) per slot, upper layers as one slab of (count, M neighbours) per (slot, layer).  Fixed slabs
// make a node's neighbourhood one contiguous read, let searches run lock-free in parallel over queries, and are the
// form in which the graph can be handed to a device wholesale.  Distances are "lower is closer":
// 0 l2_squared, 1 inner_product (-a.b), 2 cosine (1 - a.b / |a||b|; rows are stored unit-normalised).
//
// Construction is the standard one: a node draws its top layer from an exponential distribution, descends greedily
// from the entry point to that layer, and on every layer from there down runs a beam search of width
// ef_construction and keeps the neighbours chosen by the diversity heuristic (a candidate is kept only if it is
// closer to the new node than to every neighbour already kept); neighbours that overflow are re-pruned the same way.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <mutex>
#include <queue>
#include <random>
#include <shared_mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

constexpr uint32_t kNone = 0xffffffffu;
constexpr uint64_t kFileMagic = 0x31574e5348464241ull;  // "ABFHSNW1"

struct Cand {
  float d;
  uint32_t s;
};
struct Nearer {  // max-heap on distance
  bool operator()(const Cand& a, const Cand& b) const { return a.d < b.d || (a.d == b.d && a.s < b.s); }
};
struct Farther {  // min-heap on distance
  bool operator()(const Cand& a, const Cand& b) const { return a.d > b.d || (a.d == b.d && a.s > b.s); }
};

struct Hnsw {
  int dim = 0, metric = 0, M = 16, M0 = 32, efc = 200, efs = 64;
  double level_mult = 1.0 / std::log(2.0);
  std::mt19937_64 rng;
  std::vector<float> vecs;               // [slots, dim]
  std::vector<uint32_t> links0;          // [slots, M0 + 1]
  std::vector<std::vector<uint32_t>> up; // per slot: [level, M + 1]
  std::vector<int> level;                // -1 = free slot
  std::vector<uint64_t> ids;
  std::vector<std::string> meta;
  std::vector<uint32_t> free_slots;
  std::unordered_map<uint64_t, uint32_t> slot_of;
  uint32_t entry = kNone;
  int max_level = -1;
  long active = 0;
  std::vector<uint8_t> build_seen;       // visited marks of the writer (inserts hold the exclusive lock)
  mutable std::shared_mutex mu;

  const float* vec(uint32_t s) const { return vecs.data() + static_cast<size_t>(s) * dim; }
  uint32_t* nbrs(uint32_t s, int l) {
    return l == 0 ? links0.data() + static_cast<size_t>(s) * (M0 + 1) : up[s].data() + static_cast<size_t>(l - 1) * (M + 1);
  }
  const uint32_t* nbrs(uint32_t s, int l) const { return const_cast<Hnsw*>(this)->nbrs(s, l); }
  int cap(int l) const { return l == 0 ? M0 : M; }

  float dist(const float* a, const float* b) const {
    float acc = 0.0f;
    if (metric == 0) {
#pragma omp simd reduction(+ : acc)
      for (int i = 0; i < dim; ++i) {
        const float t = a[i] - b[i];
        acc += t * t;
      }
      return acc;
    }
#pragma omp simd reduction(+ : acc)
    for (int i = 0; i < dim; ++i) acc += a[i] * b[i];
    return metric == 1 ? -acc : 1.0f - acc;
  }

  // Greedy descent on one layer: move to the closest neighbour until none is closer.
  uint32_t greedy(const float* q, uint32_t start, int l, float* best_d) const {
    uint32_t cur = start;
    float cd = dist(q, vec(cur));
    for (bool moved = true; moved;) {
      moved = false;
      const uint32_t* nb = nbrs(cur, l);
      for (uint32_t i = 1; i <= nb[0]; ++i) {
        const uint32_t s = nb[i];
        if (level[s] < l) continue;
        const float d = dist(q, vec(s));
        if (d < cd) {
          cd = d;
          cur = s;
          moved = true;
        }
      }
    }
    if (best_d) *best_d = cd;
    return cur;
  }

  // Beam search on one layer.  `accept` decides which visited nodes may enter the result; every visited node still
  // steers the walk, so a filter does not disconnect the graph, and the walk goes on until ef accepted nodes bound
  // it (or the reachable graph is exhausted).  Result: ascending by distance.
  template <class Accept>
  void search_layer(const float* q, uint32_t start, int ef, int l, std::vector<uint8_t>& seen, Accept accept,
                    std::vector<Cand>& out) const {
    std::priority_queue<Cand, std::vector<Cand>, Farther> frontier;
    std::priority_queue<Cand, std::vector<Cand>, Nearer> best;
    std::vector<uint32_t> touched;
    const float d0 = dist(q, vec(start));
    frontier.push({d0, start});
    seen[start] = 1;
    touched.push_back(start);
    if (accept(start)) best.push({d0, start});
    while (!frontier.empty()) {
      const Cand c = frontier.top();
      if (static_cast<int>(best.size()) >= ef && c.d > best.top().d) break;
      frontier.pop();
      const uint32_t* nb = nbrs(c.s, l);
      for (uint32_t i = 1; i <= nb[0]; ++i) {
        const uint32_t s = nb[i];
        if (seen[s] || level[s] < l) continue;
        seen[s] = 1;
        touched.push_back(s);
        const float d = dist(q, vec(s));
        if (static_cast<int>(best.size()) >= ef && d >= best.top().d) continue;
        frontier.push({d, s});
        if (accept(s)) {
          best.push({d, s});
          if (static_cast<int>(best.size()) > ef) best.pop();
        }
      }
    }
    out.resize(best.size());
    for (size_t i = best.size(); i-- > 0;) {
      out[i] = best.top();
      best.pop();
    }
    for (uint32_t s : touched) seen[s] = 0;
  }

  // Diversity heuristic over candidates sorted ascending by distance to `base`.
  void select(const float* base, const std::vector<Cand>& cands, int m, std::vector<uint32_t>& out) const {
    out.clear();
    std::vector<uint32_t> skipped;
    for (const Cand& c : cands) {
      if (static_cast<int>(out.size()) >= m) break;
      bool keep = true;
      for (uint32_t k : out)
        if (dist(vec(c.s), vec(k)) < c.d) {
          keep = false;
          break;
        }
      if (keep) out.push_back(c.s);
      else skipped.push_back(c.s);
    }
    (void)base;
    for (uint32_t s : skipped) {  // fill what is left with the closest of the rest (keeps sparse regions connected)
      if (static_cast<int>(out.size()) >= m) break;
      out.push_back(s);
    }
  }

  void set_links(uint32_t s, int l, const std::vector<uint32_t>& list) {
    uint32_t* nb = nbrs(s, l);
    nb[0] = static_cast<uint32_t>(list.size());
    for (size_t i = 0; i < list.size(); ++i) nb[1 + i] = list[i];
  }

  // Adds the edge s -> t on layer l, re-pruning s's list when it is full.
  void connect(uint32_t s, uint32_t t, int l) {
    uint32_t* nb = nbrs(s, l);
    for (uint32_t i = 1; i <= nb[0]; ++i)
      if (nb[i] == t) return;
    if (static_cast<int>(nb[0]) < cap(l)) {
      nb[++nb[0]] = t;
      return;
    }
    std::vector<Cand> cands;
    cands.reserve(nb[0] + 1);
    for (uint32_t i = 1; i <= nb[0]; ++i) cands.push_back({dist(vec(s), vec(nb[i])), nb[i]});
    cands.push_back({dist(vec(s), vec(t)), t});
    std::sort(cands.begin(), cands.end(), [](const Cand& a, const Cand& b) { return a.d < b.d || (a.d == b.d && a.s < b.s); });
    std::vector<uint32_t> kept;
    select(vec(s), cands, cap(l), kept);
    set_links(s, l, kept);
  }

  int draw_level() {
    std::uniform_real_distribution<double> u(std::numeric_limits<double>::min(), 1.0);
    const int l = static_cast<int>(-std::log(u(rng)) * level_mult);
    return std::min(l, 30);
  }

  uint32_t alloc_slot() {
    if (!free_slots.empty()) {
      const uint32_t s = free_slots.back();
      free_slots.pop_back();
      return s;
    }
    const uint32_t s = static_cast<uint32_t>(level.size());
    level.push_back(-1);
    ids.push_back(0);
    meta.emplace_back();
    up.emplace_back();
    vecs.resize(static_cast<size_t>(s + 1) * dim);
    links0.resize(static_cast<size_t>(s + 1) * (M0 + 1), 0);
    return s;
  }

  void insert_one(uint64_t id, const float* v, const uint8_t* md, long md_len, int forced_level) {
    auto it = slot_of.find(id);
    if (it != slot_of.end()) remove_slots({it->second});
    const uint32_t s = alloc_slot();
    float* dst = vecs.data() + static_cast<size_t>(s) * dim;
    std::memcpy(dst, v, sizeof(float) * dim);
    if (metric == 2) {
      double n = 0.0;
      for (int i = 0; i < dim; ++i) n += static_cast<double>(dst[i]) * dst[i];
      const float inv = n > 0.0 ? static_cast<float>(1.0 / std::sqrt(n)) : 0.0f;
      for (int i = 0; i < dim; ++i) dst[i] *= inv;
    }
    const int lv = forced_level >= 0 ? forced_level : draw_level();
    level[s] = lv;
    ids[s] = id;
    meta[s].assign(reinterpret_cast<const char*>(md), static_cast<size_t>(md_len));
    up[s].assign(static_cast<size_t>(lv) * (M + 1), 0);
    links0[static_cast<size_t>(s) * (M0 + 1)] = 0;
    slot_of[id] = s;
    ++active;
    if (entry == kNone) {
      entry = s;
      max_level = lv;
      return;
    }
    uint32_t cur = entry;
    for (int l = max_level; l > lv; --l) cur = greedy(dst, cur, l, nullptr);
    if (build_seen.size() < level.size()) build_seen.resize(level.size() + level.size() / 2 + 64, 0);
    std::vector<Cand> found;
    std::vector<uint32_t> chosen;
    for (int l = std::min(lv, max_level); l >= 0; --l) {
      search_layer(dst, cur, efc, l, build_seen, [&](uint32_t x) { return x != s; }, found);
      if (found.empty()) continue;
      select(dst, found, M, chosen);  // a new node starts with at most M links on every layer
      set_links(s, l, chosen);
      for (uint32_t t : chosen) connect(t, s, l);
      cur = found[0].s;
    }
    if (lv > max_level) {
      max_level = lv;
      entry = s;
    }
  }

  // Removes a set of slots: drops every edge into them, reconnects the nodes that lost an edge through the removed
  // node's own neighbours, frees the slots and re-elects the entry point if it went.
  void remove_slots(const std::vector<uint32_t>& gone_list) {
    if (gone_list.empty()) return;
    std::unordered_set<uint32_t> gone(gone_list.begin(), gone_list.end());
    const uint32_t n = static_cast<uint32_t>(level.size());
    std::vector<Cand> cands;
    std::vector<uint32_t> kept;
    for (uint32_t s = 0; s < n; ++s) {
      if (level[s] < 0 || gone.count(s)) continue;
      for (int l = 0; l <= level[s]; ++l) {
        uint32_t* nb = nbrs(s, l);
        bool lost = false;
        for (uint32_t i = 1; i <= nb[0]; ++i)
          if (gone.count(nb[i])) lost = true;
        if (!lost) continue;
        // candidates: surviving neighbours, plus the surviving neighbours of every neighbour that goes
        std::unordered_set<uint32_t> pool;
        for (uint32_t i = 1; i <= nb[0]; ++i) {
          const uint32_t t = nb[i];
          if (!gone.count(t)) {
            pool.insert(t);
            continue;
          }
          if (level[t] < l) continue;
          const uint32_t* tn = nbrs(t, l);
          for (uint32_t j = 1; j <= tn[0]; ++j)
            if (!gone.count(tn[j]) && tn[j] != s && level[tn[j]] >= l) pool.insert(tn[j]);
        }
        cands.clear();
        for (uint32_t t : pool) cands.push_back({dist(vec(s), vec(t)), t});
        std::sort(cands.begin(), cands.end(), [](const Cand& a, const Cand& b) { return a.d < b.d || (a.d == b.d && a.s < b.s); });
        select(vec(s), cands, cap(l), kept);
        set_links(s, l, kept);
      }
    }
    for (uint32_t s : gone_list) {
      if (level[s] < 0) continue;
      slot_of.erase(ids[s]);
      level[s] = -1;
      up[s].clear();
      up[s].shrink_to_fit();
      meta[s].clear();
      links0[static_cast<size_t>(s) * (M0 + 1)] = 0;
      free_slots.push_back(s);
      --active;
    }
    if (entry != kNone && level[entry] < 0) {
      entry = kNone;
      max_level = -1;
      for (uint32_t s = 0; s < n; ++s)
        if (level[s] > max_level) {
          max_level = level[s];
          entry = s;
        }
    }
  }
};

bool has_prefix(const std::string& s, const uint8_t* p, int n) {
  return static_cast<int>(s.size()) >= n && std::memcmp(s.data(), p, static_cast<size_t>(n)) == 0;
}

}  // namespace

extern "C" {

// metric: 0 l2_squared, 1 inner_product, 2 cosine.  m: links per node on the upper layers and for a new node;
// m0: capacity on layer 0 (<= 0: 2 m).  level_mult <= 0: 1 / ln(m).
void* afb_hnsw_create(int dim, int metric, int m, int m0, int ef_construction, int ef_search, double level_mult,
                      uint64_t seed) {
  if (dim <= 0 || metric < 0 || metric > 2 || m < 2) return nullptr;
  Hnsw* h = new Hnsw();
  h->dim = dim;
  h->metric = metric;
  h->M = m;
  h->M0 = m0 > 0 ? std::max(m0, m) : 2 * m;
  h->efc = std::max(ef_construction, m);
  h->efs = std::max(ef_search, 1);
  h->level_mult = level_mult > 0.0 ? level_mult : 1.0 / std::log(static_cast<double>(m));
  h->rng.seed(seed);
  return h;
}

void afb_hnsw_free(void* p) { delete static_cast<Hnsw*>(p); }

// Upsert n vectors.  meta_blob / meta_offsets [n + 1] (may be null: no metadata).  levels (may be null) forces the
// top layer of each node (tests, reproducible builds).
int afb_hnsw_insert(void* p, const uint64_t* ids, const float* vecs, long n, const uint8_t* meta_blob,
                    const long* meta_offsets, const int* levels) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h || n < 0) return -1;
  std::unique_lock<std::shared_mutex> lock(h->mu);
  for (long i = 0; i < n; ++i) {
    const uint8_t* md = meta_blob && meta_offsets ? meta_blob + meta_offsets[i] : nullptr;
    const long len = meta_blob && meta_offsets ? meta_offsets[i + 1] - meta_offsets[i] : 0;
    h->insert_one(ids[i], vecs + static_cast<size_t>(i) * h->dim, md, len, levels ? levels[i] : -1);
  }
  return 0;
}

// nq queries -> out_ids / out_dist [nq, k], ascending, padded with ~0 / +inf.  prefix (may be null) keeps only nodes
// whose metadata starts with it; when the filter is selective (k >= 20 % of the matches, or fewer than 100 matches)
// the matches are scanned directly instead of walking the graph.  ef <= 0: the index default.  Returns the number of
// results written for the first query, or -1.
long afb_hnsw_search(void* p, const float* queries, long nq, int k, int ef, const uint8_t* prefix, int prefix_len,
                     uint64_t* out_ids, float* out_dist, int threads) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h || nq < 0 || k <= 0) return -1;
  std::shared_lock<std::shared_mutex> lock(h->mu);
  for (long i = 0; i < nq * k; ++i) {
    out_ids[i] = ~0ull;
    out_dist[i] = std::numeric_limits<float>::infinity();
  }
  if (h->active == 0 || nq == 0) return 0;
  const uint32_t n = static_cast<uint32_t>(h->level.size());
  const bool filtered = prefix && prefix_len > 0;
  std::vector<uint32_t> matches;
  bool direct = false;
  if (filtered) {
    for (uint32_t s = 0; s < n; ++s)
      if (h->level[s] >= 0 && has_prefix(h->meta[s], prefix, prefix_len)) matches.push_back(s);
    if (matches.empty()) return 0;
    direct = static_cast<double>(k) >= 0.2 * static_cast<double>(matches.size()) || matches.size() < 100;
  }
  const int width = std::max(ef > 0 ? ef : h->efs, k);
  std::vector<long> counts(static_cast<size_t>(nq), 0);
  auto run = [&](long lo, long hi) {
    std::vector<uint8_t> seen(n, 0);
    std::vector<Cand> found;
    std::vector<float> qn(static_cast<size_t>(h->dim));
    for (long qi = lo; qi < hi; ++qi) {
      const float* q = queries + static_cast<size_t>(qi) * h->dim;
      if (h->metric == 2) {
        double nn = 0.0;
        for (int i = 0; i < h->dim; ++i) nn += static_cast<double>(q[i]) * q[i];
        const float inv = nn > 0.0 ? static_cast<float>(1.0 / std::sqrt(nn)) : 0.0f;
        for (int i = 0; i < h->dim; ++i) qn[static_cast<size_t>(i)] = q[i] * inv;
        q = qn.data();
      }
      found.clear();
      if (direct) {
        for (uint32_t s : matches) found.push_back({h->dist(q, h->vec(s)), s});
        std::sort(found.begin(), found.end(), [](const Cand& a, const Cand& b) { return a.d < b.d || (a.d == b.d && a.s < b.s); });
      } else {
        uint32_t cur = h->entry;
        for (int l = h->max_level; l > 0; --l) cur = h->greedy(q, cur, l, nullptr);
        if (filtered)
          h->search_layer(q, cur, width, 0, seen, [&](uint32_t s) { return has_prefix(h->meta[s], prefix, prefix_len); }, found);
        else
          h->search_layer(q, cur, width, 0, seen, [](uint32_t) { return true; }, found);
      }
      const long m = std::min<long>(k, static_cast<long>(found.size()));
      for (long j = 0; j < m; ++j) {
        out_ids[qi * k + j] = h->ids[found[static_cast<size_t>(j)].s];
        out_dist[qi * k + j] = found[static_cast<size_t>(j)].d;
      }
      counts[static_cast<size_t>(qi)] = m;
    }
  };
  const int nt = static_cast<int>(std::max<long>(1, std::min<long>(threads > 0 ? threads : 1, nq)));
  if (nt == 1) {
    run(0, nq);
  } else {
    std::vector<std::thread> pool;
    const long per = (nq + nt - 1) / nt;
    for (int t = 0; t < nt; ++t) {
      const long lo = t * per, hi = std::min(nq, lo + per);
      if (lo < hi) pool.emplace_back(run, lo, hi);
    }
    for (auto& t : pool) t.join();
  }
  return counts[0];
}

long afb_hnsw_delete(void* p, const uint64_t* ids, long n) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h) return -1;
  std::unique_lock<std::shared_mutex> lock(h->mu);
  std::vector<uint32_t> gone;
  for (long i = 0; i < n; ++i) {
    auto it = h->slot_of.find(ids[i]);
    if (it != h->slot_of.end() && std::find(gone.begin(), gone.end(), it->second) == gone.end()) gone.push_back(it->second);
  }
  h->remove_slots(gone);
  return static_cast<long>(gone.size());
}

// Removes every node whose metadata equals `key`.
long afb_hnsw_delete_by_metadata(void* p, const uint8_t* key, int len) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h || len < 0) return -1;
  std::unique_lock<std::shared_mutex> lock(h->mu);
  std::vector<uint32_t> gone;
  for (uint32_t s = 0; s < h->level.size(); ++s)
    if (h->level[s] >= 0 && static_cast<int>(h->meta[s].size()) == len &&
        std::memcmp(h->meta[s].data(), key, static_cast<size_t>(len)) == 0)
      gone.push_back(s);
  h->remove_slots(gone);
  return static_cast<long>(gone.size());
}

// out[0] active nodes, [1] top layer, [2] entry id (valid when active > 0), [3] directed edges, [4] slots allocated,
// [5] nodes above layer 0.
int afb_hnsw_stats(void* p, long* out) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h) return -1;
  std::shared_lock<std::shared_mutex> lock(h->mu);
  long edges = 0, upper = 0;
  for (uint32_t s = 0; s < h->level.size(); ++s) {
    if (h->level[s] < 0) continue;
    upper += h->level[s] > 0;
    for (int l = 0; l <= h->level[s]; ++l) edges += h->nbrs(s, l)[0];
  }
  out[0] = h->active;
  out[1] = h->max_level;
  out[2] = h->entry == kNone ? 0 : static_cast<long>(h->ids[h->entry]);
  out[3] = edges;
  out[4] = static_cast<long>(h->level.size());
  out[5] = upper;
  return 0;
}

// Metadata of `id` into out (cap bytes); returns its length, -1 when the id is absent.
long afb_hnsw_get_metadata(void* p, uint64_t id, uint8_t* out, long cap) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h) return -1;
  std::shared_lock<std::shared_mutex> lock(h->mu);
  auto it = h->slot_of.find(id);
  if (it == h->slot_of.end()) return -1;
  const std::string& m = h->meta[it->second];
  std::memcpy(out, m.data(), static_cast<size_t>(std::min<long>(cap, static_cast<long>(m.size()))));
  return static_cast<long>(m.size());
}

// The stored vector of `id` into out [dim] (unit-normalised for the cosine metric); 0, or -1 when the id is absent.
int afb_hnsw_get_vector(void* p, uint64_t id, float* out) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h) return -1;
  std::shared_lock<std::shared_mutex> lock(h->mu);
  auto it = h->slot_of.find(id);
  if (it == h->slot_of.end()) return -1;
  std::memcpy(out, h->vec(it->second), sizeof(float) * static_cast<size_t>(h->dim));
  return 0;
}

// Structural self-check: 0 when every edge points at a live node that exists on that layer, no list exceeds its
// capacity or repeats a neighbour or names its own node, the id map agrees with the slots, and the entry point is a
// live node of the top layer.  Otherwise a positive code naming the first violated rule.
int afb_hnsw_check(void* p) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h) return -1;
  std::shared_lock<std::shared_mutex> lock(h->mu);
  long live = 0;
  int top = -1;
  for (uint32_t s = 0; s < h->level.size(); ++s) {
    if (h->level[s] < 0) continue;
    ++live;
    top = std::max(top, h->level[s]);
    auto it = h->slot_of.find(h->ids[s]);
    if (it == h->slot_of.end() || it->second != s) return 1;
    if (static_cast<long>(h->up[s].size()) != static_cast<long>(h->level[s]) * (h->M + 1)) return 2;
    for (int l = 0; l <= h->level[s]; ++l) {
      const uint32_t* nb = h->nbrs(s, l);
      if (static_cast<int>(nb[0]) > h->cap(l)) return 3;
      for (uint32_t i = 1; i <= nb[0]; ++i) {
        const uint32_t t = nb[i];
        if (t >= h->level.size() || h->level[t] < l) return 4;
        if (t == s) return 5;
        for (uint32_t j = 1; j < i; ++j)
          if (nb[j] == t) return 6;
      }
    }
  }
  if (live != h->active || static_cast<long>(h->slot_of.size()) != live) return 7;
  if (live == 0) return (h->entry == kNone && h->max_level == -1) ? 0 : 8;
  if (h->entry == kNone || h->level[h->entry] != top || h->max_level != top) return 9;
  return 0;
}

int afb_hnsw_save(void* p, const char* path) {
  Hnsw* h = static_cast<Hnsw*>(p);
  if (!h) return -1;
  std::shared_lock<std::shared_mutex> lock(h->mu);
  FILE* f = std::fopen(path, "wb");
  if (!f) return -2;
  bool ok = true;
  auto put = [&](const void* d, size_t n) { ok = ok && (n == 0 || std::fwrite(d, 1, n, f) == n); };
  const uint64_t n = h->level.size();
  const int64_t head[10] = {h->dim, h->metric, h->M, h->M0, h->efc, h->efs, static_cast<int64_t>(n), h->max_level,
                            h->entry == kNone ? -1 : static_cast<int64_t>(h->entry), h->active};
  put(&kFileMagic, 8);
  put(head, sizeof(head));
  put(&h->level_mult, 8);
  put(h->level.data(), n * sizeof(int));
  put(h->ids.data(), n * 8);
  put(h->vecs.data(), n * h->dim * sizeof(float));
  put(h->links0.data(), n * (h->M0 + 1) * 4);
  for (uint64_t s = 0; s < n; ++s) {
    put(h->up[s].data(), h->up[s].size() * 4);
    const uint64_t ml = h->meta[s].size();
    put(&ml, 8);
    put(h->meta[s].data(), ml);
  }
  ok = (std::fclose(f) == 0) && ok;
  return ok ? 0 : -3;
}

void* afb_hnsw_load(const char* path, uint64_t seed) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return nullptr;
  bool ok = true;
  auto get = [&](void* d, size_t n) { ok = ok && (n == 0 || std::fread(d, 1, n, f) == n); };
  uint64_t magic = 0;
  int64_t head[10] = {0};
  get(&magic, 8);
  get(head, sizeof(head));
  if (!ok || magic != kFileMagic || head[0] <= 0 || head[2] < 2 || head[3] < head[2] || head[6] < 0 ||
      head[6] > (1ll << 31)) {
    std::fclose(f);
    return nullptr;
  }
  Hnsw* h = new Hnsw();
  h->dim = static_cast<int>(head[0]); h->metric = static_cast<int>(head[1]); h->M = static_cast<int>(head[2]);
  h->M0 = static_cast<int>(head[3]); h->efc = static_cast<int>(head[4]); h->efs = static_cast<int>(head[5]);
  const uint64_t n = static_cast<uint64_t>(head[6]);
  h->max_level = static_cast<int>(head[7]);
  h->entry = head[8] < 0 ? kNone : static_cast<uint32_t>(head[8]);
  h->active = head[9];
  get(&h->level_mult, 8);
  h->level.resize(n); h->ids.resize(n); h->vecs.resize(n * h->dim); h->links0.resize(n * (h->M0 + 1));
  h->up.resize(n); h->meta.resize(n);
  get(h->level.data(), n * sizeof(int));
  get(h->ids.data(), n * 8);
  get(h->vecs.data(), n * h->dim * sizeof(float));
  get(h->links0.data(), n * (h->M0 + 1) * 4);
  for (uint64_t s = 0; s < n && ok; ++s) {
    if (h->level[s] > 30) { ok = false; break; }
    h->up[s].resize(h->level[s] > 0 ? static_cast<size_t>(h->level[s]) * (h->M + 1) : 0);
    get(h->up[s].data(), h->up[s].size() * 4);
    uint64_t ml = 0;
    get(&ml, 8);
    if (!ok || ml > (1ull << 30)) { ok = false; break; }
    h->meta[s].resize(ml);
    get(h->meta[s].data(), ml);
    if (h->level[s] >= 0) h->slot_of[h->ids[s]] = static_cast<uint32_t>(s);
    else h->free_slots.push_back(static_cast<uint32_t>(s));
  }
  std::fclose(f);
  h->rng.seed(seed);
  if (!ok || afb_hnsw_check(h) != 0) {
    delete h;
    return nullptr;
  }
  return h;
}

}  // extern "C"
