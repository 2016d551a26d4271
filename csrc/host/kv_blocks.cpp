// Paged KV-cache bookkeeping (host side): a pool of fixed-size blocks with reference counts and a free list,
// and one block table per sequence.  The cache tensors themselves live in GPU memory; this file only hands
// out block ids and slot numbers (slot = block * page + offset) that the kernels use.
//
// Behaviour mirrors the reference's KvPool / SequenceBlockTable / KvManager
// (zig/pkg/inference/src/runtime/kv/block.zig:27, block_table.zig:18-107, manager.zig:77-378):
//   attach            new empty sequence
//   attach_shared     new sequence sharing a prefix of a parent: whole blocks are shared by reference count,
//                     a partially filled last block is copied (copy-on-write pair returned to the caller)
//   append            reserve slots for n more tokens, all-or-nothing when the pool is exhausted
//   truncate          drop tail tokens (speculative-decoding rollback) and free emptied blocks
//   trim_window       release blocks that lie wholly before the sliding window
//   detach            release everything
#include <stdint.h>
#include <string.h>

#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

struct Sequence {
  std::vector<int> blocks;  // block id per page of the sequence; -1 once trimmed away
  int len = 0;              // tokens written
  int first_live_block = 0; // blocks before this index were trimmed
};

struct Pool {
  int num_blocks;
  int page;
  std::vector<int> refcount;
  std::vector<int> free_list;
  std::unordered_map<int64_t, Sequence> seqs;
  std::vector<std::pair<int, int>> cow;  // pending (src, dst) block copies
  std::mutex mu;
  uint64_t acquired_total = 0, released_total = 0, oom_total = 0;

  int acquire() {
    if (free_list.empty()) return -1;
    int b = free_list.back();
    free_list.pop_back();
    refcount[b] = 1;
    ++acquired_total;
    return b;
  }
  void release(int b) {
    if (b < 0) return;
    if (--refcount[b] == 0) {
      free_list.push_back(b);
      ++released_total;
    }
  }
};

}  // namespace

extern "C" {

void* afb_kv_create(int num_blocks, int page) {
  if (num_blocks <= 0 || page <= 0) return nullptr;
  Pool* p = new Pool();
  p->num_blocks = num_blocks;
  p->page = page;
  p->refcount.assign(num_blocks, 0);
  p->free_list.reserve(num_blocks);
  // Hand out low block ids first.
  for (int b = num_blocks - 1; b >= 0; --b) p->free_list.push_back(b);
  return p;
}

void afb_kv_destroy(void* h) { delete static_cast<Pool*>(h); }

int afb_kv_free_blocks(void* h) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  return static_cast<int>(p->free_list.size());
}

int afb_kv_num_sequences(void* h) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  return static_cast<int>(p->seqs.size());
}

int afb_kv_attach(void* h, int64_t seq) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  if (p->seqs.count(seq)) return -1;
  p->seqs.emplace(seq, Sequence());
  return 0;
}

// Returns 0, -1 (bad ids / prefix longer than parent) or -2 (pool exhausted; nothing changed).
int afb_kv_attach_shared(void* h, int64_t seq, int64_t parent, int prefix_tokens) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(parent);
  if (it == p->seqs.end() || p->seqs.count(seq)) return -1;
  const Sequence& par = it->second;
  if (prefix_tokens < 0 || prefix_tokens > par.len || par.first_live_block > 0) return -1;
  Sequence s;
  const int full = prefix_tokens / p->page;
  const int rem = prefix_tokens % p->page;
  int copy_dst = -1;
  if (rem) {
    copy_dst = p->acquire();
    if (copy_dst < 0) {
      ++p->oom_total;
      return -2;
    }
  }
  for (int i = 0; i < full; ++i) {
    ++p->refcount[par.blocks[i]];
    s.blocks.push_back(par.blocks[i]);
  }
  if (rem) {
    s.blocks.push_back(copy_dst);
    p->cow.emplace_back(par.blocks[full], copy_dst);
  }
  s.len = prefix_tokens;
  p->seqs.emplace(seq, std::move(s));
  return 0;
}

// Drains up to `max` pending copy-on-write pairs into src/dst; returns how many were written.
int afb_kv_take_cow(void* h, int* src, int* dst, int max) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  int n = 0;
  while (n < max && !p->cow.empty()) {
    src[n] = p->cow.back().first;
    dst[n] = p->cow.back().second;
    p->cow.pop_back();
    ++n;
  }
  return n;
}

// Reserves slots for n_tokens more tokens; writes their slot ids to out_slots (may be null).
// Returns 0, -1 (unknown sequence) or -2 (pool exhausted; the sequence is unchanged).
int afb_kv_append(void* h, int64_t seq, int n_tokens, int* out_slots) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end() || n_tokens < 0) return -1;
  Sequence& s = it->second;
  const int new_len = s.len + n_tokens;
  const int need = (new_len + p->page - 1) / p->page;
  const int have = static_cast<int>(s.blocks.size());
  // A shared tail block must not be appended into: copy it first.
  const bool tail_shared = have > 0 && (s.len % p->page) != 0 && s.blocks[have - 1] >= 0 &&
                           p->refcount[s.blocks[have - 1]] > 1 && n_tokens > 0;
  const int extra = (need > have ? need - have : 0) + (tail_shared ? 1 : 0);
  if (extra > static_cast<int>(p->free_list.size())) {
    ++p->oom_total;
    return -2;
  }
  if (tail_shared) {
    const int nb = p->acquire();
    p->cow.emplace_back(s.blocks[have - 1], nb);
    p->release(s.blocks[have - 1]);
    s.blocks[have - 1] = nb;
  }
  for (int i = have; i < need; ++i) s.blocks.push_back(p->acquire());
  if (out_slots) {
    for (int t = 0; t < n_tokens; ++t) {
      const int pos = s.len + t;
      out_slots[t] = s.blocks[pos / p->page] * p->page + pos % p->page;
    }
  }
  s.len = new_len;
  return 0;
}

int afb_kv_truncate(void* h, int64_t seq, int new_len) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -1;
  Sequence& s = it->second;
  if (new_len < 0 || new_len > s.len) return -1;
  // Tokens whose blocks the sliding window already released cannot become the tail again (their block is gone):
  // only a full reset may cut below the trimmed boundary.
  if (new_len != 0 && new_len < s.first_live_block * p->page) return -1;
  const int keep = (new_len + p->page - 1) / p->page;
  while (static_cast<int>(s.blocks.size()) > keep) {
    p->release(s.blocks.back());
    s.blocks.pop_back();
  }
  if (s.first_live_block > keep) s.first_live_block = keep;
  s.len = new_len;
  return 0;
}

// Releases blocks whose every token is older than the attention window AND older than the 64-key tile that
// contains the window start (the attention kernel loads whole tiles).  Returns the number of blocks released.
int afb_kv_trim_window(void* h, int64_t seq, int window) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end() || window <= 0) return -1;
  Sequence& s = it->second;
  int first_needed = s.len - window;  // oldest key any future query can see is >= this
  if (first_needed <= 0) return 0;
  first_needed = first_needed / 64 * 64;
  const int drop_until = first_needed / p->page;
  int released = 0;
  for (int i = s.first_live_block; i < drop_until && i < static_cast<int>(s.blocks.size()); ++i) {
    if (s.blocks[i] >= 0) {
      p->release(s.blocks[i]);
      s.blocks[i] = -1;
      ++released;
    }
  }
  if (drop_until > s.first_live_block) s.first_live_block = drop_until;
  return released;
}

int afb_kv_len(void* h, int64_t seq) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  return it == p->seqs.end() ? -1 : it->second.len;
}

// Copies the block table (trimmed entries become 0, a valid id the kernel never dereferences for live keys).
// Returns the number of blocks, or -1.
int afb_kv_block_table(void* h, int64_t seq, int* out, int max) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -1;
  const Sequence& s = it->second;
  const int n = static_cast<int>(s.blocks.size());
  for (int i = 0; i < n && i < max; ++i) out[i] = s.blocks[i] < 0 ? 0 : s.blocks[i];
  return n;
}

int afb_kv_detach(void* h, int64_t seq) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -1;
  for (int b : it->second.blocks) p->release(b);
  p->seqs.erase(it);
  return 0;
}

int afb_kv_refcount(void* h, int block) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  if (block < 0 || block >= p->num_blocks) return -1;
  return p->refcount[block];
}

void afb_kv_stats(void* h, uint64_t* out3) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  out3[0] = p->acquired_total;
  out3[1] = p->released_total;
  out3[2] = p->oom_total;
}

// Batched helper for the decode hot loop: for each sequence append one token and emit its slot, its new
// length and its block-table row (row pitch max_blocks).  Stops at the first failure and returns its index
// (n on success); sequences before it stay appended.
int afb_kv_append_batch(void* h, const int64_t* seqs, const int* n_tokens, int n, int* out_slots, int* out_lens,
                        int* out_tables, int max_blocks) {
  Pool* p = static_cast<Pool*>(h);
  int slot_off = 0;
  for (int i = 0; i < n; ++i) {
    const int rc = afb_kv_append(h, seqs[i], n_tokens[i], out_slots + slot_off);
    if (rc != 0) return i;
    slot_off += n_tokens[i];
    std::lock_guard<std::mutex> g(p->mu);
    const Sequence& s = p->seqs[seqs[i]];
    out_lens[i] = s.len;
    if (out_tables) {
      const int nb = static_cast<int>(s.blocks.size());
      for (int j = 0; j < nb && j < max_blocks; ++j)
        out_tables[static_cast<size_t>(i) * max_blocks + j] = s.blocks[j] < 0 ? 0 : s.blocks[j];
    }
  }
  return n;
}

}  // extern "C"
