// Continuous-batching step scheduler (host side).
//
// Every model forward pass is one "step": a packed batch of decode items (one query token each, or k+1 when a
// speculative verify is pending) and prefill chunks.  Packing rules follow the reference's
// NativeGenerateCoordinator (zig/pkg/inference/src/runtime/scheduler/native_generate.zig:40-57, 353-470):
//   * decode items are admitted before prefill chunks,
//   * a step holds at most max_items items and max_query_tokens query tokens,
//   * the first item considered (the leader) is always admitted, whatever the budgets say,
//   * after `decode_streak` consecutive decode-only steps while prefill work is waiting, the next step admits
//     prefill chunks first,
//   * prompts are prefilled in chunks of at most prefill_chunk tokens; a tail smaller than min_chunk is only
//     split off when it is the whole remainder,
//   * an optional KV-block budget skips items whose block estimate does not fit (leader exempt),
//   * a failed step returns every claimed item to the state it had before the claim.
// The reference's defaults are 16 items / 512 query tokens / chunk 256 (min 32) / streak 4; the B200 engine
// raises the budgets but keeps the rules.
#include <stdint.h>

#include <algorithm>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

enum Phase : int { kWaiting = 0, kPrefill = 1, kDecode = 2, kFinished = 3 };

struct Request {
  int64_t id;
  int prompt_len;
  int max_new_tokens;
  int prompt_done = 0;
  int generated = 0;
  int decode_width = 1;  // query tokens of the next decode step (k+1 for a speculative verify)
  Phase phase = kWaiting;
  bool in_flight = false;
  int claimed_q = 0;
  bool atomic_prefill = false;  // the whole prompt goes into one step (prompts whose tokens attend to later ones)
};

struct Sched {
  int max_items, max_query_tokens, prefill_chunk, min_chunk, decode_streak_limit;
  int max_kv_blocks;  // <= 0: no budget
  int page;
  int max_queue;
  std::deque<int64_t> order;  // admission order
  std::unordered_map<int64_t, Request> reqs;
  std::vector<int64_t> claimed;
  int decode_streak = 0;
  std::mutex mu;
  // counters (same meaning as the reference's Stats)
  uint64_t step_batches_total = 0, step_prefill_items_total = 0, step_decode_items_total = 0,
           step_query_tokens_total = 0, step_singleton_batches_total = 0, step_kv_block_skips_total = 0,
           queue_full_total = 0, failed_steps_total = 0;
};

int blocks_for(const Sched* s, int tokens) { return (tokens + s->page - 1) / s->page; }

}  // namespace

extern "C" {

void* afb_sched_create(int max_items, int max_query_tokens, int prefill_chunk, int min_chunk, int decode_streak,
                       int max_kv_blocks, int page, int max_queue) {
  Sched* s = new Sched();
  s->max_items = std::max(max_items, 1);
  s->max_query_tokens = std::max(max_query_tokens, 1);
  s->prefill_chunk = std::max(prefill_chunk, 1);
  s->min_chunk = std::max(min_chunk, 1);
  s->decode_streak_limit = std::max(decode_streak, 1);
  s->max_kv_blocks = max_kv_blocks;
  s->page = std::max(page, 1);
  s->max_queue = max_queue;
  return s;
}

void afb_sched_destroy(void* h) { delete static_cast<Sched*>(h); }

// 0 ok, -1 duplicate id / bad args, -2 queue full (the caller answers HTTP 503).
int afb_sched_admit(void* h, int64_t id, int prompt_len, int max_new_tokens) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  if (prompt_len <= 0 || s->reqs.count(id)) return -1;
  if (s->max_queue > 0 && static_cast<int>(s->reqs.size()) >= s->max_queue) {
    ++s->queue_full_total;
    return -2;
  }
  Request r;
  r.id = id;
  r.prompt_len = prompt_len;
  r.max_new_tokens = max_new_tokens;
  s->reqs.emplace(id, r);
  s->order.push_back(id);
  return 0;
}

// As afb_sched_admit for a request whose first `prompt_done` prompt tokens are already in the KV cache (a shared
// prefix): prefill starts after them.  At least one prompt token must remain so the first output token has logits.
int afb_sched_admit_prefilled(void* h, int64_t id, int prompt_len, int max_new_tokens, int prompt_done) {
  if (prompt_done < 0 || prompt_done >= prompt_len) return -1;
  const int rc = afb_sched_admit(h, id, prompt_len, max_new_tokens);
  if (rc != 0) return rc;
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  s->reqs[id].prompt_done = prompt_done;
  return 0;
}

// A request flagged here is never prefilled in chunks: its prompt is claimed whole, as the leader of a step if
// it does not fit beside other items.
int afb_sched_set_atomic_prefill(void* h, int64_t id, int on) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  it->second.atomic_prefill = on != 0;
  return 0;
}

int afb_sched_set_decode_width(void* h, int64_t id, int width) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end() || width < 1) return -1;
  it->second.decode_width = width;
  return 0;
}

// Packs the next step.  Outputs, per item: request id, mode (0 decode, 1 prefill), query length, and the
// number of tokens of the sequence already in the KV cache before this step (kv offset).
// Returns the number of items (0 = nothing to do), or -1 if a step is already in flight.
int afb_sched_claim_step(void* h, int64_t* ids, int* modes, int* q_lens, int* kv_before, int max_out) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  if (!s->claimed.empty()) return -1;
  int items = 0, qtok = 0, kvb = 0, n_dec = 0, n_pre = 0;
  bool any_prefill_pending = false, any_decode_pending = false;
  for (int64_t id : s->order) {
    const Request& r = s->reqs[id];
    if (r.phase == kDecode) any_decode_pending = true;
    if (r.phase == kWaiting || r.phase == kPrefill) any_prefill_pending = true;
  }
  const bool prefill_first =
      any_prefill_pending && (!any_decode_pending || s->decode_streak >= s->decode_streak_limit);

  auto try_add = [&](Request& r, int mode, int q, int kv_prev) -> bool {
    const bool leader = items == 0;
    if (!leader) {
      if (items >= s->max_items || items >= max_out) return false;
      if (qtok + q > s->max_query_tokens) return false;
    }
    const int est = blocks_for(s, kv_prev + q);
    if (s->max_kv_blocks > 0 && !leader && kvb + est > s->max_kv_blocks) {
      ++s->step_kv_block_skips_total;
      return false;
    }
    ids[items] = r.id; modes[items] = mode; q_lens[items] = q; kv_before[items] = kv_prev;
    ++items; qtok += q; kvb += est;
    r.in_flight = true; r.claimed_q = q;
    s->claimed.push_back(r.id);
    if (mode == 0) ++n_dec; else ++n_pre;
    return true;
  };
  auto add_decodes = [&]() {
    for (int64_t id : s->order) {
      Request& r = s->reqs[id];
      if (r.phase != kDecode || r.in_flight) continue;
      if (items >= std::min(s->max_items, max_out) && items > 0) break;
      try_add(r, 0, r.decode_width, r.prompt_len + r.generated - 1);
    }
  };
  auto add_prefills = [&]() {
    for (int64_t id : s->order) {
      Request& r = s->reqs[id];
      if ((r.phase != kWaiting && r.phase != kPrefill) || r.in_flight) continue;
      if (items >= std::min(s->max_items, max_out) && items > 0) break;
      const int remaining = r.prompt_len - r.prompt_done;
      int chunk = r.atomic_prefill ? remaining : std::min(remaining, s->prefill_chunk);
      if (items > 0) {
        const int room = s->max_query_tokens - qtok;
        if (room <= 0) break;
        if (chunk > room) {
          if (r.atomic_prefill) continue;  // waits for a step it can lead or fit into whole
          // Shrink to the budget, but never below min_chunk unless it finishes the prompt.
          if (room < s->min_chunk && room < remaining) continue;
          chunk = room;
        }
      }
      try_add(r, 1, chunk, r.prompt_done);
    }
  };
  if (prefill_first) { add_prefills(); add_decodes(); } else { add_decodes(); add_prefills(); }
  if (items == 0) return 0;
  ++s->step_batches_total;
  s->step_prefill_items_total += n_pre;
  s->step_decode_items_total += n_dec;
  s->step_query_tokens_total += qtok;
  if (items == 1) ++s->step_singleton_batches_total;
  if (n_pre == 0) ++s->decode_streak; else s->decode_streak = 0;
  return items;
}

// Reports the outcome of the claimed step.  tokens_out[i]: for a decode item the number of tokens the
// sequence grew by (1, or matched+1 after a speculative verify); for a prefill chunk that completed its prompt,
// 1 (the first sampled token), else 0.  finished[i] != 0 retires the request.
int afb_sched_complete_step(void* h, int n, const int64_t* ids, const int* tokens_out, const int* finished) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  for (int i = 0; i < n; ++i) {
    auto it = s->reqs.find(ids[i]);
    if (it == s->reqs.end()) continue;
    Request& r = it->second;
    if (!r.in_flight) continue;
    r.in_flight = false;
    if (r.phase == kDecode) {
      r.generated += tokens_out[i];
      r.decode_width = 1;
    } else {
      r.prompt_done += r.claimed_q;
      r.phase = kPrefill;
      if (r.prompt_done >= r.prompt_len) {
        r.phase = kDecode;
        r.generated += tokens_out[i];
      }
    }
    if (finished[i] || (r.max_new_tokens > 0 && r.generated >= r.max_new_tokens)) r.phase = kFinished;
    if (r.phase == kFinished) {
      s->order.erase(std::remove(s->order.begin(), s->order.end(), r.id), s->order.end());
      s->reqs.erase(it);
    }
  }
  s->claimed.clear();
  return 0;
}

// The forward pass failed: every claimed item goes back to where it was.
int afb_sched_fail_step(void* h) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  for (int64_t id : s->claimed) {
    auto it = s->reqs.find(id);
    if (it != s->reqs.end()) { it->second.in_flight = false; it->second.claimed_q = 0; }
  }
  s->claimed.clear();
  ++s->failed_steps_total;
  return 0;
}

int afb_sched_cancel(void* h, int64_t id) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  if (it->second.in_flight) return -2;
  s->order.erase(std::remove(s->order.begin(), s->order.end(), id), s->order.end());
  s->reqs.erase(it);
  return 0;
}

// out: waiting, prefill, decode, in_flight
void afb_sched_snapshot(void* h, int* out4) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
  for (auto& kv : s->reqs) {
    const Request& r = kv.second;
    if (r.phase == kWaiting) ++out4[0];
    else if (r.phase == kPrefill) ++out4[1];
    else if (r.phase == kDecode) ++out4[2];
    if (r.in_flight) ++out4[3];
  }
}

void afb_sched_stats(void* h, uint64_t* out8) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  out8[0] = s->step_batches_total; out8[1] = s->step_prefill_items_total; out8[2] = s->step_decode_items_total;
  out8[3] = s->step_query_tokens_total; out8[4] = s->step_singleton_batches_total;
  out8[5] = s->step_kv_block_skips_total; out8[6] = s->queue_full_total; out8[7] = s->failed_steps_total;
}

}  // extern "C"
