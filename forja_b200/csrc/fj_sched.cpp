// Continuous-batching admission and prompt-budget policy on the host (reference:
// crates/forja-serve/src/scheduler.rs:16-196 SchedulerPolicy, crates/forja-host/src/prompt.rs:20-41
// PromptChunking, crates/forja-serve/src/engine/continuous/batch.rs:1139-1152 reservations_fit,
// crates/forja-sdk/src/nn/blocks.rs:892-911 chunked prefill plan).
//
// The policy is integer bookkeeping that runs once per step, so it stays on the host like the
// reference's; what it decides (which requests enter, which bucket decodes, how many prompt tokens
// each prefilling lane gets) feeds fj_kvpool_reserve and fj_pack_step. Layout: the waiting line is
// a vector consumed from a moving head (admission pops near the front), the prompt ledger is a
// vector kept sorted by request id (round-robin = binary search for the cursor, then wrap).
#include <algorithm>
#include <cstdint>
#include <new>
#include <utility>
#include <vector>

#include "../../include/forja_cuda.h"

namespace {

constexpr uint8_t kBypassLimit = 8;  // scheduler.rs:3

struct Waiting {
  uint64_t id, reserved_tokens;
  uint8_t bypasses;
};

uint32_t floor_to(uint32_t value, uint32_t piece) { return value - value % piece; }

}  // namespace

struct fj_sched {
  std::vector<Waiting> line;  // live entries are line[head..]
  size_t head = 0;
  std::vector<std::pair<uint64_t, uint32_t>> ledger;  // (request id, prompt tokens left), ascending ids
  std::vector<uint32_t> buckets;                      // ascending, unique
  size_t active_limit = 0, prefill_limit = 0, active = 0;
  uint32_t busy_budget = 0, idle_budget = 0, piece = 1;
  bool merged = false, has_cursor = false;
  uint64_t cursor = 0;  // id served last by prompt_batch

  size_t waiting() const { return line.size() - head; }
  Waiting& at(size_t i) { return line[head + i]; }
  void compact() {
    if (head > 64 && head * 2 > line.size()) { line.erase(line.begin(), line.begin() + static_cast<ptrdiff_t>(head)); head = 0; }
  }
  void remove(size_t i) {
    if (i == 0) { ++head; compact(); }
    else line.erase(line.begin() + static_cast<ptrdiff_t>(head + i));
  }
  std::vector<std::pair<uint64_t, uint32_t>>::iterator find(uint64_t id) {
    auto it = std::lower_bound(ledger.begin(), ledger.end(), id, [](const std::pair<uint64_t, uint32_t>& e, uint64_t key) { return e.first < key; });
    return it != ledger.end() && it->first == id ? it : ledger.end();
  }
};

extern "C" {

uint32_t fj_prompt_chunk_work(uint32_t piece, uint32_t remaining, uint32_t allowance) {
  if (piece == 0) return 0;
  return remaining <= allowance ? remaining : floor_to(allowance, piece);
}

uint32_t fj_prompt_chunk_merged_work(uint32_t piece, uint32_t remaining, uint32_t allowance) {
  if (piece == 0) return 0;
  const uint32_t available = std::min(remaining, allowance);
  return remaining < piece ? available : floor_to(available, piece);
}

int32_t fj_sched_create(const uint32_t* buckets, uint32_t bucket_count, uint64_t active_limit, uint64_t prefill_limit, uint32_t prompt_budget,
                        uint32_t idle_prompt_budget, fj_sched** out) {
  if (!out || (bucket_count && !buckets)) return FJ_INVALID_INPUT;
  std::vector<uint32_t> sorted(buckets, buckets + bucket_count);
  std::sort(sorted.begin(), sorted.end());
  sorted.erase(std::unique(sorted.begin(), sorted.end()), sorted.end());
  // "decode buckets must span the active-lane ceiling" / "prefill limits must be positive"
  if (sorted.empty() || sorted.front() != 1 || static_cast<uint64_t>(sorted.back()) < active_limit) return FJ_INVALID_INPUT;
  if (prefill_limit == 0 || prompt_budget == 0 || idle_prompt_budget == 0) return FJ_INVALID_INPUT;
  fj_sched* s = new (std::nothrow) fj_sched();
  if (!s) return FJ_ALLOCATION_FAILED;
  s->buckets.swap(sorted);
  s->active_limit = static_cast<size_t>(active_limit);
  s->prefill_limit = static_cast<size_t>(prefill_limit);
  s->busy_budget = prompt_budget;
  s->idle_budget = idle_prompt_budget;
  s->piece = std::min(prompt_budget, idle_prompt_budget);
  *out = s;
  return FJ_OK;
}

void fj_sched_destroy(fj_sched* s) { delete s; }

void fj_sched_set_prompt_chunk_multiple(fj_sched* s, uint32_t multiple) {
  if (!s || multiple == 0) return;
  s->piece = multiple;
  s->merged = true;
}

void fj_sched_enqueue(fj_sched* s, uint64_t id, uint64_t reserved_tokens) {
  if (s) s->line.push_back(Waiting{id, reserved_tokens, 0});
}

void fj_sched_reconcile_active(fj_sched* s, uint64_t active) {
  if (s) s->active = static_cast<size_t>(std::min<uint64_t>(active, s->active_limit));
}

void fj_sched_complete(fj_sched* s, uint64_t id) {
  if (!s) return;
  auto it = s->find(id);
  if (it != s->ledger.end()) s->ledger.erase(it);
  if (s->active) --s->active;
}

void fj_sched_retry_admission(fj_sched* s, uint64_t id, uint64_t reserved_tokens) {
  if (!s) return;
  if (s->active) --s->active;
  // back to the very front, and nobody may overtake it any more
  const Waiting w{id, reserved_tokens, kBypassLimit};
  if (s->head > 0) s->line[--s->head] = w;
  else s->line.insert(s->line.begin(), w);
}

uint64_t fj_sched_admit(fj_sched* s, fj_sched_reserve_fn reserve, void* user, uint64_t* ids, uint64_t cap) {
  if (!s || !reserve) return 0;
  uint64_t admitted = 0;
  while (s->active < s->active_limit && s->waiting() != 0) {
    size_t pick = 0;
    const Waiting front = s->at(0);
    if (!reserve(user, front.id, front.reserved_tokens)) {
      if (front.bypasses >= kBypassLimit) break;
      // the first strictly smaller request behind the head that can be reserved overtakes it
      pick = SIZE_MAX;
      for (size_t i = 1; i < s->waiting(); ++i) {
        const Waiting& w = s->at(i);
        if (w.reserved_tokens < front.reserved_tokens && reserve(user, w.id, w.reserved_tokens)) { pick = i; break; }
      }
      if (pick == SIZE_MAX) break;
      if (s->at(0).bypasses != UINT8_MAX) ++s->at(0).bypasses;
    }
    const uint64_t id = s->at(pick).id;
    s->remove(pick);
    ++s->active;
    if (ids && admitted < cap) ids[admitted] = id;
    ++admitted;
  }
  return admitted;
}

namespace {
struct PageBudget { uint32_t page_tokens; uint64_t* free_pages; };
int32_t reserve_pages(void* user, uint64_t, uint64_t reserved_tokens) {
  auto* b = static_cast<PageBudget*>(user);
  const uint64_t pages = reserved_tokens / b->page_tokens + (reserved_tokens % b->page_tokens ? 1 : 0);
  if (pages > *b->free_pages) return 0;
  *b->free_pages -= pages;
  return 1;
}
}  // namespace

uint64_t fj_sched_admit_pages(fj_sched* s, uint32_t page_tokens, uint64_t* free_pages, uint64_t* ids, uint64_t cap) {
  if (!s || !free_pages || page_tokens == 0) return 0;
  PageBudget budget{page_tokens, free_pages};
  return fj_sched_admit(s, reserve_pages, &budget, ids, cap);
}

int64_t fj_sched_decode_bucket(const fj_sched* s, const uint32_t* slots, uint64_t count) {
  if (!s || count == 0 || !slots) return -1;
  uint32_t highest = 0;
  for (uint64_t i = 0; i < count; ++i) highest = std::max(highest, slots[i]);
  const uint32_t needed = highest == UINT32_MAX ? highest : highest + 1;  // saturating slot + 1
  auto it = std::lower_bound(s->buckets.begin(), s->buckets.end(), needed);
  return it == s->buckets.end() ? -1 : static_cast<int64_t>(*it);
}

void fj_sched_ready_prompt(fj_sched* s, uint64_t id, uint32_t tokens) {
  if (!s) return;
  auto it = std::lower_bound(s->ledger.begin(), s->ledger.end(), id, [](const std::pair<uint64_t, uint32_t>& e, uint64_t key) { return e.first < key; });
  if (it != s->ledger.end() && it->first == id) it->second = tokens;
  else s->ledger.insert(it, std::make_pair(id, tokens));
}

uint64_t fj_sched_prompt_batch(fj_sched* s, int32_t decoding, uint64_t* ids, uint32_t* spend, uint64_t cap) {
  if (!s) return 0;
  uint32_t budget = decoding ? s->busy_budget : s->idle_budget;
  // visit order: ids after the cursor first, then wrap; fixed before anything is removed
  std::vector<uint64_t> order;
  order.reserve(s->ledger.size());
  size_t first = 0;
  if (s->has_cursor) {
    first = static_cast<size_t>(std::upper_bound(s->ledger.begin(), s->ledger.end(), s->cursor, [](uint64_t key, const std::pair<uint64_t, uint32_t>& e) { return key < e.first; }) - s->ledger.begin());
  }
  for (size_t i = 0; i < s->ledger.size(); ++i) order.push_back(s->ledger[(first + i) % s->ledger.size()].first);
  uint64_t served = 0;
  for (uint64_t id : order) {
    if (served == s->prefill_limit) break;
    auto it = s->find(id);
    if (it == s->ledger.end()) continue;
    const uint32_t left = it->second;
    const uint32_t take = s->merged ? fj_prompt_chunk_merged_work(s->piece, left, budget) : fj_prompt_chunk_work(s->piece, left, budget);
    if (take == 0) break;
    if (ids && spend && served < cap) { ids[served] = id; spend[served] = take; }
    ++served;
    s->has_cursor = true;
    s->cursor = id;
    budget -= take;
    if (take == left) s->ledger.erase(it); else it->second = left - take;
  }
  return served;
}

uint64_t fj_sched_waiting(const fj_sched* s) { return s ? s->line.size() - s->head : 0; }
uint64_t fj_sched_active(const fj_sched* s) { return s ? s->active : 0; }

int32_t fj_reservations_fit(uint32_t page_tokens, uint32_t max_context, const uint64_t* reservations, uint64_t count) {
  if (page_tokens == 0 || (count && !reservations)) return 0;
  const uint64_t capacity = (static_cast<uint64_t>(max_context) + page_tokens - 1) / page_tokens;
  uint64_t pages = 0;
  for (uint64_t i = 0; i < count; ++i) {
    const uint64_t need = reservations[i] / page_tokens + (reservations[i] % page_tokens ? 1 : 0);
    if (need > UINT64_MAX - pages) return 0;  // checked_add
    pages += need;
  }
  return pages <= capacity ? 1 : 0;
}

uint64_t fj_prefill_plan(uint32_t sequence, uint32_t chunk, uint32_t tail_chunk, uint32_t* out, uint64_t cap) {
  if (sequence == 0 || chunk == 0) return 0;
  if (sequence < chunk) {
    if (out && cap) out[0] = sequence;
    return 1;
  }
  uint64_t pieces = 0;
  for (uint32_t left = sequence; left != 0;) {
    const uint32_t real = left >= chunk ? chunk : std::min(left, tail_chunk);
    if (real == 0) return 0;
    if (out && pieces < cap) out[pieces] = real;
    ++pieces;
    left -= real;
  }
  return pieces;
}

}  // extern "C"
