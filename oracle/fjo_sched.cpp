// CPU oracle: continuous-batching policy and ragged-batch packing, restating
// crates/forja-serve/src/scheduler.rs:16-196, crates/forja-host/src/prompt.rs:20-41,
// crates/forja-serve/src/engine/continuous/batch.rs:1139-1152,
// crates/forja-sdk/src/nn/blocks.rs:892-911 and the lane metadata of
// crates/forja-host/src/lib.rs:4977-5065. Test infrastructure only; see fjo.h.
#include "fjo.h"

#include <algorithm>
#include <deque>
#include <functional>
#include <map>
#include <vector>

namespace {
const uint8_t MAX_BYPASSES = 8;
struct Admission { uint64_t id; uint64_t reserved_tokens; };
struct Queued { Admission admission; uint8_t bypasses; };
}  // namespace

struct fjo_sched {
  std::deque<Queued> queue;
  std::map<uint64_t, uint32_t> prompt;
  std::vector<uint32_t> buckets;
  size_t active_limit, prefill_limit;
  uint32_t prompt_budget, idle_prompt_budget;
  uint32_t piece;
  bool merge_prompt_chunks = false;
  bool has_last = false;
  uint64_t last_prompt = 0;
  size_t active = 0;

  // admission_candidate, scheduler.rs:125-152
  long candidate(const std::function<bool(Admission)>& reserve) {
    if (queue.empty()) return -1;
    Admission head = queue.front().admission;
    if (reserve(head)) return 0;
    if (queue.front().bypasses >= MAX_BYPASSES) return -1;
    long found = -1;
    for (size_t i = 1; i < queue.size(); ++i) {
      if (queue[i].admission.reserved_tokens < head.reserved_tokens && reserve(queue[i].admission)) { found = static_cast<long>(i); break; }
    }
    if (found >= 0 && queue.front().bypasses < 255) queue.front().bypasses += 1;
    return found;
  }
  // admit, scheduler.rs:109-123
  size_t admit(const std::function<bool(Admission)>& reserve, uint64_t* ids, size_t cap) {
    size_t n = 0;
    while (active < active_limit && !queue.empty()) {
      long index = candidate(reserve);
      if (index < 0) break;
      Queued q = queue[index];
      queue.erase(queue.begin() + index);
      active += 1;
      if (n < cap) ids[n] = q.admission.id;
      ++n;
    }
    return n;
  }
};

extern "C" {

uint32_t fjo_chunk_work(uint32_t piece, uint32_t remaining, uint32_t allowance) {
  return remaining <= allowance ? remaining : allowance / piece * piece;
}
uint32_t fjo_chunk_merged_work(uint32_t piece, uint32_t remaining, uint32_t allowance) {
  uint32_t available = remaining < allowance ? remaining : allowance;
  return remaining < piece ? available : available / piece * piece;
}

int fjo_sched_new(const uint32_t* buckets, size_t n, size_t active_limit, size_t prefill_limit,
                  uint32_t prompt_budget, uint32_t idle_prompt_budget, fjo_sched** out) {
  std::vector<uint32_t> b(buckets, buckets + n);
  std::sort(b.begin(), b.end());
  b.erase(std::unique(b.begin(), b.end()), b.end());
  if (b.empty() || b.front() != 1 || b.back() < active_limit) return FJO_INVALID_INPUT;
  if (prefill_limit == 0 || prompt_budget == 0 || idle_prompt_budget == 0) return FJO_INVALID_INPUT;
  auto* s = new fjo_sched();
  s->buckets = b;
  s->active_limit = active_limit;
  s->prefill_limit = prefill_limit;
  s->prompt_budget = prompt_budget;
  s->idle_prompt_budget = idle_prompt_budget;
  s->piece = std::min(prompt_budget, idle_prompt_budget);
  *out = s;
  return FJO_OK;
}
void fjo_sched_free(fjo_sched* s) { delete s; }
void fjo_sched_chunk_multiple(fjo_sched* s, uint32_t multiple) {
  if (multiple != 0) { s->piece = multiple; s->merge_prompt_chunks = true; }
}
void fjo_sched_enqueue(fjo_sched* s, uint64_t id, uint64_t reserved_tokens) { s->queue.push_back({{id, reserved_tokens}, 0}); }
void fjo_sched_reconcile_active(fjo_sched* s, size_t active) { s->active = std::min(active, s->active_limit); }
void fjo_sched_complete(fjo_sched* s, uint64_t id) { s->prompt.erase(id); if (s->active > 0) s->active -= 1; }
void fjo_sched_retry_admission(fjo_sched* s, uint64_t id, uint64_t reserved_tokens) {
  if (s->active > 0) s->active -= 1;
  s->queue.push_front({{id, reserved_tokens}, MAX_BYPASSES});
}
size_t fjo_sched_admit_below(fjo_sched* s, uint64_t reserve_below, uint64_t* ids, size_t cap) {
  return s->admit([&](Admission a) { return a.reserved_tokens < reserve_below; }, ids, cap);
}
size_t fjo_sched_admit_pages(fjo_sched* s, uint32_t page_tokens, uint64_t* free_pages, uint64_t* ids, size_t cap) {
  return s->admit([&](Admission a) {
    uint64_t need = (a.reserved_tokens + page_tokens - 1) / page_tokens;
    if (need > *free_pages) return false;
    *free_pages -= need;
    return true;
  }, ids, cap);
}
// decode_bucket, scheduler.rs:89-95
int64_t fjo_sched_decode_bucket(fjo_sched* s, const uint32_t* slots, size_t n) {
  if (n == 0) return -1;
  uint32_t needed = 0;
  for (size_t i = 0; i < n; ++i) { uint32_t v = slots[i] == 0xFFFFFFFFu ? slots[i] : slots[i] + 1; needed = std::max(needed, v); }
  for (uint32_t b : s->buckets) if (b >= needed) return b;
  return -1;
}
void fjo_sched_ready_prompt(fjo_sched* s, uint64_t id, uint32_t tokens) { s->prompt[id] = tokens; }
// prompt_batch, scheduler.rs:158-195
size_t fjo_sched_prompt_batch(fjo_sched* s, int decoding, uint64_t* ids_out, uint32_t* spend_out, size_t cap) {
  uint32_t remaining = decoding ? s->prompt_budget : s->idle_prompt_budget;
  std::vector<uint64_t> ids;
  for (auto& kv : s->prompt) ids.push_back(kv.first);
  if (s->has_last) {
    size_t next = std::upper_bound(ids.begin(), ids.end(), s->last_prompt) - ids.begin();
    std::rotate(ids.begin(), ids.begin() + next, ids.end());
  }
  size_t n = 0;
  for (uint64_t id : ids) {
    if (n == s->prefill_limit) break;
    auto it = s->prompt.find(id);
    if (it == s->prompt.end()) continue;
    uint32_t tokens = it->second;
    uint32_t spend = s->merge_prompt_chunks ? fjo_chunk_merged_work(s->piece, tokens, remaining) : fjo_chunk_work(s->piece, tokens, remaining);
    if (spend == 0) break;
    if (n < cap) { ids_out[n] = id; spend_out[n] = spend; }
    ++n;
    s->has_last = true;
    s->last_prompt = id;
    remaining -= spend;
    if (spend == tokens) s->prompt.erase(id); else s->prompt[id] = tokens - spend;
  }
  return n;
}

int fjo_reservations_fit(uint32_t page_tokens, uint32_t max_context, const uint64_t* reservations, size_t n) {
  uint64_t pt = page_tokens;
  uint64_t capacity = (static_cast<uint64_t>(max_context) + pt - 1) / pt;
  uint64_t total = 0;
  for (size_t i = 0; i < n; ++i) {
    uint64_t pages = reservations[i] / pt + (reservations[i] % pt != 0 ? 1 : 0);
    if (__builtin_add_overflow(total, pages, &total)) return 0;
  }
  return total <= capacity ? 1 : 0;
}

size_t fjo_prefill_plan(uint32_t sequence, uint32_t chunk, uint32_t tail_chunk, uint32_t* out, size_t cap) {
  if (sequence == 0) return 0;
  size_t n = 0;
  uint32_t remaining = sequence;
  if (remaining < chunk) { if (cap > 0) out[0] = remaining; return 1; }
  while (remaining > 0) {
    uint32_t real = remaining >= chunk ? chunk : std::min(remaining, tail_chunk);
    if (real == 0 || real > chunk) return 0;
    if (n < cap) out[n] = real;
    ++n;
    remaining -= real;
  }
  return n;
}

int64_t fjo_pack_step(const uint32_t* lanes_start, const uint32_t* lanes_tokens,
                      const uint32_t* lanes_logical_len, size_t lanes, const uint32_t* tables,
                      size_t table_pages, uint32_t page_tokens, uint32_t* logical_lengths,
                      uint32_t* query_starts, uint32_t* absolute_positions, uint32_t* activity,
                      uint32_t* cu_seqlens, uint32_t* positions, uint32_t* slot_mapping,
                      uint32_t* row_lane, size_t rows_cap) {
  size_t rows = 0;
  cu_seqlens[0] = 0;
  for (size_t lane = 0; lane < lanes; ++lane) {
    uint32_t tokens = lanes_tokens[lane];
    if (tokens != 0) {
      uint32_t start = lanes_start[lane];
      uint64_t end = static_cast<uint64_t>(start) + tokens;
      if (end - 1 > 0xFFFFFFFFull) return -1;  // "batch absolute position overflowed"
      logical_lengths[lane] = lanes_logical_len[lane];
      query_starts[lane] = start;
      absolute_positions[lane] = static_cast<uint32_t>(end - 1);
      activity[lane] = 1;
      for (uint32_t t = 0; t < tokens; ++t) {
        if (rows >= rows_cap) return -1;
        uint64_t position = static_cast<uint64_t>(start) + t;
        uint64_t logical_page = position / page_tokens;
        uint32_t slot = 0xFFFFFFFFu;
        if (logical_page < table_pages) {
          uint32_t page = tables[(lane * table_pages + logical_page) * 2];
          uint32_t generation = tables[(lane * table_pages + logical_page) * 2 + 1];
          if (generation != 0xFFFFFFFFu) slot = page * page_tokens + static_cast<uint32_t>(position % page_tokens);
        }
        positions[rows] = static_cast<uint32_t>(position);
        slot_mapping[rows] = slot;
        row_lane[rows] = static_cast<uint32_t>(lane);
        ++rows;
      }
    } else {
      logical_lengths[lane] = 0;
      query_starts[lane] = 0;
      absolute_positions[lane] = 0;
      activity[lane] = 0;
    }
    cu_seqlens[lane + 1] = static_cast<uint32_t>(rows);
  }
  return static_cast<int64_t>(rows);
}

}  // extern "C"
