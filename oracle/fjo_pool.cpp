// CPU oracle: paged-KV allocator, restating crates/forja-core/src/paged_pool.rs (PagePool,
// PagedSequence, SequenceCheckpoint, PagedSlotBanks). Single-threaded restatement: the
// reference's mutexes guard the same state transitions. Test infrastructure only; see fjo.h.
#include "fjo.h"

#include <algorithm>
#include <cstdint>
#include <vector>

namespace {

const uint32_t POISON_GENERATION = 0xFFFFFFFFu;
enum Lifecycle { FREE, ALLOCATED, RETIRING };

struct PageState { uint32_t generation = 0; uint32_t references = 0; uint64_t last_use = 0; Lifecycle lifecycle = FREE; };
struct PageLease { uint32_t index; uint32_t generation; bool operator==(const PageLease& o) const { return index == o.index && generation == o.generation; } };
struct Memory { uint64_t slab = 0, table = 0, slot = 0, graph = 0, scratch = 0; };

bool checked_add(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_add_overflow(a, b, out); }
bool checked_mul(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_mul_overflow(a, b, out); }

}  // namespace

struct fjo_pool {
  uint32_t page_tokens;
  uint64_t total_page_bytes;
  uint32_t pages_per_slab;
  uint64_t byte_limit;
  bool fixed_capacity;
  std::vector<PageState> pages;
  std::vector<uint32_t> free;
  uint64_t completed_serial = 0;
  Memory memory;
  uint64_t next_identity = 1;

  bool memory_total(uint64_t* total) const {
    uint64_t t = memory.slab;
    return checked_add(t, memory.table, &t) && checked_add(t, memory.slot, &t) && checked_add(t, memory.graph, &t) &&
           checked_add(t, memory.scratch, &t) && ((*total = t), true);
  }
  // paged_slab_bytes, paged_pool.rs:1210-1216
  int slab_bytes(uint64_t* out) const {
    uint64_t b;
    if (!checked_add(total_page_bytes, 4, &b) || !checked_mul(b, pages_per_slab, &b)) return FJO_ARITHMETIC_OVERFLOW;
    *out = b;
    return FJO_OK;
  }
  // add_slab, paged_pool.rs:1229-1242
  int add_slab() {
    uint64_t start = pages.size();
    uint64_t end = start + pages_per_slab;
    if (end > 0xFFFFFFFFull) return FJO_ARITHMETIC_OVERFLOW;
    pages.resize(end);
    for (uint64_t p = end; p-- > start;) free.push_back(static_cast<uint32_t>(p));
    return FJO_OK;
  }
  // next_generation, paged_pool.rs:1298-1303
  static int next_generation(uint32_t current, uint32_t* next) {
    if (current == 0xFFFFFFFFu) return FJO_ARITHMETIC_OVERFLOW;
    if (current + 1 == POISON_GENERATION) return FJO_ARITHMETIC_OVERFLOW;
    *next = current + 1;
    return FJO_OK;
  }
  // preflight_pages, paged_pool.rs:1244-1281
  int preflight(uint64_t count, uint64_t extra_bytes) const {
    uint64_t take = std::min<uint64_t>(count, free.size());
    for (uint64_t i = 0; i < take; ++i) {
      uint32_t index = free[free.size() - 1 - i];
      if (index >= pages.size()) return FJO_CORRUPT_STATE;
      uint32_t g;
      int st = next_generation(pages[index].generation, &g);
      if (st) return st;
    }
    uint64_t missing = count > free.size() ? count - free.size() : 0;
    if (missing > 0 && fixed_capacity) return FJO_QUOTA_EXCEEDED;
    uint64_t slabs = (missing + pages_per_slab - 1) / pages_per_slab;
    uint64_t slab, growth, total, projected;
    int st = slab_bytes(&slab);
    if (st) return st;
    if (!checked_mul(slab, slabs, &growth)) return FJO_ARITHMETIC_OVERFLOW;
    if (!memory_total(&total) || !checked_add(total, growth, &projected) || !checked_add(projected, extra_bytes, &projected)) return FJO_ARITHMETIC_OVERFLOW;
    if (projected > byte_limit) return FJO_QUOTA_EXCEEDED;
    return FJO_OK;
  }
  // grow_for, paged_pool.rs:1283-1296
  int grow_for(uint64_t count) {
    while (free.size() < count) {
      int st = add_slab();
      if (st) return st;
      uint64_t slab;
      st = slab_bytes(&slab);
      if (st) return st;
      if (!checked_add(memory.slab, slab, &memory.slab)) return FJO_ARITHMETIC_OVERFLOW;
    }
    return FJO_OK;
  }
  // allocate_pages, paged_pool.rs:1305-1326
  int allocate(uint64_t count, std::vector<PageLease>* out) {
    for (uint64_t i = 0; i < count; ++i) {
      if (free.empty()) return FJO_CORRUPT_STATE;
      uint32_t index = free.back();
      free.pop_back();
      if (index >= pages.size()) return FJO_CORRUPT_STATE;
      PageState& page = pages[index];
      if (page.lifecycle != FREE || page.references != 0) return FJO_CORRUPT_STATE;
      uint32_t g;
      int st = next_generation(page.generation, &g);
      if (st) return st;
      page.generation = g;
      page.references = 1;
      page.lifecycle = ALLOCATED;
      out->push_back({index, g});
    }
    return FJO_OK;
  }
  // live_page_mut, paged_pool.rs:1328-1337
  PageState* live(PageLease lease) {
    if (lease.index >= pages.size()) return nullptr;
    PageState& page = pages[lease.index];
    if (page.lifecycle != ALLOCATED || page.generation != lease.generation) return nullptr;
    return &page;
  }
  // retain, paged_pool.rs:290-306
  int retain(const std::vector<PageLease>& leases) {
    for (auto l : leases) { PageState* p = live(l); if (!p) return FJO_CORRUPT_STATE; if (p->references == 0xFFFFFFFFu) return FJO_ARITHMETIC_OVERFLOW; }
    for (auto l : leases) { PageState* p = live(l); if (!p) return FJO_CORRUPT_STATE; if (p->references == 0xFFFFFFFFu) return FJO_CORRUPT_STATE; p->references += 1; }
    return FJO_OK;
  }
  // release, paged_pool.rs:308-327
  int release(const std::vector<PageLease>& leases) {
    for (auto l : leases) {
      PageState* p = live(l);
      if (!p) return FJO_CORRUPT_STATE;
      if (p->references == 0) return FJO_CORRUPT_STATE;
      p->references -= 1;
      if (p->references == 0) {
        if (p->last_use <= completed_serial) { p->lifecycle = FREE; free.push_back(l.index); }
        else p->lifecycle = RETIRING;
      }
    }
    return FJO_OK;
  }
  int refcount(PageLease lease, uint32_t* out) { PageState* p = live(lease); if (!p) return FJO_CORRUPT_STATE; *out = p->references; return FJO_OK; }
  // allocate_one, paged_pool.rs:329-336
  int allocate_one(PageLease* out) {
    int st = preflight(1, 0);
    if (st) return st;
    st = grow_for(1);
    if (st) return st;
    std::vector<PageLease> v;
    st = allocate(1, &v);
    if (st) return st;
    *out = v[0];
    return FJO_OK;
  }
};

struct fjo_seq {
  fjo_pool* pool;
  std::vector<PageLease> pages;
  std::vector<bool> immutable;
  uint64_t logical_len = 0;
  uint64_t reserved_tokens = 0;
  uint64_t table_bytes = 0;
  uint64_t identity = 0;

  // validate_exclusive, paged_pool.rs:820-843
  int validate_exclusive(uint64_t start, uint64_t end) {
    if (end > reserved_tokens) return FJO_UNRESERVED_WRITE;
    if (end == start) return FJO_OK;
    uint64_t pt = pool->page_tokens;
    uint64_t first = start / pt, last = (end - 1) / pt;
    for (uint64_t page = first; page <= last; ++page) {
      bool imm = page < immutable.size() ? immutable[page] : true;
      if (imm) return FJO_SHARED_TAIL;
      if (page >= pages.size()) return FJO_UNRESERVED_WRITE;
      uint32_t refs;
      int st = pool->refcount(pages[page], &refs);
      if (st) return st;
      if (refs != 1) return FJO_SHARED_TAIL;
    }
    return FJO_OK;
  }
};

struct CheckpointTail { size_t index; PageLease page; bool immutable; bool retained; };
struct fjo_checkpoint {
  fjo_pool* pool;
  uint64_t sequence;
  uint64_t logical_len;
  bool has_tail;
  CheckpointTail tail;
  bool active;
};

struct Slot { std::vector<uint32_t> entries; uint64_t logical_len = 0, append_start = 0; bool active = false; };
struct fjo_banks {
  fjo_pool* pool;
  size_t table_pages;
  std::vector<Slot> banks[2];
  bool has_submitted[2] = {false, false};
  uint64_t submitted[2] = {0, 0};
  uint64_t charged_bytes;

  Slot poisoned() const {
    Slot s;
    s.entries.resize(table_pages * 2);
    for (size_t i = 0; i < table_pages; ++i) { s.entries[2 * i] = 0; s.entries[2 * i + 1] = POISON_GENERATION; }
    return s;
  }
  // ensure_rebindable, paged_pool.rs:715-729
  int ensure_rebindable(size_t bank) {
    if (bank >= 2) return FJO_FOREIGN_RESOURCE;
    if (has_submitted[bank] && submitted[bank] > pool->completed_serial) return FJO_BANK_IN_FLIGHT;
    has_submitted[bank] = false;
    return FJO_OK;
  }
};

static uint64_t pages_for(uint64_t tokens, uint32_t page_tokens, int* st) {
  *st = FJO_OK;
  if (tokens == 0) return 0;
  uint64_t t;
  if (!checked_add(tokens, static_cast<uint64_t>(page_tokens) - 1, &t)) { *st = FJO_ARITHMETIC_OVERFLOW; return 0; }
  return t / page_tokens;
}

extern "C" {

int fjo_pool_new(uint32_t page_tokens, uint64_t total_page_bytes, uint32_t pages_per_slab,
                 uint64_t byte_limit, int fixed, fjo_pool** out) {
  if (pages_per_slab == 0) return FJO_EMPTY_SLAB;
  auto* pool = new fjo_pool();
  pool->page_tokens = page_tokens;
  pool->total_page_bytes = total_page_bytes;
  pool->pages_per_slab = pages_per_slab;
  pool->byte_limit = byte_limit;
  pool->fixed_capacity = fixed != 0;
  uint64_t slab;
  int st = pool->slab_bytes(&slab);
  if (st == FJO_OK && slab > byte_limit) st = FJO_QUOTA_EXCEEDED;
  if (st == FJO_OK) { pool->memory.slab = slab; st = pool->add_slab(); }
  if (st != FJO_OK) { delete pool; return st; }
  *out = pool;
  return FJO_OK;
}
void fjo_pool_free(fjo_pool* pool) { delete pool; }

// observe_completion, paged_pool.rs:176-191
int fjo_pool_observe_completion(fjo_pool* pool, uint64_t serial) {
  pool->completed_serial = std::max(pool->completed_serial, serial);
  std::vector<uint32_t> reclaimed;
  for (size_t i = 0; i < pool->pages.size(); ++i) {
    PageState& page = pool->pages[i];
    if (page.lifecycle == RETIRING && page.last_use <= pool->completed_serial) { page.lifecycle = FREE; reclaimed.push_back(static_cast<uint32_t>(i)); }
  }
  std::sort(reclaimed.begin(), reclaimed.end(), [](uint32_t l, uint32_t r) { return l > r; });
  pool->free.insert(pool->free.end(), reclaimed.begin(), reclaimed.end());
  return FJO_OK;
}

// reserve, paged_pool.rs:204-232
int fjo_pool_reserve(fjo_pool* pool, uint64_t tokens, fjo_seq** out) {
  int st;
  uint64_t page_count = pages_for(tokens, pool->page_tokens, &st);
  if (st) return st;
  uint64_t table_bytes;
  if (!checked_mul(page_count, 8, &table_bytes)) return FJO_ARITHMETIC_OVERFLOW;
  st = pool->preflight(page_count, table_bytes);
  if (st) return st;
  st = pool->grow_for(page_count);
  if (st) return st;
  auto* seq = new fjo_seq();
  st = pool->allocate(page_count, &seq->pages);
  if (st) { delete seq; return st; }
  if (!checked_add(pool->memory.table, table_bytes, &pool->memory.table)) { delete seq; return FJO_ARITHMETIC_OVERFLOW; }
  seq->pool = pool;
  seq->immutable.assign(page_count, false);
  seq->reserved_tokens = tokens;
  seq->table_bytes = table_bytes;
  seq->identity = pool->next_identity++;
  *out = seq;
  return FJO_OK;
}

int fjo_pool_memory(fjo_pool* pool, uint64_t usage[5], uint64_t* limit) {
  usage[0] = pool->memory.slab; usage[1] = pool->memory.table; usage[2] = pool->memory.slot;
  usage[3] = pool->memory.graph; usage[4] = pool->memory.scratch;
  *limit = pool->byte_limit;
  return FJO_OK;
}

// replace_aux_charge, paged_pool.rs:367-387
static int replace_aux(fjo_pool* pool, uint64_t* field, uint64_t bytes) {
  uint64_t total, projected;
  if (!pool->memory_total(&total) || total < *field) return FJO_ARITHMETIC_OVERFLOW;
  if (!checked_add(total - *field, bytes, &projected)) return FJO_ARITHMETIC_OVERFLOW;
  if (projected > pool->byte_limit) return FJO_QUOTA_EXCEEDED;
  *field = bytes;
  return FJO_OK;
}
int fjo_pool_set_graph_arena_bytes(fjo_pool* pool, uint64_t maximum_arena_bytes) {
  uint64_t bytes;
  if (!checked_mul(maximum_arena_bytes, 2, &bytes)) return FJO_ARITHMETIC_OVERFLOW;
  return replace_aux(pool, &pool->memory.graph, bytes);
}
int fjo_pool_set_scratch_bytes(fjo_pool* pool, uint64_t primary, uint64_t overlap) {
  uint64_t bytes;
  if (!checked_add(primary, overlap, &bytes)) return FJO_ARITHMETIC_OVERFLOW;
  return replace_aux(pool, &pool->memory.scratch, bytes);
}
size_t fjo_pool_physical_pages(fjo_pool* pool) { return pool->pages.size(); }
int fjo_pool_generations(fjo_pool* pool, uint32_t* out, size_t n) {
  if (n < pool->pages.size()) return FJO_INVALID_INPUT;
  for (size_t i = 0; i < pool->pages.size(); ++i) out[i] = pool->pages[i].generation;
  return FJO_OK;
}
size_t fjo_pool_free_list(fjo_pool* pool, uint32_t* out, size_t cap) {
  for (size_t i = 0; i < pool->free.size() && i < cap; ++i) out[i] = pool->free[i];
  return pool->free.size();
}
int fjo_pool_debug_set_generation(fjo_pool* pool, uint32_t page, uint32_t generation) {
  if (page >= pool->pages.size()) return FJO_INVALID_INPUT;
  pool->pages[page].generation = generation;
  return FJO_OK;
}

// Drop for PagedSequence, paged_pool.rs:1126-1133
void fjo_seq_drop(fjo_seq* seq) {
  if (!seq) return;
  seq->pool->release(seq->pages);
  seq->pool->memory.table = seq->pool->memory.table >= seq->table_bytes ? seq->pool->memory.table - seq->table_bytes : 0;
  delete seq;
}
uint64_t fjo_seq_logical_len(fjo_seq* seq) { return seq->logical_len; }
uint64_t fjo_seq_reserved_tokens(fjo_seq* seq) { return seq->reserved_tokens; }
size_t fjo_seq_pages(fjo_seq* seq) { return seq->pages.size(); }
int fjo_seq_table(fjo_seq* seq, uint32_t* entries, size_t cap_pages) {
  if (cap_pages < seq->pages.size()) return FJO_INVALID_INPUT;
  for (size_t i = 0; i < seq->pages.size(); ++i) {
    // PageTable::new validates each entry against current generations (paged_pool.rs:904-913)
    if (!seq->pool->live(seq->pages[i])) return FJO_CORRUPT_STATE;
    entries[2 * i] = seq->pages[i].index;
    entries[2 * i + 1] = seq->pages[i].generation;
  }
  return FJO_OK;
}
int fjo_seq_refcounts(fjo_seq* seq, uint32_t* out, size_t cap_pages) {
  if (cap_pages < seq->pages.size()) return FJO_INVALID_INPUT;
  for (size_t i = 0; i < seq->pages.size(); ++i) { int st = seq->pool->refcount(seq->pages[i], &out[i]); if (st) return st; }
  return FJO_OK;
}
// validate_write, paged_pool.rs:790-798
int fjo_seq_validate_write(fjo_seq* seq, uint64_t start, uint64_t tokens) {
  uint64_t end;
  if (!checked_add(start, tokens, &end)) return FJO_ARITHMETIC_OVERFLOW;
  if (start != seq->logical_len) return FJO_UNRESERVED_WRITE;
  return seq->validate_exclusive(start, end);
}
// validate_append, paged_pool.rs:805-818
int fjo_seq_validate_append(fjo_seq* seq, uint64_t win_start, uint64_t win_end, uint64_t start, uint64_t tokens) {
  uint64_t end;
  if (!checked_add(start, tokens, &end)) return FJO_ARITHMETIC_OVERFLOW;
  if (start < win_start || end > win_end) return FJO_UNRESERVED_WRITE;
  return seq->validate_exclusive(start, end);
}
// commit_write, paged_pool.rs:850-857
int fjo_seq_commit_write(fjo_seq* seq, uint64_t tokens) {
  int st = fjo_seq_validate_write(seq, seq->logical_len, tokens);
  if (st) return st;
  seq->logical_len += tokens;
  return FJO_OK;
}
// rewind_private, paged_pool.rs:864-883
int fjo_seq_rewind_private(fjo_seq* seq, uint64_t logical_len) {
  if (logical_len >= seq->logical_len) return FJO_INVALID_CHECKPOINT;
  uint64_t pt = seq->pool->page_tokens;
  uint64_t first = logical_len / pt, last = (seq->logical_len + pt - 1) / pt;
  for (uint64_t page = first; page < last; ++page) {
    uint32_t refs;
    int st = seq->pool->refcount(seq->pages[page], &refs);
    if (seq->immutable[page]) return FJO_SHARED_TAIL;
    if (st) return st;
    if (refs != 1) return FJO_SHARED_TAIL;
  }
  seq->logical_len = logical_len;
  return FJO_OK;
}
// mark_submitted, paged_pool.rs:890-897
int fjo_seq_mark_submitted(fjo_seq* seq, uint64_t serial) {
  for (auto lease : seq->pages) {
    PageState* page = seq->pool->live(lease);
    if (!page) return FJO_CORRUPT_STATE;
    page->last_use = std::max(page->last_use, serial);
  }
  return FJO_OK;
}
// fork_reserved, paged_pool.rs:949-1018
int fjo_seq_fork_reserved(fjo_seq* seq, uint64_t prefix_tokens, uint64_t reserved_tokens, fjo_seq** out) {
  if (prefix_tokens > seq->logical_len) return FJO_UNRESERVED_WRITE;
  if (reserved_tokens < prefix_tokens) return FJO_UNRESERVED_WRITE;
  fjo_pool* pool = seq->pool;
  int st;
  uint64_t shared_pages = pages_for(prefix_tokens, pool->page_tokens, &st);
  if (st) return st;
  uint64_t reserved_pages = pages_for(reserved_tokens, pool->page_tokens, &st);
  if (st) return st;
  uint64_t private_pages = reserved_pages - shared_pages;
  if (shared_pages > seq->pages.size()) return FJO_CORRUPT_STATE;
  std::vector<PageLease> pages(seq->pages.begin(), seq->pages.begin() + shared_pages);
  uint64_t table_bytes;
  if (!checked_mul(reserved_pages, 8, &table_bytes)) return FJO_ARITHMETIC_OVERFLOW;
  st = pool->preflight(private_pages, table_bytes);
  if (st) return st;
  st = pool->retain(pages);
  if (st) return st;
  std::vector<PageLease> priv;
  uint64_t new_table_bytes = 0;
  st = pool->preflight(private_pages, table_bytes);
  if (st == FJO_OK && !checked_add(pool->memory.table, table_bytes, &new_table_bytes)) st = FJO_ARITHMETIC_OVERFLOW;
  if (st == FJO_OK) st = pool->grow_for(private_pages);
  if (st == FJO_OK) st = pool->allocate(private_pages, &priv);
  if (st != FJO_OK) { pool->release(pages); return st; }
  pool->memory.table = new_table_bytes;
  pages.insert(pages.end(), priv.begin(), priv.end());
  for (uint64_t i = 0; i < shared_pages; ++i) seq->immutable[i] = true;
  auto* fork = new fjo_seq();
  fork->pool = pool;
  fork->pages = pages;
  fork->immutable.assign(reserved_pages, false);
  for (uint64_t i = 0; i < shared_pages; ++i) fork->immutable[i] = true;
  fork->logical_len = prefix_tokens;
  fork->reserved_tokens = reserved_tokens;
  fork->table_bytes = table_bytes;
  fork->identity = pool->next_identity++;
  *out = fork;
  return FJO_OK;
}
// cow_tail, paged_pool.rs:1025-1054
int fjo_seq_cow_tail(fjo_seq* seq, int* copied, uint32_t* src, uint32_t* dst, uint32_t* token_count) {
  *copied = 0;
  if (seq->logical_len == 0) return FJO_OK;
  uint64_t pt = seq->pool->page_tokens;
  if (seq->logical_len % pt == 0) return FJO_OK;
  uint64_t tail = (seq->logical_len - 1) / pt;
  if (tail >= seq->pages.size()) return FJO_CORRUPT_STATE;
  PageLease old = seq->pages[tail];
  uint32_t refs;
  bool imm = tail < seq->immutable.size() ? seq->immutable[tail] : true;
  if (!imm) {
    int st = seq->pool->refcount(old, &refs);
    if (st) return st;
    if (refs == 1) return FJO_OK;
  }
  PageLease fresh;
  int st = seq->pool->allocate_one(&fresh);
  if (st) return st;
  seq->pages[tail] = fresh;
  seq->immutable[tail] = false;
  st = seq->pool->release({old});
  if (st) {
    seq->pages[tail] = old;
    seq->immutable[tail] = true;
    int st2 = seq->pool->release({fresh});
    return st2 ? st2 : st;
  }
  *copied = 1;
  *src = old.index;
  *dst = fresh.index;
  *token_count = static_cast<uint32_t>(seq->logical_len % pt);
  return FJO_OK;
}
// checkpoint, paged_pool.rs:1061-1089
int fjo_seq_checkpoint(fjo_seq* seq, fjo_checkpoint** out) {
  auto* cp = new fjo_checkpoint();
  cp->pool = seq->pool;
  cp->sequence = seq->identity;
  cp->logical_len = seq->logical_len;
  cp->has_tail = false;
  cp->active = true;
  if (seq->logical_len != 0) {
    size_t tail = static_cast<size_t>((seq->logical_len - 1) / seq->pool->page_tokens);
    if (tail >= seq->pages.size()) { delete cp; return FJO_CORRUPT_STATE; }
    PageLease page = seq->pages[tail];
    bool imm = tail < seq->immutable.size() ? seq->immutable[tail] : true;
    bool retained = imm;
    if (!retained) {
      uint32_t refs;
      int st = seq->pool->refcount(page, &refs);
      if (st) { delete cp; return st; }
      retained = refs > 1;
    }
    if (retained) { int st = seq->pool->retain({page}); if (st) { delete cp; return st; } }
    cp->has_tail = true;
    cp->tail = {tail, page, imm, retained};
  }
  *out = cp;
  return FJO_OK;
}
int fjo_checkpoint_belongs_to(fjo_checkpoint* cp, fjo_seq* seq) {
  return cp->active && cp->pool == seq->pool && cp->sequence == seq->identity;
}
// Drop for SequenceCheckpoint, paged_pool.rs:1167-1175
void fjo_checkpoint_drop(fjo_checkpoint* cp) {
  if (!cp) return;
  if (cp->has_tail && cp->tail.retained) cp->pool->release({cp->tail.page});
  delete cp;
}
// rollback, paged_pool.rs:1096-1123
int fjo_seq_rollback(fjo_seq* seq, fjo_checkpoint* cp) {
  if (!fjo_checkpoint_belongs_to(cp, seq)) { fjo_checkpoint_drop(cp); return FJO_INVALID_CHECKPOINT; }
  if (cp->has_tail) {
    CheckpointTail& tail = cp->tail;
    if (tail.index >= seq->pages.size()) { fjo_checkpoint_drop(cp); return FJO_CORRUPT_STATE; }
    PageLease& current = seq->pages[tail.index];
    if (current == tail.page) {
      // The reference leaves `retained` set here, so the checkpoint's Drop (below) releases the
      // page a second time (paged_pool.rs:1109-1113 with :1167-1175); restated as written.
      if (tail.retained) { int st = seq->pool->release({tail.page}); if (st) { fjo_checkpoint_drop(cp); return st; } }
    } else {
      int st = seq->pool->release({current});
      if (st) { fjo_checkpoint_drop(cp); return st; }
      current = tail.page;
      tail.retained = false;
    }
    seq->immutable[tail.index] = tail.immutable;
  }
  seq->logical_len = cp->logical_len;
  cp->active = false;
  fjo_checkpoint_drop(cp);
  return FJO_OK;
}

// PagedSlotBanks::new, paged_pool.rs:446-478
int fjo_banks_new(fjo_pool* pool, size_t lanes, size_t table_pages, fjo_banks** out) {
  if (lanes == 0 || table_pages == 0) return FJO_UNRESERVED_WRITE;
  uint64_t meta, one, charged;
  if (!checked_mul(lanes, 16, &meta) || !checked_mul(lanes, table_pages, &one) || !checked_mul(one, 8, &one) ||
      !checked_add(one, meta, &one) || !checked_mul(one, 2, &charged))
    return FJO_ARITHMETIC_OVERFLOW;
  uint64_t total, projected;  // charge_slots, paged_pool.rs:343-359
  if (!pool->memory_total(&total) || !checked_add(total, charged, &projected)) return FJO_ARITHMETIC_OVERFLOW;
  if (projected > pool->byte_limit) return FJO_QUOTA_EXCEEDED;
  pool->memory.slot += charged;
  auto* banks = new fjo_banks();
  banks->pool = pool;
  banks->table_pages = table_pages;
  banks->charged_bytes = charged;
  for (int b = 0; b < 2; ++b) banks->banks[b].assign(lanes, banks->poisoned());
  *out = banks;
  return FJO_OK;
}
void fjo_banks_free(fjo_banks* banks) {
  if (!banks) return;
  banks->pool->memory.slot = banks->pool->memory.slot >= banks->charged_bytes ? banks->pool->memory.slot - banks->charged_bytes : 0;
  delete banks;
}
static int padded_table(fjo_banks* banks, fjo_seq* seq, std::vector<uint32_t>* entries) {
  if (seq->pages.size() > banks->table_pages) return FJO_UNRESERVED_WRITE;  // pad_with_poison refuses
  entries->assign(banks->table_pages * 2, 0);
  for (size_t i = 0; i < banks->table_pages; ++i) (*entries)[2 * i + 1] = POISON_GENERATION;
  return fjo_seq_table(seq, entries->data(), banks->table_pages);
}
// bind, paged_pool.rs:516-543
int fjo_banks_bind(fjo_banks* banks, size_t bank, size_t lane, fjo_seq* seq) {
  if (seq->pool != banks->pool) return FJO_FOREIGN_RESOURCE;
  int st = banks->ensure_rebindable(bank);
  if (st) return st;
  std::vector<uint32_t> entries;
  st = padded_table(banks, seq, &entries);
  if (st) return st;
  if (lane >= banks->banks[bank].size()) return FJO_FOREIGN_RESOURCE;
  Slot& slot = banks->banks[bank][lane];
  slot.entries = entries;
  slot.logical_len = seq->logical_len;
  slot.append_start = seq->logical_len;
  slot.active = true;
  return FJO_OK;
}
// bind_all, paged_pool.rs:551-591
int fjo_banks_bind_all(fjo_banks* banks, size_t lane, fjo_seq* seq) {
  if (seq->pool != banks->pool) return FJO_FOREIGN_RESOURCE;
  std::vector<uint32_t> entries;
  int st = padded_table(banks, seq, &entries);
  if (st) return st;
  for (size_t bank = 0; bank < 2; ++bank) {
    if (lane >= banks->banks[bank].size()) return FJO_FOREIGN_RESOURCE;
    if (banks->has_submitted[bank] && banks->submitted[bank] > banks->pool->completed_serial) return FJO_BANK_IN_FLIGHT;
  }
  for (size_t bank = 0; bank < 2; ++bank) {
    Slot& slot = banks->banks[bank][lane];
    slot.entries = entries;
    slot.logical_len = seq->logical_len;
    slot.append_start = seq->logical_len;
    slot.active = true;
  }
  return FJO_OK;
}
// poison, paged_pool.rs:616-631
int fjo_banks_poison(fjo_banks* banks, size_t bank, size_t lane) {
  int st = banks->ensure_rebindable(bank);
  if (st) return st;
  if (lane >= banks->banks[bank].size()) return FJO_FOREIGN_RESOURCE;
  banks->banks[bank][lane] = banks->poisoned();
  return FJO_OK;
}
// open_append, paged_pool.rs:655-678
int fjo_banks_open_append(fjo_banks* banks, size_t bank, size_t lane, uint64_t start, uint64_t logical_len) {
  if (start > logical_len) return FJO_UNRESERVED_WRITE;
  if (bank >= 2 || lane >= banks->banks[bank].size()) return FJO_FOREIGN_RESOURCE;
  Slot& slot = banks->banks[bank][lane];
  if (!slot.active) return FJO_FOREIGN_RESOURCE;
  slot.logical_len = logical_len;
  slot.append_start = start;
  return FJO_OK;
}
int fjo_banks_mark_submitted(fjo_banks* banks, size_t bank, uint64_t serial) {
  if (bank >= 2) return FJO_FOREIGN_RESOURCE;
  banks->has_submitted[bank] = true;
  banks->submitted[bank] = serial;
  return FJO_OK;
}
int fjo_banks_slot(fjo_banks* banks, size_t bank, size_t lane, uint32_t* entries, uint64_t info[3]) {
  if (bank >= 2 || lane >= banks->banks[bank].size()) return FJO_FOREIGN_RESOURCE;
  const Slot& slot = banks->banks[bank][lane];
  for (size_t i = 0; i < slot.entries.size(); ++i) entries[i] = slot.entries[i];
  info[0] = slot.logical_len; info[1] = slot.append_start; info[2] = slot.active ? 1 : 0;
  return FJO_OK;
}

}  // extern "C"
