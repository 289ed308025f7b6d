// CPU oracle: paged storage (copy, attention, append), restating crates/forja-cpu/src/paged.rs
// and crates/forja-cpu/src/lib.rs:189-380, 1519-1535 with the page-table rules of
// crates/forja-core/src/paged.rs:68-194. Test infrastructure only; see fjo.h.
#include "fjo.h"
#include "fjo_convert.h"

#include <cmath>
#include <cstring>
#include <vector>

namespace fjo {
bool decode(const void* src, int dt, float* dst, size_t n);
bool encode(const float* src, void* dst, int dt, size_t n);
size_t dtype_size(int dt);
extern int g_threads;

namespace {
const uint32_t POISON_GENERATION = 0xFFFFFFFFu;

struct Table {
  const uint32_t* entries; size_t pages; const uint32_t* generations; size_t physical;
  // validate_entry, paged.rs:186-194
  int validate(uint32_t page, uint32_t generation) const {
    if (page >= physical) return 2;
    if (generations[page] != generation) return 3;
    return 0;
  }
  // PageTable::from_padded, paged.rs:97-117: poisoned entries are skipped, others must authenticate
  bool from_padded_ok() const {
    for (size_t i = 0; i < pages; ++i) {
      uint32_t page = entries[2 * i], gen = entries[2 * i + 1];
      if (page != 0 || gen != POISON_GENERATION) if (validate(page, gen) != 0) return false;
    }
    return true;
  }
  // PageTable::resolve, paged.rs:152-163
  int resolve(uint64_t logical, uint32_t* physical_page) const {
    if (logical >= pages) return 1;
    int st = validate(entries[2 * logical], entries[2 * logical + 1]);
    if (st) return st;
    *physical_page = entries[2 * logical];
    return 0;
  }
};

// CpuPagePool::token_range, paged.rs:283-315 (alignment == dtype size: page bytes are unpadded)
bool token_offset(const Table& table, uint64_t logical_token, uint32_t page_tokens, size_t row_bytes, size_t* offset) {
  uint32_t physical;
  if (table.resolve(logical_token / page_tokens, &physical) != 0) return false;
  if (physical >= table.physical) return false;
  *offset = static_cast<size_t>(physical) * page_tokens * row_bytes + static_cast<size_t>(logical_token % page_tokens) * row_bytes;
  return true;
}

inline float load(const char* plane, int dt, size_t byte_offset) {
  switch (dt) {
    case FJO_F32: { float v; std::memcpy(&v, plane + byte_offset, 4); return v; }
    case FJO_F16: { uint16_t h; std::memcpy(&h, plane + byte_offset, 2); return f16_to_f32(h); }
    default: { uint16_t h; std::memcpy(&h, plane + byte_offset, 2); return bf16_to_f32(h); }
  }
}

// softmax, paged.rs:378-388 (no -inf guard; sum accumulated while exponentiating)
void softmax_paged(std::vector<float>& values) {
  float maximum = -INFINITY;
  for (float v : values) maximum = std::fmax(maximum, v);
  float sum = 0.0f;
  for (float& v : values) { v = std::exp(v - maximum); sum += v; }
  for (float& v : values) v /= sum;
}

bool lane_active(const uint32_t* activity) { return activity == nullptr || *activity != 0; }

int paged_copy(int into_pages, void* ordinary, int o_dt, void* pool, int p_dt, const Table& table,
               uint32_t start, uint32_t tokens, uint32_t page_tokens, size_t elements) {
  if (!table.from_padded_ok()) return FJO_EXECUTION_FAILED;  // cpu_page_table, lib.rs:1519-1535
  const size_t row_bytes = elements * dtype_size(p_dt);
  std::vector<float> row(elements);
  if (into_pages) {
    // decode ordinary -> encode to pool dtype -> copy_in row by row (lib.rs:220-231, paged.rs:77-116)
    std::vector<char> staged(static_cast<size_t>(tokens) * row_bytes);
    for (uint32_t t = 0; t < tokens; ++t) {
      if (!decode(static_cast<const char*>(ordinary) + static_cast<size_t>(t) * elements * dtype_size(o_dt), o_dt, row.data(), elements)) return FJO_EXECUTION_FAILED;
      if (!encode(row.data(), staged.data() + static_cast<size_t>(t) * row_bytes, p_dt, elements)) return FJO_EXECUTION_FAILED;
    }
    // the reference resolves every destination before it writes the pool back; an invalid
    // entry fails the whole op with the pool unchanged (it works on a copy, lib.rs:217-242)
    std::vector<size_t> offsets(tokens);
    for (uint32_t t = 0; t < tokens; ++t)
      if (!token_offset(table, static_cast<uint64_t>(start) + t, page_tokens, row_bytes, &offsets[t])) return FJO_INVALID_INPUT;
    for (uint32_t t = 0; t < tokens; ++t)
      std::memcpy(static_cast<char*>(pool) + offsets[t], staged.data() + static_cast<size_t>(t) * row_bytes, row_bytes);
    return FJO_OK;
  }
  std::vector<size_t> offsets(tokens);
  for (uint32_t t = 0; t < tokens; ++t)
    if (!token_offset(table, static_cast<uint64_t>(start) + t, page_tokens, row_bytes, &offsets[t])) return FJO_INVALID_INPUT;
  for (uint32_t t = 0; t < tokens; ++t) {
    if (!decode(static_cast<const char*>(pool) + offsets[t], p_dt, row.data(), elements)) return FJO_EXECUTION_FAILED;
    if (!encode(row.data(), static_cast<char*>(ordinary) + static_cast<size_t>(t) * elements * dtype_size(o_dt), o_dt, elements)) return FJO_EXECUTION_FAILED;
  }
  return FJO_OK;
}

// CpuPagePool::sdpa, paged.rs:161-259
int paged_sdpa(const void* q, int q_dt, const void* kpool, int k_dt, const void* vpool, int v_dt,
               const Table& table, void* out, int out_dt, uint32_t q_heads, uint32_t q_len,
               uint32_t kv_heads, uint32_t width, uint32_t value_width, uint32_t key_length,
               uint32_t q_start, float scale, bool causal, uint32_t page_tokens) {
  if (q_heads == 0 || kv_heads == 0 || q_heads % kv_heads != 0 || !std::isfinite(scale)) return FJO_INVALID_INPUT;
  if (!table.from_padded_ok()) return FJO_EXECUTION_FAILED;
  const size_t qn = static_cast<size_t>(q_heads) * q_len * width;
  std::vector<float> query(qn);
  if (!decode(q, q_dt, query.data(), qn)) return FJO_EXECUTION_FAILED;
  const size_t k_row_bytes = static_cast<size_t>(kv_heads) * width * dtype_size(k_dt);
  const size_t v_row_bytes = static_cast<size_t>(kv_heads) * value_width * dtype_size(v_dt);
  const uint32_t per_group = q_heads / kv_heads;
  std::vector<float> output(static_cast<size_t>(q_heads) * q_len * value_width);
  // token offsets are shared by every head: resolve once per key row
  uint32_t max_attended = causal ? std::min<uint64_t>(key_length, static_cast<uint64_t>(q_start) + q_len) : key_length;
  std::vector<size_t> k_off(max_attended), v_off(max_attended);
  for (uint32_t t = 0; t < max_attended; ++t) {
    if (!token_offset(table, t, page_tokens, k_row_bytes, &k_off[t])) return FJO_INVALID_INPUT;
    if (!token_offset(table, t, page_tokens, v_row_bytes, &v_off[t])) return FJO_INVALID_INPUT;
  }
  const char* kp = static_cast<const char*>(kpool);
  const char* vp = static_cast<const char*>(vpool);
  const size_t ksz = dtype_size(k_dt), vsz = dtype_size(v_dt);
  int failed = 0;
#pragma omp parallel for collapse(2) if (g_threads > 1)
  for (uint32_t head = 0; head < q_heads; ++head) {
    for (uint32_t query_row = 0; query_row < q_len; ++query_row) {
      uint32_t kv_head = head / per_group;
      const float* qr = &query[(static_cast<size_t>(head) * q_len + query_row) * width];
      uint64_t limit = static_cast<uint64_t>(q_start) + query_row + 1;
      if (causal && limit > 0xFFFFFFFFull) { failed = 1; continue; }
      uint32_t attended = causal ? static_cast<uint32_t>(std::min<uint64_t>(key_length, limit)) : key_length;
      std::vector<float> scores(attended);
      for (uint32_t key_row = 0; key_row < attended; ++key_row) {
        float score = 0.0f;
        for (uint32_t column = 0; column < width; ++column)
          score += qr[column] * load(kp, k_dt, k_off[key_row] + (static_cast<size_t>(kv_head) * width + column) * ksz);
        scores[key_row] = score * scale;
      }
      softmax_paged(scores);
      float* orow = &output[(static_cast<size_t>(head) * q_len + query_row) * value_width];
      for (uint32_t column = 0; column < value_width; ++column) {
        float sum = 0.0f;
        for (uint32_t key_row = 0; key_row < attended; ++key_row)
          sum += scores[key_row] * load(vp, v_dt, v_off[key_row] + (static_cast<size_t>(kv_head) * value_width + column) * vsz);
        orow[column] = sum;
      }
    }
  }
  if (failed) return FJO_INVALID_INPUT;
  return encode(output.data(), out, out_dt, output.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

}  // namespace
}  // namespace fjo

using namespace fjo;

extern "C" {

int fjo_paged_copy(int into_pages, void* ordinary, int o_dt, void* pool, int p_dt,
                   const uint32_t* table, size_t table_pages, const uint32_t* generations,
                   size_t physical_pages, uint32_t start, uint32_t tokens, uint32_t page_tokens,
                   size_t elements, const uint32_t* activity) {
  if (!lane_active(activity)) return FJO_OK;  // lib.rs:197-199
  if (physical_pages == 0 || page_tokens == 0) return FJO_INVALID_INPUT;
  Table t{table, table_pages, generations, physical_pages};
  return paged_copy(into_pages, ordinary, o_dt, pool, p_dt, t, start, tokens, page_tokens, elements);
}

int fjo_paged_sdpa(const void* q, int q_dt, const void* kpool, int k_dt, const void* vpool, int v_dt,
                   const uint32_t* table, size_t table_pages, const uint32_t* generations,
                   size_t physical_pages, void* out, int out_dt, uint32_t q_heads, uint32_t q_len,
                   uint32_t kv_heads, uint32_t width, uint32_t value_width, uint32_t key_length,
                   uint32_t q_start, float scale, int causal, uint32_t page_tokens,
                   const uint32_t* activity) {
  if (!lane_active(activity)) {  // lib.rs:319-328: inactive lane writes zeros, reads nothing
    std::vector<float> zeros(static_cast<size_t>(q_heads) * q_len * value_width, 0.0f);
    return encode(zeros.data(), out, out_dt, zeros.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
  }
  if (physical_pages == 0 || page_tokens == 0) return FJO_INVALID_INPUT;
  Table t{table, table_pages, generations, physical_pages};
  return paged_sdpa(q, q_dt, kpool, k_dt, vpool, v_dt, t, out, out_dt, q_heads, q_len, kv_heads, width,
                    value_width, key_length, q_start, scale, causal != 0, page_tokens);
}

int fjo_paged_sdpa_append(const void* q, int q_dt, const void* k_new, int kn_dt, const void* v_new,
                          int vn_dt, void* kpool, int k_dt, void* vpool, int v_dt,
                          const uint32_t* table, size_t table_pages, const uint32_t* generations,
                          size_t physical_pages, void* out, int out_dt, uint32_t q_heads,
                          uint32_t kv_heads, uint32_t width, uint32_t value_width, uint32_t q_start,
                          float scale, uint32_t page_tokens, const uint32_t* activity) {
  if (q_start == 0xFFFFFFFFu) return FJO_INVALID_INPUT;  // q_start + 1 must not overflow (lib.rs:303)
  // two IntoPages copies of one row each, then causal attention with key_length = q_start + 1
  int st = fjo_paged_copy(1, const_cast<void*>(k_new), kn_dt, kpool, k_dt, table, table_pages, generations,
                          physical_pages, q_start, 1, page_tokens, static_cast<size_t>(kv_heads) * width, activity);
  if (st != FJO_OK) return st;
  st = fjo_paged_copy(1, const_cast<void*>(v_new), vn_dt, vpool, v_dt, table, table_pages, generations,
                      physical_pages, q_start, 1, page_tokens, static_cast<size_t>(kv_heads) * value_width, activity);
  if (st != FJO_OK) return st;
  return fjo_paged_sdpa(q, q_dt, kpool, k_dt, vpool, v_dt, table, table_pages, generations, physical_pages,
                        out, out_dt, q_heads, 1, kv_heads, width, value_width, q_start + 1, q_start, scale, 1,
                        page_tokens, activity);
}

int fjo_paged_layout_page_bytes(uint32_t page_tokens, int dtype, uint64_t elements_per_token,
                                uint64_t alignment, uint64_t* page_bytes) {
  uint64_t size = dtype_size(dtype);
  if (page_tokens == 0 || page_tokens > 4096) return FJO_INVALID_INPUT;
  if (elements_per_token == 0 || size == 0) return FJO_INVALID_INPUT;
  if (alignment == 0 || (alignment & (alignment - 1)) != 0 || alignment < size || alignment % size != 0) return FJO_INVALID_INPUT;
  unsigned __int128 bytes = static_cast<unsigned __int128>(page_tokens) * elements_per_token * size;
  if (bytes > 0xFFFFFFFFFFFFFFFFull - (alignment - 1)) return FJO_ARITHMETIC_OVERFLOW;
  *page_bytes = (static_cast<uint64_t>(bytes) + alignment - 1) & ~(alignment - 1);
  return FJO_OK;
}

int fjo_page_table_resolve(const uint32_t* table, size_t table_pages, const uint32_t* generations,
                           size_t physical_pages, uint32_t logical_page, uint32_t* physical) {
  Table t{table, table_pages, generations, physical_pages};
  return t.resolve(logical_page, physical);
}

}  // extern "C"
