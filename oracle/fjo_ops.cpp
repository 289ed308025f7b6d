// CPU oracle: restatement of the trusted operators of the reference CPU backend
// (crates/forja-cpu/src/lib.rs). Test infrastructure only; see fjo.h.
#include "fjo.h"
#include "fjo_convert.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace fjo {

int g_threads = 1;

size_t dtype_size(int dt) {
  switch (dt) {
    case FJO_F32: case FJO_I32: case FJO_U32: return 4;
    case FJO_F16: case FJO_BF16: return 2;
    default: return 0;
  }
}

// decode, lib.rs:1790-1809
bool decode(const void* src, int dt, float* dst, size_t n) {
  switch (dt) {
    case FJO_F32: std::memcpy(dst, src, n * 4); return true;
    case FJO_F16: { auto p = static_cast<const uint16_t*>(src); for (size_t i = 0; i < n; ++i) dst[i] = f16_to_f32(p[i]); return true; }
    case FJO_BF16: { auto p = static_cast<const uint16_t*>(src); for (size_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(p[i]); return true; }
    default: return false;
  }
}
std::vector<float> decode_vec(const void* src, int dt, size_t n, bool* ok) {
  std::vector<float> v(n);
  *ok = decode(src, dt, v.data(), n);
  return v;
}
// encode, lib.rs:1836-1847
bool encode(const float* src, void* dst, int dt, size_t n) {
  switch (dt) {
    case FJO_F32: std::memcpy(dst, src, n * 4); return true;
    case FJO_F16: { auto p = static_cast<uint16_t*>(dst); for (size_t i = 0; i < n; ++i) p[i] = f32_to_f16(src[i]); return true; }
    case FJO_BF16: { auto p = static_cast<uint16_t*>(dst); for (size_t i = 0; i < n; ++i) p[i] = f32_to_bf16(src[i]); return true; }
    default: return false;
  }
}

// f32::total_cmp
static inline int32_t total_key(float v) {
  int32_t b = static_cast<int32_t>(f32_bits(v));
  b ^= static_cast<int32_t>(static_cast<uint32_t>(b >> 31) >> 1);
  return b;
}
static inline int total_cmp(float a, float b) {
  int32_t x = total_key(a), y = total_key(b);
  return x < y ? -1 : (x > y ? 1 : 0);
}

static inline void record_invalid(bool* have, uint32_t* lowest, uint32_t index) {
  if (!*have || index < *lowest) *lowest = index;
  *have = true;
}

// affine_quant_dot, lib.rs:1277-1310
static inline float affine_quant_dot(const float* activation, size_t inner, const uint32_t* packed,
                                     const float* scales, const float* biases, size_t packed_row,
                                     size_t group_row, size_t group_size, uint32_t bits) {
  const size_t values_per_word = 32 / bits;
  const uint32_t mask = (1u << bits) - 1;
  float sum = 0.0f;
  for (size_t index = 0; index < inner; ++index) {
    uint32_t word = packed[packed_row + index / values_per_word];
    uint32_t shift = static_cast<uint32_t>((index % values_per_word) * bits);
    uint32_t quantized = (word >> shift) & mask;
    size_t group = group_row + index / group_size;
    sum = sum + activation[index] * (scales[group] * static_cast<float>(quantized) + biases[group]);
  }
  return sum;
}

// softmax, lib.rs:1821-1834 (contiguous-cache SDPA)
void softmax_lib(std::vector<float>& values) {
  float maximum = -INFINITY;
  for (float v : values) maximum = std::fmax(maximum, v);
  if (maximum == -INFINITY) { std::fill(values.begin(), values.end(), 0.0f); return; }
  for (float& v : values) v = std::exp(v - maximum);
  float sum = 0.0f;
  for (float v : values) sum += v;
  for (float& v : values) v /= sum;
}

}  // namespace fjo

using namespace fjo;

extern "C" {

size_t fjo_dtype_size(int dtype) { return dtype_size(dtype); }
void fjo_set_threads(int threads) {
  g_threads = threads < 1 ? 1 : threads;
#ifdef _OPENMP
  omp_set_num_threads(g_threads);
#endif
}
int fjo_get_max_threads(void) {
#ifdef _OPENMP
  return omp_get_num_procs();
#else
  return 1;
#endif
}

int fjo_decode(const void* src, int dtype, float* dst, size_t n) { return decode(src, dtype, dst, n) ? FJO_OK : FJO_EXECUTION_FAILED; }
int fjo_encode(const float* src, void* dst, int dtype, size_t n) { return encode(src, dst, dtype, n) ? FJO_OK : FJO_EXECUTION_FAILED; }

int fjo_copy(const void* in, int in_dt, void* out, int out_dt, size_t n) {
  if (in_dt == FJO_I32 || in_dt == FJO_U32) {  // lib.rs:172-183: raw byte copy
    if (dtype_size(out_dt) != 4) return FJO_INVALID_INPUT;
    std::memcpy(out, in, n * 4);
    return FJO_OK;
  }
  bool ok;
  auto values = decode_vec(in, in_dt, n, &ok);
  if (!ok || !encode(values.data(), out, out_dt, n)) return FJO_EXECUTION_FAILED;
  return FJO_OK;
}

int fjo_rms_norm(const void* x, int x_dt, const void* w, int w_dt, void* out, int out_dt,
                 size_t rows, size_t width, float eps) {
  bool ok1, ok2;
  auto values = decode_vec(x, x_dt, rows * width, &ok1);
  auto weights = decode_vec(w, w_dt, width, &ok2);
  if (!ok1 || !ok2) return FJO_EXECUTION_FAILED;
  std::vector<float> normalized(rows * width);
#pragma omp parallel for if (g_threads > 1)
  for (size_t r = 0; r < rows; ++r) {
    const float* row = &values[r * width];
    float sum = 0.0f, count = 0.0f;
    for (size_t i = 0; i < width; ++i) sum = sum + row[i] * row[i];
    for (size_t i = 0; i < width; ++i) count = count + 1.0f;
    float scale = 1.0f / std::sqrt(sum / count + eps);
    for (size_t i = 0; i < width; ++i) normalized[r * width + i] = row[i] * scale * weights[i];
  }
  return encode(normalized.data(), out, out_dt, rows * width) ? FJO_OK : FJO_EXECUTION_FAILED;
}

int fjo_argmax(const void* x, int x_dt, uint32_t* out, size_t rows, size_t width) {
  if (width == 0) return FJO_EXECUTION_FAILED;
  bool ok;
  auto values = decode_vec(x, x_dt, rows * width, &ok);
  if (!ok) return FJO_EXECUTION_FAILED;
  for (size_t r = 0; r < rows; ++r) {
    const float* row = &values[r * width];
    size_t best = 0;  // Iterator::max_by keeps the last of equal maxima
    for (size_t i = 1; i < width; ++i) if (total_cmp(row[i], row[best]) >= 0) best = i;
    out[r] = static_cast<uint32_t>(best);
  }
  return FJO_OK;
}

int fjo_top_k(const void* x, int x_dt, void* values_out, int v_dt, uint32_t* indices_out,
              size_t rows, size_t width, uint32_t k, int normalize) {
  if (k == 0 || k > width) return FJO_EXECUTION_FAILED;
  bool ok;
  auto values = decode_vec(x, x_dt, rows * width, &ok);
  if (!ok) return FJO_EXECUTION_FAILED;
  std::vector<float> selected(rows * k);
  for (size_t r = 0; r < rows; ++r) {
    const float* row = &values[r * width];
    std::vector<size_t> indices(width);
    std::iota(indices.begin(), indices.end(), 0);
    std::sort(indices.begin(), indices.end(), [&](size_t left, size_t right) {
      int c = total_cmp(row[right], row[left]);
      return c != 0 ? c < 0 : left < right;
    });
    float* sel = &selected[r * k];
    for (uint32_t j = 0; j < k; ++j) { sel[j] = row[indices[j]]; indices_out[r * k + j] = static_cast<uint32_t>(indices[j]); }
    if (normalize) {
      float maximum = sel[0];
      for (uint32_t j = 0; j < k; ++j) sel[j] = std::exp(sel[j] - maximum);
      float sum = 0.0f;
      for (uint32_t j = 0; j < k; ++j) sum += sel[j];
      for (uint32_t j = 0; j < k; ++j) sel[j] /= sum;
    }
  }
  return encode(selected.data(), values_out, v_dt, rows * k) ? FJO_OK : FJO_EXECUTION_FAILED;
}

// splitmix64 / sampled_score, lib.rs:1682-1700
static inline uint64_t splitmix64(uint64_t value) {
  value += 0x9e3779b97f4a7c15ULL;
  value = (value ^ (value >> 30)) * 0xbf58476d1ce4e5b9ULL;
  value = (value ^ (value >> 27)) * 0x94d049bb133111ebULL;
  return value ^ (value >> 31);
}
struct SamplingParameters { float temperature; uint32_t top_k; float top_p; uint64_t seed; };
static float sampled_score(float logit, const SamplingParameters& p, uint32_t position, size_t index) {
  if (!std::isfinite(logit)) return logit;
  uint64_t counter = p.seed ^ (static_cast<uint64_t>(position) << 32) ^ static_cast<uint64_t>(index);
  uint64_t random = splitmix64(counter);
  uint32_t mantissa = static_cast<uint32_t>(random >> 40);
  float uniform = (static_cast<float>(mantissa) + 0.5f) * (1.0f / 16777216.0f);
  return logit / p.temperature - std::log(-std::log(uniform));
}
// sample_allowed, lib.rs:1597-1638
static int sample_allowed(const float* row, const SamplingParameters& p, uint32_t position,
                          std::vector<size_t> allowed, uint32_t* out) {
  if (allowed.empty()) return FJO_INVALID_INPUT;
  if (p.temperature == 0.0f || p.top_k == 1) {
    size_t best = allowed[0];
    for (size_t j = 1; j < allowed.size(); ++j) {
      size_t c = allowed[j];
      int cmp = total_cmp(row[c], row[best]);
      if (cmp > 0 || (cmp == 0 && c >= best)) best = c;
    }
    *out = static_cast<uint32_t>(best);
    return FJO_OK;
  }
  std::sort(allowed.begin(), allowed.end(), [&](size_t left, size_t right) {
    int c = total_cmp(row[right], row[left]);
    return c != 0 ? c < 0 : right < left;
  });
  size_t cap = p.top_k == 0 ? allowed.size() : p.top_k;
  allowed.resize(std::min(cap, allowed.size()));
  if (p.top_p < 1.0f) {  // truncate_top_p, lib.rs:1655-1680
    size_t maximum = allowed[0];
    std::vector<float> weights(allowed.size());
    for (size_t j = 0; j < allowed.size(); ++j) weights[j] = std::exp((row[allowed[j]] - row[maximum]) / p.temperature);
    float total = 0.0f;
    for (float w : weights) total += w;
    if (std::isfinite(total) && total > 0.0f) {
      float cumulative = 0.0f;
      size_t keep = weights.size();
      for (size_t j = 0; j < weights.size(); ++j) {
        cumulative += weights[j] / total;
        if (cumulative >= p.top_p) { keep = j + 1; break; }
      }
      allowed.resize(std::max<size_t>(keep, 1));
    } else {
      allowed.resize(1);
    }
  }
  size_t best = allowed[0];
  float best_score = sampled_score(row[best], p, position, best);
  for (size_t j = 1; j < allowed.size(); ++j) {
    size_t c = allowed[j];
    float s = sampled_score(row[c], p, position, c);
    int cmp = total_cmp(s, best_score);
    if (cmp > 0 || (cmp == 0 && c >= best)) { best = c; best_score = s; }
  }
  *out = static_cast<uint32_t>(best);
  return FJO_OK;
}

int fjo_sample(const void* x, int x_dt, const uint32_t* params, const uint32_t* allow,
               uint32_t* out, size_t rows, size_t width, uint32_t position) {
  bool ok;
  auto values = decode_vec(x, x_dt, rows * width, &ok);
  if (!ok) return FJO_EXECUTION_FAILED;
  SamplingParameters p;  // SamplingParameters::from_words, lib.rs:1553-1575
  p.temperature = bits_f32(params[0]);
  p.top_k = params[1];
  p.top_p = bits_f32(params[2]);
  p.seed = static_cast<uint64_t>(params[3]) | (static_cast<uint64_t>(params[4]) << 32);
  if (!std::isfinite(p.temperature) || p.temperature < 0.0f || !std::isfinite(p.top_p) ||
      !(p.top_p >= 0.0f && p.top_p <= 1.0f) || p.top_p == 0.0f)
    return FJO_INVALID_INPUT;
  if (allow) {  // validate_allow_mask, lib.rs:1640-1653
    size_t words = (width + 31) / 32, remainder = width % 32;
    if (remainder != 0 && (allow[words - 1] & ~((1u << remainder) - 1)) != 0) return FJO_INVALID_INPUT;
    bool any = false;
    for (size_t i = 0; i < words; ++i) any |= allow[i] != 0;
    if (!any) return FJO_INVALID_INPUT;
  }
  for (size_t r = 0; r < rows; ++r) {
    std::vector<size_t> allowed;
    for (size_t i = 0; i < width; ++i)
      if (!allow || (allow[i / 32] & (1u << (i % 32))) != 0) allowed.push_back(i);
    int st = sample_allowed(&values[r * width], p, position, std::move(allowed), &out[r]);
    if (st != FJO_OK) return st;
  }
  return FJO_OK;
}

int fjo_rope(const void* x, int x_dt, const uint32_t* positions, void* out, int out_dt,
             size_t tokens, size_t heads, size_t width, float theta) {
  bool ok;
  auto values = decode_vec(x, x_dt, tokens * heads * width, &ok);
  if (!ok) return FJO_EXECUTION_FAILED;
  size_t half = width / 2;
  std::vector<float> inv_freq(half);
  for (size_t i = 0; i < half; ++i)
    inv_freq[i] = 1.0f / std::pow(theta, 2.0f * static_cast<float>(i) / static_cast<float>(width));
  for (size_t t = 0; t < tokens; ++t) {
    for (size_t h = 0; h < heads; ++h) {
      float* head = &values[(t * heads + h) * width];
      for (size_t i = 0; i < half; ++i) {
        float angle = static_cast<float>(positions[t]) * inv_freq[i];
        float s = std::sin(angle), c = std::cos(angle);
        float first = head[i], second = head[i + half];
        head[i] = first * c - second * s;
        head[i + half] = second * c + first * s;
      }
    }
  }
  return encode(values.data(), out, out_dt, values.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

int fjo_embed(const void* table, int t_dt, const uint32_t* ids, void* out, int out_dt,
              size_t vocab, size_t width, size_t count, uint32_t* bad_index) {
  std::vector<float> values(count * width, 0.0f);
  bool have = false; uint32_t lowest = 0;
  const size_t esz = dtype_size(t_dt);
  for (size_t i = 0; i < count; ++i) {
    if (ids[i] < vocab) {
      if (!decode(static_cast<const char*>(table) + static_cast<size_t>(ids[i]) * width * esz, t_dt, &values[i * width], width))
        return FJO_EXECUTION_FAILED;
    } else {
      record_invalid(&have, &lowest, ids[i]);
    }
  }
  if (!encode(values.data(), out, out_dt, values.size())) return FJO_EXECUTION_FAILED;
  if (have) { if (bad_index) *bad_index = lowest; return FJO_INDEX_OUT_OF_RANGE; }
  return FJO_OK;
}

int fjo_quant_embed(const uint32_t* packed, const void* scales_p, const void* biases_p, int p_dt,
                    const uint32_t* ids, void* out, int out_dt, size_t vocab, size_t packed_width,
                    size_t count, uint32_t bits, uint32_t group_size, uint32_t* bad_index) {
  const size_t values_per_word = 32 / bits;
  const size_t width = packed_width * values_per_word;
  const size_t groups = width / group_size;
  const uint32_t mask = (1u << bits) - 1;
  bool ok1, ok2;
  auto scales = decode_vec(scales_p, p_dt, vocab * groups, &ok1);
  auto biases = decode_vec(biases_p, p_dt, vocab * groups, &ok2);
  if (!ok1 || !ok2) return FJO_EXECUTION_FAILED;
  std::vector<float> values(count * width, 0.0f);
  bool have = false; uint32_t lowest = 0;
  for (size_t i = 0; i < count; ++i) {
    size_t row = ids[i];
    if (row >= vocab) { record_invalid(&have, &lowest, ids[i]); continue; }
    for (size_t column = 0; column < width; ++column) {
      uint32_t word = packed[row * packed_width + column / values_per_word];
      uint32_t quantized = (word >> ((column % values_per_word) * bits)) & mask;
      size_t group = row * groups + column / group_size;
      values[i * width + column] = scales[group] * static_cast<float>(quantized) + biases[group];
    }
  }
  if (!encode(values.data(), out, out_dt, values.size())) return FJO_EXECUTION_FAILED;
  if (have) { if (bad_index) *bad_index = lowest; return FJO_INDEX_OUT_OF_RANGE; }
  return FJO_OK;
}

int fjo_matmul(const void* left_p, int l_dt, const void* right_p, int r_dt, void* out, int out_dt,
               size_t batch, size_t rows, size_t inner, size_t cols, int right_transposed) {
  bool ok1, ok2;
  auto left = decode_vec(left_p, l_dt, batch * rows * inner, &ok1);
  auto right = decode_vec(right_p, r_dt, batch * inner * cols, &ok2);
  if (!ok1 || !ok2) return FJO_EXECUTION_FAILED;
  std::vector<float> values(batch * rows * cols);
  for (size_t b = 0; b < batch; ++b) {
    const float* lb = &left[b * rows * inner];
    const float* rb = &right[b * inner * cols];
    float* ob = &values[b * rows * cols];
#pragma omp parallel for collapse(2) if (g_threads > 1)
    for (size_t r = 0; r < rows; ++r) {
      for (size_t c = 0; c < cols; ++c) {
        const float* row = lb + r * inner;
        float sum = 0.0f;  // fold(0.0, |sum, (l, b_row)| sum + l * b_row[column]), k ascending
        if (right_transposed) {
          const float* col = rb + c * inner;
          for (size_t k = 0; k < inner; ++k) sum = sum + row[k] * col[k];
        } else {
          for (size_t k = 0; k < inner; ++k) sum = sum + row[k] * rb[k * cols + c];
        }
        ob[r * cols + c] = sum;
      }
    }
  }
  return encode(values.data(), out, out_dt, values.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

int fjo_quant_matmul(const void* x, int x_dt, const uint32_t* packed, const void* scales_p,
                     const void* biases_p, int p_dt, void* out, int out_dt, size_t rows,
                     size_t inner, size_t cols, uint32_t bits, uint32_t group_size) {
  const size_t packed_width = inner * bits / 32;
  const size_t group_count = inner / group_size;
  bool ok0, ok1, ok2;
  auto activations = decode_vec(x, x_dt, rows * inner, &ok0);
  auto scales = decode_vec(scales_p, p_dt, cols * group_count, &ok1);
  auto biases = decode_vec(biases_p, p_dt, cols * group_count, &ok2);
  if (!ok0 || !ok1 || !ok2) return FJO_EXECUTION_FAILED;
  std::vector<float> values(rows * cols);
#pragma omp parallel for collapse(2) if (g_threads > 1)
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c)
      values[r * cols + c] = affine_quant_dot(&activations[r * inner], inner, packed, scales.data(), biases.data(),
                                              c * packed_width, c * group_count, group_size, bits);
  return encode(values.data(), out, out_dt, values.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

// execute_gather_matmul, crates/forja-cpu/src/lib.rs:850-912: out[r, j, c] = sum_i x[r, i] * W[idx[r, j], i, c]
// (dense experts stored [experts, inner, columns]); a route naming a missing expert leaves zeros and the
// lowest such id is reported after everything else was written.
int fjo_gather_matmul(const void* x, int x_dt, const void* weights_p, int w_dt, const uint32_t* indices, void* out, int out_dt,
                      size_t rows, size_t inner, size_t experts, size_t cols, size_t routes, uint32_t* bad_index) {
  bool ok0, ok1;
  auto activations = decode_vec(x, x_dt, rows * inner, &ok0);
  auto weights = decode_vec(weights_p, w_dt, experts * inner * cols, &ok1);
  if (!ok0 || !ok1) return FJO_EXECUTION_FAILED;
  std::vector<float> values(rows * routes * cols, 0.0f);
  bool have = false; uint32_t lowest = 0;
  for (size_t r = 0; r < rows * routes; ++r)
    if (indices[r] >= experts) record_invalid(&have, &lowest, indices[r]);
#pragma omp parallel for collapse(2) if (g_threads > 1)
  for (size_t r = 0; r < rows; ++r) {
    for (size_t j = 0; j < routes; ++j) {
      const size_t expert = indices[r * routes + j];
      if (expert >= experts) continue;
      const float* w = &weights[expert * inner * cols];
      for (size_t c = 0; c < cols; ++c) {
        float sum = 0.0f;
        for (size_t i = 0; i < inner; ++i) sum = sum + activations[r * inner + i] * w[i * cols + c];
        values[(r * routes + j) * cols + c] = sum;
      }
    }
  }
  if (!encode(values.data(), out, out_dt, values.size())) return FJO_EXECUTION_FAILED;
  if (have) { if (bad_index) *bad_index = lowest; return FJO_INDEX_OUT_OF_RANGE; }
  return FJO_OK;
}

int fjo_gather_quant_matmul(const void* x, int x_dt, const uint32_t* packed, const void* scales_p,
                            const void* biases_p, int p_dt, const uint32_t* indices, void* out,
                            int out_dt, size_t rows, size_t inner, size_t experts, size_t cols,
                            size_t k, uint32_t bits, uint32_t group_size, uint32_t* bad_index) {
  const size_t packed_width = inner * bits / 32;
  const size_t group_count = inner / group_size;
  const size_t expert_packed = cols * packed_width, expert_groups = cols * group_count;
  bool ok0, ok1, ok2;
  auto activations = decode_vec(x, x_dt, rows * inner, &ok0);
  auto scales = decode_vec(scales_p, p_dt, experts * expert_groups, &ok1);
  auto biases = decode_vec(biases_p, p_dt, experts * expert_groups, &ok2);
  if (!ok0 || !ok1 || !ok2) return FJO_EXECUTION_FAILED;
  std::vector<float> values(rows * k * cols, 0.0f);
  bool have = false; uint32_t lowest = 0;
  for (size_t r = 0; r < rows; ++r)
    for (size_t j = 0; j < k; ++j)
      if (indices[r * k + j] >= experts) record_invalid(&have, &lowest, indices[r * k + j]);
#pragma omp parallel for collapse(2) if (g_threads > 1)
  for (size_t r = 0; r < rows; ++r) {
    for (size_t j = 0; j < k; ++j) {
      size_t expert = indices[r * k + j];
      if (expert >= experts) continue;
      for (size_t c = 0; c < cols; ++c)
        values[(r * k + j) * cols + c] =
            affine_quant_dot(&activations[r * inner], inner, packed, scales.data(), biases.data(),
                             expert * expert_packed + c * packed_width, expert * expert_groups + c * group_count,
                             group_size, bits);
    }
  }
  if (!encode(values.data(), out, out_dt, values.size())) return FJO_EXECUTION_FAILED;
  if (have) { if (bad_index) *bad_index = lowest; return FJO_INDEX_OUT_OF_RANGE; }
  return FJO_OK;
}

int fjo_gather_quant_weighted_sum(const void* act, int a_dt, const uint32_t* packed,
                                  const void* scales_p, const void* biases_p, int p_dt,
                                  const uint32_t* indices, const void* weights_p, int w_dt,
                                  void* out, int out_dt, size_t rows, size_t routes, size_t inner,
                                  size_t experts, size_t cols, uint32_t bits, uint32_t group_size,
                                  uint32_t* bad_index) {
  const size_t packed_width = inner * bits / 32;
  const size_t group_count = inner / group_size;
  const size_t expert_packed = cols * packed_width, expert_groups = cols * group_count;
  bool ok0, ok1, ok2, ok3;
  auto activations = decode_vec(act, a_dt, rows * routes * inner, &ok0);
  auto scales = decode_vec(scales_p, p_dt, experts * expert_groups, &ok1);
  auto biases = decode_vec(biases_p, p_dt, experts * expert_groups, &ok2);
  auto weights = decode_vec(weights_p, w_dt, rows * routes, &ok3);
  if (!ok0 || !ok1 || !ok2 || !ok3) return FJO_EXECUTION_FAILED;
  std::vector<float> values(rows * cols, 0.0f);
  bool have = false; uint32_t lowest = 0;
  for (size_t i = 0; i < rows * routes; ++i)
    if (indices[i] >= experts) record_invalid(&have, &lowest, indices[i]);
#pragma omp parallel for if (g_threads > 1)
  for (size_t r = 0; r < rows; ++r) {
    for (size_t route = 0; route < routes; ++route) {
      size_t route_offset = r * routes + route;
      size_t expert = indices[route_offset];
      if (expert >= experts) continue;
      const float* activation = &activations[route_offset * inner];
      float route_weight = weights[route_offset];
      for (size_t c = 0; c < cols; ++c) {
        float value = affine_quant_dot(activation, inner, packed, scales.data(), biases.data(),
                                       expert * expert_packed + c * packed_width,
                                       expert * expert_groups + c * group_count, group_size, bits);
        values[r * cols + c] += route_weight * value;
      }
    }
  }
  if (!encode(values.data(), out, out_dt, values.size())) return FJO_EXECUTION_FAILED;
  if (have) { if (bad_index) *bad_index = lowest; return FJO_INDEX_OUT_OF_RANGE; }
  return FJO_OK;
}

int fjo_sdpa(const void* q, int q_dt, const void* k, int k_dt, const void* v, int v_dt, void* out,
             int out_dt, size_t q_heads, size_t q_len, size_t width, size_t kv_heads,
             size_t kv_len, size_t value_width, float scale, int causal, uint32_t q_start) {
  bool ok0, ok1, ok2;
  auto query = decode_vec(q, q_dt, q_heads * q_len * width, &ok0);
  auto key = decode_vec(k, k_dt, kv_heads * kv_len * width, &ok1);
  auto value = decode_vec(v, v_dt, kv_heads * kv_len * value_width, &ok2);
  if (!ok0 || !ok1 || !ok2 || kv_heads == 0 || q_heads % kv_heads != 0) return FJO_EXECUTION_FAILED;
  // a causal window must end inside the cache (crates/forja-core/src/ops.rs check_sdpa: q_start + q_len <= kv_len)
  if (causal && static_cast<uint64_t>(q_start) + q_len > kv_len) return FJO_INVALID_INPUT;
  size_t group = q_heads / kv_heads;
  std::vector<float> result(q_heads * q_len * value_width);
  for (size_t h = 0; h < q_heads; ++h) {
    size_t kvh = h / group;
    const float* key_rows = &key[kvh * kv_len * width];
    const float* value_rows = &value[kvh * kv_len * value_width];
    for (size_t qi = 0; qi < q_len; ++qi) {
      const float* q_row = &query[(h * q_len + qi) * width];
      size_t attended = causal ? std::min<size_t>(static_cast<size_t>(q_start) + qi + 1, kv_len) : kv_len;
      std::vector<float> scores(attended);
      for (size_t t = 0; t < attended; ++t) {
        float sum = 0.0f;
        for (size_t c = 0; c < width; ++c) sum = sum + q_row[c] * key_rows[t * width + c];
        scores[t] = sum * scale;
      }
      softmax_lib(scores);
      for (size_t c = 0; c < value_width; ++c) {
        float sum = 0.0f;
        for (size_t t = 0; t < attended; ++t) sum = sum + scores[t] * value_rows[t * value_width + c];
        result[(h * q_len + qi) * value_width + c] = sum;
      }
    }
  }
  return encode(result.data(), out, out_dt, result.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

// ---- direct restatements of the guest programs (blocks.rs:380-444), interpreter order ----

int fjo_prog_rms_norm(const void* x, int dt, const void* w, int w_dt, void* out, int out_dt,
                      size_t rows, size_t width, float eps) {
  bool ok1, ok2;
  auto values = decode_vec(x, dt, rows * width, &ok1);
  auto weights = decode_vec(w, w_dt, width, &ok2);
  if (!ok1 || !ok2) return FJO_EXECUTION_FAILED;
  std::vector<float> result(rows * width);
  const float extent = static_cast<float>(static_cast<uint32_t>(width));
#pragma omp parallel for if (g_threads > 1)
  for (size_t r = 0; r < rows; ++r) {
    const float* row = &values[r * width];
    float sum = 0.0f;
    for (size_t i = 0; i < width; ++i) sum = sum + row[i] * row[i];
    float inverse = 1.0f / std::sqrt(sum / extent + eps);  // Rsqrt = sqrt().recip(), interpreter.rs:290
    for (size_t i = 0; i < width; ++i) result[r * width + i] = row[i] * inverse * weights[i];
  }
  return encode(result.data(), out, out_dt, result.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

int fjo_prog_residual_norm(const void* residual, const void* update, int dt, const void* w, int w_dt,
                           void* sum_out, void* norm_out, int out_dt, size_t rows, size_t width,
                           float eps) {
  bool ok0, ok1, ok2;
  auto res = decode_vec(residual, dt, rows * width, &ok0);
  auto upd = decode_vec(update, dt, rows * width, &ok1);
  auto weights = decode_vec(w, w_dt, width, &ok2);
  if (!ok0 || !ok1 || !ok2) return FJO_EXECUTION_FAILED;
  std::vector<float> value(rows * width), norm(rows * width);
  const float extent = static_cast<float>(static_cast<uint32_t>(width));
#pragma omp parallel for if (g_threads > 1)
  for (size_t r = 0; r < rows; ++r) {
    float sum = 0.0f;
    for (size_t i = 0; i < width; ++i) {
      float v = res[r * width + i] + upd[r * width + i];
      value[r * width + i] = v;
      sum = sum + v * v;
    }
    float inverse = 1.0f / std::sqrt(sum / extent + eps);
    for (size_t i = 0; i < width; ++i) norm[r * width + i] = value[r * width + i] * inverse * weights[i];
  }
  if (!encode(value.data(), sum_out, out_dt, value.size())) return FJO_EXECUTION_FAILED;
  return encode(norm.data(), norm_out, out_dt, norm.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

int fjo_prog_add(const void* a, const void* b, int dt, void* out, int out_dt, size_t n) {
  bool ok0, ok1;
  auto x = decode_vec(a, dt, n, &ok0);
  auto y = decode_vec(b, dt, n, &ok1);
  if (!ok0 || !ok1) return FJO_EXECUTION_FAILED;
  for (size_t i = 0; i < n; ++i) x[i] = x[i] + y[i];
  return encode(x.data(), out, out_dt, n) ? FJO_OK : FJO_EXECUTION_FAILED;
}

int fjo_prog_silu_mul(const void* gate, const void* up, int dt, void* out, int out_dt, size_t n) {
  bool ok0, ok1;
  auto g = decode_vec(gate, dt, n, &ok0);
  auto u = decode_vec(up, dt, n, &ok1);
  if (!ok0 || !ok1) return FJO_EXECUTION_FAILED;
#pragma omp parallel for if (g_threads > 1)
  for (size_t i = 0; i < n; ++i) {
    float sigmoid = 1.0f / (1.0f + std::exp(-g[i]));  // interpreter.rs:294
    g[i] = g[i] * sigmoid * u[i];
  }
  return encode(g.data(), out, out_dt, n) ? FJO_OK : FJO_EXECUTION_FAILED;
}

int fjo_prog_qk_norm_rope(const void* x, int dt, const void* w, int w_dt, int per_head_weight,
                          const float* positions, void* out, int out_dt, size_t tokens,
                          size_t heads, size_t width, float eps, float theta) {
  const size_t half = width / 2;
  bool ok0, ok1;
  auto values = decode_vec(x, dt, tokens * heads * width, &ok0);
  auto weights = decode_vec(w, w_dt, per_head_weight ? heads * width : width, &ok1);
  if (!ok0 || !ok1) return FJO_EXECUTION_FAILED;
  std::vector<float> result(values.size());
  const float head_dim = static_cast<float>(width);
  const float exponent_scale = -2.0f / head_dim;
#pragma omp parallel for collapse(2) if (g_threads > 1)
  for (size_t t = 0; t < tokens; ++t) {
    for (size_t h = 0; h < heads; ++h) {
      const float* lo = &values[(t * heads + h) * width];
      const float* hi = lo + half;
      const float* wl = per_head_weight ? &weights[h * width] : weights.data();
      const float* wh = wl + half;
      float square_sum = 0.0f;
      for (size_t i = 0; i < half; ++i) square_sum = square_sum + (lo[i] * lo[i] + hi[i] * hi[i]);
      float inverse = 1.0f / std::sqrt(square_sum / head_dim + eps);
      float* olo = &result[(t * heads + h) * width];
      float* ohi = olo + half;
      for (size_t i = 0; i < half; ++i) {
        float nlo = lo[i] * inverse * wl[i];
        float nhi = hi[i] * inverse * wh[i];
        float exponent = static_cast<float>(static_cast<uint32_t>(i)) * exponent_scale;
        float angle = positions[t] * std::pow(theta, exponent);
        float c = std::cos(angle), s = std::sin(angle);
        olo[i] = nlo * c - nhi * s;
        ohi[i] = nhi * c + nlo * s;
      }
    }
  }
  return encode(result.data(), out, out_dt, result.size()) ? FJO_OK : FJO_EXECUTION_FAILED;
}

}  // extern "C"
