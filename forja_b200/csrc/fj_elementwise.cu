// Elementwise, normalisation, rotary, gather and selection kernels of the forward step.
// Reference semantics: crates/forja-cpu/src/lib.rs:171-187 (copy), :495-608 (rms_norm, argmax,
// top_k), :681-813 (rope, embed, quant_embed) and the guest programs of
// crates/forja-sdk/src/nn/blocks.rs:380-444 as evaluated by crates/forja-cpu/src/interpreter.rs.
// All of these are HBM-bound: one pass over the data, f32 math, one rounding per stored output.
#include "fj_kernels.h"

namespace fj {

namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(size_t n, int threads, int sm_count) {
  size_t blocks = (n + threads - 1) / threads;
  size_t cap = static_cast<size_t>(sm_count) * 32;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  return static_cast<unsigned>(blocks);
}

__global__ void copy_kernel(View in, View out, size_t n) {
  const bool raw = (in.dtype == I32 || in.dtype == U32);
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    size_t src = view_offset(in, i), dst = view_offset(out, i);
    if (raw || (in.dtype == out.dtype && in.dtype == F32)) {
      static_cast<unsigned*>(out.base)[dst] = static_cast<const unsigned*>(in.base)[src];
    } else if (in.dtype == out.dtype) {
      static_cast<unsigned short*>(out.base)[dst] = static_cast<const unsigned short*>(in.base)[src];
    } else {
      store_from_f32(out.base, out.dtype, dst, load_as_f32(in.base, in.dtype, src));
    }
  }
}

__global__ void add_kernel(View a, View b, View out, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float x = load_as_f32(a.base, a.dtype, view_offset(a, i));
    float y = load_as_f32(b.base, b.dtype, view_offset(b, i));
    store_from_f32(out.base, out.dtype, view_offset(out, i), x + y);
  }
}

__device__ inline float sigmoid_ref(float v) { return 1.0f / (1.0f + expf(-v)); }  // interpreter.rs:294

__global__ void silu_mul_kernel(View gate, View up, View out, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float g = load_as_f32(gate.base, gate.dtype, view_offset(gate, i));
    float u = load_as_f32(up.base, up.dtype, view_offset(up, i));
    store_from_f32(out.base, out.dtype, view_offset(out, i), g * sigmoid_ref(g) * u);
  }
}

// One warp per row; lanes stride over the last axis.
__global__ void rms_norm_kernel(View x, View w, View out, size_t rows, unsigned width, float eps) {
  const int lane = threadIdx.x & 31;
  const size_t warps_per_block = blockDim.x >> 5;
  for (size_t row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += static_cast<size_t>(gridDim.x) * warps_per_block) {
    float sum = 0.0f;
    for (unsigned i = lane; i < width; i += 32) {
      float v = load_as_f32(x.base, x.dtype, view_offset(x, row * width + i));
      sum += v * v;
    }
    sum = warp_sum(sum);
    const float inverse = 1.0f / sqrtf(sum / static_cast<float>(width) + eps);
    for (unsigned i = lane; i < width; i += 32) {
      size_t e = row * width + i;
      float v = load_as_f32(x.base, x.dtype, view_offset(x, e));
      float g = load_as_f32(w.base, w.dtype, view_offset(w, e));
      store_from_f32(out.base, out.dtype, view_offset(out, e), v * inverse * g);
    }
  }
}

__global__ void residual_norm_kernel(View residual, View update, View w, View sum_out, View norm_out, size_t rows, int round_sum,
                                     unsigned width, float eps) {
  const int lane = threadIdx.x & 31;
  const size_t warps_per_block = blockDim.x >> 5;
  for (size_t row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += static_cast<size_t>(gridDim.x) * warps_per_block) {
    float sum = 0.0f;
    for (unsigned i = lane; i < width; i += 32) {
      size_t e = row * width + i;
      float v = load_as_f32(residual.base, residual.dtype, view_offset(residual, e)) +
                load_as_f32(update.base, update.dtype, view_offset(update, e));
      if (round_sum) v = round_through(v, sum_out.dtype);
      sum += v * v;
    }
    sum = warp_sum(sum);
    const float inverse = 1.0f / sqrtf(sum / static_cast<float>(width) + eps);
    for (unsigned i = lane; i < width; i += 32) {
      size_t e = row * width + i;
      // the row program normalises the unrounded f32 sum; the unfused add + rms_norm pair of the
      // SmolLM2 graph normalises the sum after it was stored (round_sum)
      float v = load_as_f32(residual.base, residual.dtype, view_offset(residual, e)) +
                load_as_f32(update.base, update.dtype, view_offset(update, e));
      if (round_sum) v = round_through(v, sum_out.dtype);
      float g = load_as_f32(w.base, w.dtype, view_offset(w, e));
      store_from_f32(norm_out.base, norm_out.dtype, view_offset(norm_out, e), v * inverse * g);
      store_from_f32(sum_out.base, sum_out.dtype, view_offset(sum_out, e), v);
    }
  }
}

__device__ inline float position_value(const View& pos, size_t e) {
  size_t off = view_offset(pos, e);
  if (pos.dtype == U32) return static_cast<float>(static_cast<const unsigned*>(pos.base)[off]);
  return load_as_f32(pos.base, pos.dtype, off);
}

// qk_norm_rope_rows (blocks.rs:419-444): one warp per half row.
__global__ void qk_norm_rope_kernel(View lo, View hi, View wlo, View whi, View pos, View out_lo, View out_hi, size_t rows,
                                    unsigned half, float head_dim, float eps, const float* __restrict__ inv_freq) {
  const int lane = threadIdx.x & 31;
  const size_t warps_per_block = blockDim.x >> 5;
  for (size_t row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += static_cast<size_t>(gridDim.x) * warps_per_block) {
    float sum = 0.0f;
    for (unsigned i = lane; i < half; i += 32) {
      size_t e = row * half + i;
      float a = load_as_f32(lo.base, lo.dtype, view_offset(lo, e));
      float b = load_as_f32(hi.base, hi.dtype, view_offset(hi, e));
      sum += a * a + b * b;
    }
    sum = warp_sum(sum);
    const float inverse = 1.0f / sqrtf(sum / head_dim + eps);
    for (unsigned i = lane; i < half; i += 32) {
      size_t e = row * half + i;
      float a = load_as_f32(lo.base, lo.dtype, view_offset(lo, e)) * inverse * load_as_f32(wlo.base, wlo.dtype, view_offset(wlo, e));
      float b = load_as_f32(hi.base, hi.dtype, view_offset(hi, e)) * inverse * load_as_f32(whi.base, whi.dtype, view_offset(whi, e));
      float angle = position_value(pos, e) * inv_freq[i];
      float s, c;
      sincosf(angle, &s, &c);
      store_from_f32(out_lo.base, out_lo.dtype, view_offset(out_lo, e), a * c - b * s);
      store_from_f32(out_hi.base, out_hi.dtype, view_offset(out_hi, e), b * c + a * s);
    }
  }
}

__global__ void rope_pairs_kernel(View first, View second, View pos, View out_first, View out_second, size_t n, unsigned half,
                                  const float* __restrict__ inv_freq) {
  for (size_t e = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; e < n; e += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float a = load_as_f32(first.base, first.dtype, view_offset(first, e));
    float b = load_as_f32(second.base, second.dtype, view_offset(second, e));
    float angle = position_value(pos, e) * inv_freq[e % half];
    float s, c;
    sincosf(angle, &s, &c);
    store_from_f32(out_first.base, out_first.dtype, view_offset(out_first, e), a * c - b * s);
    store_from_f32(out_second.base, out_second.dtype, view_offset(out_second, e), b * c + a * s);
  }
}

__global__ void embed_kernel(const void* table, int t_dt, const unsigned* __restrict__ ids, void* out, int out_dt, unsigned vocab,
                             unsigned width, unsigned count, ErrorRecord* err) {
  for (unsigned row = blockIdx.x; row < count; row += gridDim.x) {
    unsigned id = ids[row];
    bool ok = id < vocab;
    if (!ok && threadIdx.x == 0) report_error(err, ERR_INDEX, id);
    for (unsigned i = threadIdx.x; i < width; i += blockDim.x) {
      float v = ok ? load_as_f32(table, t_dt, static_cast<size_t>(id) * width + i) : 0.0f;
      store_from_f32(out, out_dt, static_cast<size_t>(row) * width + i, v);
    }
  }
}

__global__ void quant_embed_kernel(const unsigned* __restrict__ packed, const void* scales, const void* biases, int p_dt,
                                   const unsigned* __restrict__ ids, void* out, int out_dt, unsigned vocab, unsigned packed_width,
                                   unsigned count, unsigned bits, unsigned group_size, ErrorRecord* err) {
  const unsigned vpw = 32 / bits, width = packed_width * vpw, groups = width / group_size, mask = (1u << bits) - 1;
  for (unsigned row = blockIdx.x; row < count; row += gridDim.x) {
    unsigned id = ids[row];
    bool ok = id < vocab;
    if (!ok && threadIdx.x == 0) report_error(err, ERR_INDEX, id);
    for (unsigned c = threadIdx.x; c < width; c += blockDim.x) {
      float v = 0.0f;
      if (ok) {
        unsigned word = packed[static_cast<size_t>(id) * packed_width + c / vpw];
        unsigned q = (word >> ((c % vpw) * bits)) & mask;
        size_t g = static_cast<size_t>(id) * groups + c / group_size;
        // separate multiply and add (no FMA contraction): same two roundings as the reference
        v = __fadd_rn(__fmul_rn(load_as_f32(scales, p_dt, g), static_cast<float>(q)), load_as_f32(biases, p_dt, g));
      }
      store_from_f32(out, out_dt, static_cast<size_t>(row) * width + c, v);
    }
  }
}

// ---- argmax: chunked partials + finalize. key = (total-order key << 32) | index, max wins, so
// equal values select the highest index (crates/forja-core/src/ops.rs:184-186).
constexpr unsigned kArgmaxChunk = 4096;

__global__ void argmax_partial_kernel(const void* x, int dt, size_t row_stride, unsigned width, unsigned chunks,
                                      unsigned long long* partial) {
  pdl_sync();
  const unsigned row = blockIdx.y, chunk = blockIdx.x;
  const unsigned begin = chunk * kArgmaxChunk;
  const unsigned end = min(width, begin + kArgmaxChunk);
  unsigned long long best = 0;
  for (unsigned i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const unsigned bits = load_f32_bits(x, dt, static_cast<size_t>(row) * row_stride + i);
    unsigned long long key = (static_cast<unsigned long long>(total_order_key_bits(bits)) << 32) | i;
    best = key > best ? key : best;
  }
  best = warp_max_u64(best);
  __shared__ unsigned long long warp_best[8];
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (unsigned w = 1; w < (blockDim.x >> 5); ++w) best = warp_best[w] > best ? warp_best[w] : best;
    partial[static_cast<size_t>(row) * chunks + chunk] = best;
  }
}

__global__ void argmax_final_kernel(const unsigned long long* partial, unsigned chunks, unsigned* out, unsigned rows) {
  pdl_sync();
  unsigned row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  unsigned long long best = 0;
  for (unsigned c = threadIdx.x & 31; c < chunks; c += 32) {
    unsigned long long k = partial[static_cast<size_t>(row) * chunks + c];
    best = k > best ? k : best;
  }
  best = warp_max_u64(best);
  if ((threadIdx.x & 31) == 0) out[row] = static_cast<unsigned>(best & 0xFFFFFFFFull);
}

// ---- top-k: one CTA per row, k rounds of block-wide max over (key << 32 | ~index) so that equal
// values select the lower index first (crates/forja-cpu/src/lib.rs:572-584).
__global__ void top_k_kernel(const void* x, int dt, void* values, int v_dt, unsigned* indices, unsigned width, unsigned k,
                             int normalize) {
  pdl_sync();
  extern __shared__ unsigned long long keys[];  // width entries
  __shared__ unsigned long long warp_best[8];
  __shared__ unsigned long long selected;
  __shared__ float chosen[64];
  const unsigned row = blockIdx.x;
  for (unsigned i = threadIdx.x; i < width; i += blockDim.x) {
    const unsigned bits = load_f32_bits(x, dt, static_cast<size_t>(row) * width + i);
    keys[i] = (static_cast<unsigned long long>(total_order_key_bits(bits)) << 32) | (0xFFFFFFFFu - i);
  }
  __syncthreads();
  for (unsigned j = 0; j < k; ++j) {
    unsigned long long best = 0;
    for (unsigned i = threadIdx.x; i < width; i += blockDim.x) best = keys[i] > best ? keys[i] : best;
    best = warp_max_u64(best);
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (unsigned w = 1; w < (blockDim.x >> 5); ++w) best = warp_best[w] > best ? warp_best[w] : best;
      unsigned index = 0xFFFFFFFFu - static_cast<unsigned>(best & 0xFFFFFFFFull);
      selected = best;
      keys[index] = 0;  // below every real key (real keys have a nonzero low word or high word)
      indices[static_cast<size_t>(row) * k + j] = index;
      const unsigned bits = key_to_bits(static_cast<unsigned>(best >> 32));
      if (normalize) chosen[j] = __uint_as_float(bits);
      else if (v_dt == F32) static_cast<unsigned*>(values)[static_cast<size_t>(row) * k + j] = bits;  // NaN payloads survive
      else store_from_f32(values, v_dt, static_cast<size_t>(row) * k + j, __uint_as_float(bits));
    }
    __syncthreads();
  }
  if (normalize && threadIdx.x == 0) {
    // sequential, in selection order, like the reference (lib.rs:585-595)
    float maximum = chosen[0], sum = 0.0f;
    for (unsigned j = 0; j < k; ++j) { chosen[j] = expf(chosen[j] - maximum); }
    for (unsigned j = 0; j < k; ++j) sum += chosen[j];
    for (unsigned j = 0; j < k; ++j) store_from_f32(values, v_dt, static_cast<size_t>(row) * k + j, chosen[j] / sum);
  }
  (void)selected;
}

// ---- fused q/k norm + rope + KV append (dense step). One warp per (row, head) over q, k and v heads.
template <typename T>
__global__ void qknorm_rope_append_kernel(const T* __restrict__ qkv, const T* __restrict__ q_norm_w, const T* __restrict__ k_norm_w,
                                          const unsigned* __restrict__ positions, const unsigned* __restrict__ slot_mapping,
                                          T* __restrict__ q_out, T* __restrict__ k_plane, T* __restrict__ v_plane, unsigned rows,
                                          unsigned q_heads, unsigned kv_heads, unsigned head_dim, float eps,
                                          const float* __restrict__ inv_freq, int qk_norm, unsigned plane_slots) {
  pdl_sync();
  const unsigned heads_total = q_heads + 2 * kv_heads;
  const unsigned half = head_dim / 2;
  const int lane = threadIdx.x & 31;
  const size_t warps_per_block = blockDim.x >> 5;
  const size_t items = static_cast<size_t>(rows) * heads_total;
  for (size_t item = blockIdx.x * warps_per_block + (threadIdx.x >> 5); item < items; item += static_cast<size_t>(gridDim.x) * warps_per_block) {
    const unsigned row = static_cast<unsigned>(item / heads_total), head = static_cast<unsigned>(item % heads_total);
    const T* src = qkv + static_cast<size_t>(row) * heads_total * head_dim + static_cast<size_t>(head) * head_dim;
    const unsigned slot = slot_mapping[row];
    if (head >= q_heads + kv_heads) {  // value head: straight copy into the V plane
      if (slot >= plane_slots) continue;
      T* dst = v_plane + (static_cast<size_t>(slot) * kv_heads + (head - q_heads - kv_heads)) * head_dim;
      for (unsigned i = lane; i < head_dim; i += 32) dst[i] = src[i];
      continue;
    }
    const bool is_q = head < q_heads;
    T* dst;
    if (is_q) dst = q_out + (static_cast<size_t>(row) * q_heads + head) * head_dim;
    else {
      if (slot >= plane_slots) continue;
      dst = k_plane + (static_cast<size_t>(slot) * kv_heads + (head - q_heads)) * head_dim;
    }
    float inverse = 1.0f;
    const T* w = is_q ? q_norm_w : k_norm_w;
    if (qk_norm) {
      float sum = 0.0f;
      for (unsigned i = lane; i < half; i += 32) {
        float a = to_f32(src[i]), b = to_f32(src[i + half]);
        sum += a * a + b * b;
      }
      sum = warp_sum(sum);
      inverse = 1.0f / sqrtf(sum / static_cast<float>(head_dim) + eps);
    }
    const float position = static_cast<float>(positions[row]);
    for (unsigned i = lane; i < half; i += 32) {
      float a = to_f32(src[i]), b = to_f32(src[i + half]);
      if (qk_norm) {
        a = a * inverse * to_f32(w[i]);
        b = b * inverse * to_f32(w[i + half]);
      }
      float s, c;
      sincosf(position * inv_freq[i], &s, &c);
      // the reference materialises the rotated tensor in the activation dtype before the paged
      // copy converts it to the plane dtype; both are T here, so one rounding is identical
      dst[i] = from_f32<T>(a * c - b * s);
      dst[i + half] = from_f32<T>(b * c + a * s);
    }
  }
}

// ---- dense fast paths: rows of 16-bit elements, 16-byte vector accesses, one CTA per row -------
// Same arithmetic as the generic kernels above; chosen by the launchers when every operand is a
// plain row-major matrix (last stride 1, 16-byte aligned rows, width a multiple of 8).

struct DenseRow {
  bool ok;
  char* base;
  size_t row_stride;  // elements
};

inline DenseRow dense_rows(const View& v, size_t rows, unsigned width, bool broadcast_rows) {
  DenseRow d{false, static_cast<char*>(v.base), 0};
  if (v.dtype != BF16 && v.dtype != F16) return d;
  if (v.rank < 1 || v.shape[v.rank - 1] != width || v.strides[v.rank - 1] != 1) return d;
  // leading axes must collapse to one row index
  size_t expect = 0;
  for (int a = v.rank - 2; a >= 0; --a) {
    if (v.shape[a] == 1) continue;
    if (expect == 0) { d.row_stride = v.strides[a]; expect = v.strides[a] * v.shape[a]; }
    else if (v.strides[a] != expect) return d;
    else expect *= v.shape[a];
  }
  if (broadcast_rows ? d.row_stride != 0 : (rows > 1 && d.row_stride < width)) return d;
  if (width % 8 != 0 || d.row_stride % 8 != 0 || reinterpret_cast<size_t>(v.base) % 16 != 0) return d;
  d.ok = true;
  return d;
}

template <typename T> __device__ inline void unpack8(const uint4& v, float* out) {
  const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = to_f32(p[i]);
}
template <typename T> __device__ inline uint4 pack8(const float* in) {
  uint4 v;
  T* p = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < 8; ++i) p[i] = from_f32<T>(in[i]);
  return v;
}

// residual == nullptr: plain rms_norm of `update`.
template <typename T>
__global__ void __launch_bounds__(128) norm_dense_kernel(const T* residual, size_t r_stride, const T* update, size_t u_stride, const T* __restrict__ w,
                                                         T* sum_out, size_t s_stride, T* norm_out, size_t n_stride, unsigned width, float eps,
                                                         int round_sum) {
  __shared__ float red[32];
  pdl_sync();
  const size_t row = blockIdx.x;
  const unsigned vecs = width / 8;
  float sum = 0.0f;
  for (unsigned v = threadIdx.x; v < vecs; v += blockDim.x) {
    float x[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(update + row * u_stride + v * 8), x);
    if (residual) {
      float r[8];
      unpack8<T>(*reinterpret_cast<const uint4*>(residual + row * r_stride + v * 8), r);
#pragma unroll
      for (int i = 0; i < 8; ++i) { x[i] = r[i] + x[i]; if (round_sum) x[i] = to_f32(from_f32<T>(x[i])); }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sum += x[i] * x[i];
  }
  sum = block_sum(sum, red);
  const float inverse = 1.0f / sqrtf(sum / static_cast<float>(width) + eps);
  for (unsigned v = threadIdx.x; v < vecs; v += blockDim.x) {
    float x[8], g[8], y[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(update + row * u_stride + v * 8), x);
    if (residual) {
      float r[8];
      unpack8<T>(*reinterpret_cast<const uint4*>(residual + row * r_stride + v * 8), r);
#pragma unroll
      for (int i = 0; i < 8; ++i) { x[i] = r[i] + x[i]; if (round_sum) x[i] = to_f32(from_f32<T>(x[i])); }
      *reinterpret_cast<uint4*>(sum_out + row * s_stride + v * 8) = pack8<T>(x);
    }
    unpack8<T>(*reinterpret_cast<const uint4*>(w + v * 8), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = x[i] * inverse * g[i];
    *reinterpret_cast<uint4*>(norm_out + row * n_stride + v * 8) = pack8<T>(y);
  }
}

// mode 0: a + b; mode 1: a * sigmoid(a) * b
template <typename T>
__global__ void map2_dense_kernel(const T* a, size_t a_stride, const T* b, size_t b_stride, T* out, size_t o_stride, size_t rows, unsigned width, int mode) {
  pdl_sync();
  const unsigned vecs = width / 8;
  const size_t total = rows * vecs;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = idx / vecs, v = idx % vecs;
    float x[8], y[8], z[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(a + row * a_stride + v * 8), x);
    unpack8<T>(*reinterpret_cast<const uint4*>(b + row * b_stride + v * 8), y);
#pragma unroll
    for (int i = 0; i < 8; ++i) z[i] = mode == 0 ? x[i] + y[i] : x[i] * sigmoid_ref(x[i]) * y[i];
    *reinterpret_cast<uint4*>(out + row * o_stride + v * 8) = pack8<T>(z);
  }
}

template <typename T>
bool try_norm_dense(Ctx& ctx, const View* residual, const View& update, const View& w, const View* sum_out, const View& norm_out, size_t rows, unsigned width,
                    float eps, int round_sum) {
  const int dt = update.dtype;
  if (w.dtype != dt || norm_out.dtype != dt || (residual && (residual->dtype != dt || sum_out->dtype != dt))) return false;
  DenseRow u = dense_rows(update, rows, width, false), g = dense_rows(w, rows, width, true), n = dense_rows(norm_out, rows, width, false);
  DenseRow r{true, nullptr, 0}, s{true, nullptr, 0};
  if (residual) { r = dense_rows(*residual, rows, width, false); s = dense_rows(*sum_out, rows, width, false); }
  if (!u.ok || !g.ok || !n.ok || !r.ok || !s.ok || rows > 0x7FFFFFFFull) return false;
  launch_pdl(norm_dense_kernel<T>, dim3(static_cast<unsigned>(rows)), dim3(128), 0, ctx.stream, reinterpret_cast<const T*>(r.base), r.row_stride, reinterpret_cast<const T*>(u.base),
             u.row_stride, reinterpret_cast<const T*>(g.base), reinterpret_cast<T*>(s.base), s.row_stride, reinterpret_cast<T*>(n.base), n.row_stride, width, eps, round_sum);
  ctx.launches++;
  return true;
}

template <typename T>
bool try_map2_dense(Ctx& ctx, const View& a, const View& b, const View& out, size_t n, int mode) {
  if (a.rank < 1 || a.dtype != b.dtype || a.dtype != out.dtype) return false;
  const unsigned width = a.shape[a.rank - 1];
  if (width == 0 || n % width != 0) return false;
  const size_t rows = n / width;
  DenseRow x = dense_rows(a, rows, width, false), y = dense_rows(b, rows, width, false), o = dense_rows(out, rows, width, false);
  if (!x.ok || !y.ok || !o.ok) return false;
  const size_t total = rows * (width / 8);
  launch_pdl(map2_dense_kernel<T>, dim3(grid_for(total, kThreads, ctx.sm_count)), dim3(kThreads), 0, ctx.stream, reinterpret_cast<const T*>(x.base), x.row_stride,
             reinterpret_cast<const T*>(y.base), y.row_stride, reinterpret_cast<T*>(o.base), o.row_stride, rows, width, mode);
  ctx.launches++;
  return true;
}

}  // namespace

void launch_copy(Ctx& ctx, const View& in, const View& out, size_t n) {
  if (n == 0) return;
  copy_kernel<<<grid_for(n, kThreads, ctx.sm_count), kThreads, 0, ctx.stream>>>(in, out, n);
  ctx.launches++;
}
void launch_fill_zero(Ctx& ctx, void* ptr, size_t bytes) {
  if (bytes) cudaMemsetAsync(ptr, 0, bytes, ctx.stream);
}
void launch_add(Ctx& ctx, const View& a, const View& b, const View& out, size_t n) {
  if (n == 0) return;
  if (a.dtype == BF16 && try_map2_dense<__nv_bfloat16>(ctx, a, b, out, n, 0)) return;
  if (a.dtype == F16 && try_map2_dense<__half>(ctx, a, b, out, n, 0)) return;
  add_kernel<<<grid_for(n, kThreads, ctx.sm_count), kThreads, 0, ctx.stream>>>(a, b, out, n);
  ctx.launches++;
}
void launch_silu_mul(Ctx& ctx, const View& gate, const View& up, const View& out, size_t n) {
  if (n == 0) return;
  if (gate.dtype == BF16 && try_map2_dense<__nv_bfloat16>(ctx, gate, up, out, n, 1)) return;
  if (gate.dtype == F16 && try_map2_dense<__half>(ctx, gate, up, out, n, 1)) return;
  silu_mul_kernel<<<grid_for(n, kThreads, ctx.sm_count), kThreads, 0, ctx.stream>>>(gate, up, out, n);
  ctx.launches++;
}
void launch_rms_norm(Ctx& ctx, const View& x, const View& w, const View& out, size_t rows, unsigned width, float eps) {
  if (rows == 0) return;
  if (x.dtype == BF16 && try_norm_dense<__nv_bfloat16>(ctx, nullptr, x, w, nullptr, out, rows, width, eps, 0)) return;
  if (x.dtype == F16 && try_norm_dense<__half>(ctx, nullptr, x, w, nullptr, out, rows, width, eps, 0)) return;
  rms_norm_kernel<<<grid_for(rows * 32, kThreads, ctx.sm_count), kThreads, 0, ctx.stream>>>(x, w, out, rows, width, eps);
  ctx.launches++;
}
void launch_residual_norm(Ctx& ctx, const View& residual, const View& update, const View& w, const View& sum_out,
                          const View& norm_out, size_t rows, unsigned width, float eps, int round_sum) {
  if (rows == 0) return;
  if (residual.dtype == BF16 && try_norm_dense<__nv_bfloat16>(ctx, &residual, update, w, &sum_out, norm_out, rows, width, eps, round_sum)) return;
  if (residual.dtype == F16 && try_norm_dense<__half>(ctx, &residual, update, w, &sum_out, norm_out, rows, width, eps, round_sum)) return;
  residual_norm_kernel<<<grid_for(rows * 32, kThreads, ctx.sm_count), kThreads, 0, ctx.stream>>>(residual, update, w, sum_out, norm_out, rows, round_sum, width, eps);
  ctx.launches++;
}
void launch_qk_norm_rope(Ctx& ctx, const View& lo, const View& hi, const View& wlo, const View& whi, const View& pos,
                         const View& out_lo, const View& out_hi, size_t rows, unsigned half, float head_dim, float eps,
                         const float* inv_freq) {
  if (rows == 0) return;
  qk_norm_rope_kernel<<<grid_for(rows * 32, kThreads, ctx.sm_count), kThreads, 0, ctx.stream>>>(lo, hi, wlo, whi, pos, out_lo, out_hi, rows, half, head_dim, eps, inv_freq);
  ctx.launches++;
}
void launch_rope_pairs(Ctx& ctx, const View& first, const View& second, const View& pos, const View& out_first,
                       const View& out_second, size_t n, unsigned half, const float* inv_freq) {
  if (n == 0) return;
  rope_pairs_kernel<<<grid_for(n, kThreads, ctx.sm_count), kThreads, 0, ctx.stream>>>(first, second, pos, out_first, out_second, n, half, inv_freq);
  ctx.launches++;
}
void launch_embed(Ctx& ctx, const void* table, int t_dt, const unsigned* ids, void* out, int out_dt, unsigned vocab,
                  unsigned width, unsigned count, ErrorRecord* err) {
  if (count == 0) return;
  embed_kernel<<<min(count, 65535u), 128, 0, ctx.stream>>>(table, t_dt, ids, out, out_dt, vocab, width, count, err);
  ctx.launches++;
}
void launch_quant_embed(Ctx& ctx, const unsigned* packed, const void* scales, const void* biases, int p_dt,
                        const unsigned* ids, void* out, int out_dt, unsigned vocab, unsigned packed_width, unsigned count,
                        unsigned bits, unsigned group_size, ErrorRecord* err) {
  if (count == 0) return;
  quant_embed_kernel<<<min(count, 65535u), 128, 0, ctx.stream>>>(packed, scales, biases, p_dt, ids, out, out_dt, vocab, packed_width, count, bits, group_size, err);
  ctx.launches++;
}
size_t argmax_scratch_bytes(unsigned rows, unsigned width) {
  unsigned chunks = (width + kArgmaxChunk - 1) / kArgmaxChunk;
  return static_cast<size_t>(rows) * chunks * sizeof(unsigned long long);
}
void launch_argmax(Ctx& ctx, const void* x, int x_dt, size_t row_stride, unsigned* out, unsigned rows, unsigned width,
                   void* scratch) {
  if (rows == 0 || width == 0) return;
  unsigned chunks = (width + kArgmaxChunk - 1) / kArgmaxChunk;
  auto* partial = static_cast<unsigned long long*>(scratch);
  for (unsigned r0 = 0; r0 < rows; r0 += 65535) {  // gridDim.y limit
    unsigned nr = min(rows - r0, 65535u);
    argmax_partial_kernel<<<dim3(chunks, nr), 256, 0, ctx.stream>>>(static_cast<const char*>(x) + static_cast<size_t>(r0) * row_stride * dtype_size(x_dt), x_dt, row_stride, width, chunks, partial + static_cast<size_t>(r0) * chunks);
    ctx.launches++;
  }
  argmax_final_kernel<<<(rows + 3) / 4, 128, 0, ctx.stream>>>(partial, chunks, out, rows);
  ctx.launches++;
}
void launch_top_k(Ctx& ctx, const void* x, int x_dt, void* values, int v_dt, unsigned* indices, unsigned rows,
                  unsigned width, unsigned k, bool normalize) {
  if (rows == 0) return;
  size_t smem = static_cast<size_t>(width) * sizeof(unsigned long long);
  int threads = width >= 1024 ? 256 : (width >= 128 ? 128 : 32);
  launch_pdl(top_k_kernel, dim3(rows), dim3(threads), smem, ctx.stream, x, x_dt, values, v_dt, indices, width, k, normalize ? 1 : 0);
  ctx.launches++;
}

void launch_qknorm_rope_append(Ctx& ctx, const void* qkv, int dt, const void* q_norm_w, const void* k_norm_w,
                               const unsigned* positions, const unsigned* slot_mapping, void* q_out, void* k_plane,
                               void* v_plane, unsigned rows, unsigned q_heads, unsigned kv_heads, unsigned head_dim,
                               float eps, const float* inv_freq, int qk_norm, unsigned plane_slots) {
  if (rows == 0) return;
  size_t items = static_cast<size_t>(rows) * (q_heads + 2 * kv_heads);
  unsigned grid = grid_for(items * 32, kThreads, ctx.sm_count);
  if (dt == BF16)
    launch_pdl(qknorm_rope_append_kernel<__nv_bfloat16>, dim3(grid), dim3(kThreads), 0, ctx.stream,
        static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(q_norm_w), static_cast<const __nv_bfloat16*>(k_norm_w),
        positions, slot_mapping, static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_plane), static_cast<__nv_bfloat16*>(v_plane),
        rows, q_heads, kv_heads, head_dim, eps, inv_freq, qk_norm, plane_slots);
  else if (dt == F16)
    launch_pdl(qknorm_rope_append_kernel<__half>, dim3(grid), dim3(kThreads), 0, ctx.stream,
        static_cast<const __half*>(qkv), static_cast<const __half*>(q_norm_w), static_cast<const __half*>(k_norm_w), positions, slot_mapping,
        static_cast<__half*>(q_out), static_cast<__half*>(k_plane), static_cast<__half*>(v_plane), rows, q_heads, kv_heads, head_dim, eps,
        inv_freq, qk_norm, plane_slots);
  else
    launch_pdl(qknorm_rope_append_kernel<float>, dim3(grid), dim3(kThreads), 0, ctx.stream,
        static_cast<const float*>(qkv), static_cast<const float*>(q_norm_w), static_cast<const float*>(k_norm_w), positions, slot_mapping,
        static_cast<float*>(q_out), static_cast<float*>(k_plane), static_cast<float*>(v_plane), rows, q_heads, kv_heads, head_dim, eps,
        inv_freq, qk_norm, plane_slots);
  ctx.launches++;
}

}  // namespace fj
