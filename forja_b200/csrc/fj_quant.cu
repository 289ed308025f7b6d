// MLX-style affine group-quantised projections (reference: Op::QuantMatmul and
// Op::GatherQuantMatmul, crates/forja-cpu/src/lib.rs:914-1204 with affine_quant_dot :1277-1310):
//   y[m,n] = sum_k x[m,k] * (scale[n,k/g] * q[n,k] + bias[n,k/g]),  q = (word >> bits*(k % vpw)) & mask,
// packed u32 [N, K*bits/32] with the lowest nibble first, scales/biases [N, K/g] in f16 or bf16.
//
// The decode kernels here are HBM-bound on the weight stream: 0.5625 bytes per weight for q4 with
// group 64 (4 bits + two 16-bit parameters per 64 weights). One warp owns one output column; each
// lane streams 16-byte packed words and uses the algebraic split of the reference Metal kernels,
//   sum_k x (s q + b) = s * sum_k x q + b * sum_k x   per group,
// so the inner loop is one multiply-add per weight plus one running sum of x.
#include "fj_kernels.h"

namespace fj {

namespace {

constexpr int QM = 8;  // activation rows handled per pass

__device__ inline void load_x_generic(const void* x, int dt, size_t index, int count, float* out) {
  if (dt == F32) {
    const float* p = static_cast<const float*>(x) + index;
#pragma unroll 4
    for (int i = 0; i < count; i += 4) {
      float4 v = *reinterpret_cast<const float4*>(p + i);
      out[i] = v.x; out[i + 1] = v.y; out[i + 2] = v.z; out[i + 3] = v.w;
    }
  } else {
    const unsigned short* p = static_cast<const unsigned short*>(x) + index;
#pragma unroll 2
    for (int i = 0; i < count; i += 8) {
      uint4 v = *reinterpret_cast<const uint4*>(p + i);
      const unsigned short* h = reinterpret_cast<const unsigned short*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        out[i + j] = dt == BF16 ? __bfloat162float(__ushort_as_bfloat16(h[j])) : __half2float(__ushort_as_half(h[j]));
    }
  }
}

// Accumulates one lane's slice (VPL consecutive k of one column) for up to QM rows.
template <int BITS>
__device__ inline void quant_slice(const uint4 words, float scale, float bias, const void* x, int x_dt, size_t x_index,
                                   size_t x_row_stride, unsigned rows, float* acc) {
  constexpr int VPL = 128 / BITS;       // values per 16-byte load
  constexpr int VPW = 32 / BITS;
  constexpr unsigned MASK = (1u << BITS) - 1;
  const unsigned w[4] = {words.x, words.y, words.z, words.w};
  float q[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) q[i] = static_cast<float>((w[i / VPW] >> ((i % VPW) * BITS)) & MASK);
#pragma unroll
  for (int r = 0; r < QM; ++r) {
    if (r < static_cast<int>(rows)) {
      float xv[VPL];
      load_x_generic(x, x_dt, x_index + static_cast<size_t>(r) * x_row_stride, VPL, xv);
      float dot = 0.0f, sum = 0.0f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) { dot += xv[i] * q[i]; sum += xv[i]; }
      acc[r] += scale * dot + bias * sum;
    }
  }
}

// Scalar tail / unaligned path: exact reference form, element by element.
__device__ inline float quant_dot_scalar(const void* x, int x_dt, size_t x_index, unsigned k_begin, unsigned k_end,
                                         const unsigned* packed_row, const void* scales, const void* biases, int p_dt,
                                         size_t group_row, unsigned bits, unsigned group_size, int lane) {
  const unsigned vpw = 32 / bits, mask = (1u << bits) - 1;
  float sum = 0.0f;
  for (unsigned k = k_begin + lane; k < k_end; k += 32) {
    unsigned q = (packed_row[k / vpw] >> ((k % vpw) * bits)) & mask;
    size_t g = group_row + k / group_size;
    sum += load_as_f32(x, x_dt, x_index + k) * (load_as_f32(scales, p_dt, g) * static_cast<float>(q) + load_as_f32(biases, p_dt, g));
  }
  return sum;
}

struct QuantArgs {
  const void* x; int x_dt; size_t x_row_stride;
  const unsigned* packed; const void* scales; const void* biases; int p_dt;
  unsigned k, n, bits, group_size;
};

// Computes acc[r] (r < rows) = column `col` of the projection for rows starting at x_index.
template <int BITS>
__device__ inline void quant_column(const QuantArgs& a, size_t x_index, unsigned rows, size_t expert_packed_base,
                                    size_t expert_group_base, unsigned col, int lane, float* acc) {
  constexpr int VPL = 128 / BITS;
  const unsigned packed_width = a.k * BITS / 32, groups = a.k / a.group_size;
  const unsigned* prow = a.packed + expert_packed_base + static_cast<size_t>(col) * packed_width;
  const size_t grow = expert_group_base + static_cast<size_t>(col) * groups;
  const bool x_vec = a.x_dt == F32 ? (a.x_row_stride % 4 == 0 && reinterpret_cast<size_t>(a.x) % 16 == 0 && x_index % 4 == 0)
                                   : (a.x_row_stride % 8 == 0 && reinterpret_cast<size_t>(a.x) % 16 == 0 && x_index % 8 == 0);
  const bool vec_ok = x_vec && (reinterpret_cast<size_t>(prow) % 16 == 0) && (a.group_size % VPL == 0);
  unsigned k_vec = vec_ok ? (a.k / VPL) * VPL : 0;
  for (unsigned k0 = lane * VPL; k0 < k_vec; k0 += 32 * VPL) {
    uint4 words = __ldg(reinterpret_cast<const uint4*>(prow + k0 * BITS / 32));
    const size_t g = grow + k0 / a.group_size;
    float scale = load_as_f32(a.scales, a.p_dt, g), bias = load_as_f32(a.biases, a.p_dt, g);
    quant_slice<BITS>(words, scale, bias, a.x, a.x_dt, x_index + k0, a.x_row_stride, rows, acc);
  }
  if (k_vec < a.k) {
#pragma unroll
    for (int r = 0; r < QM; ++r)
      if (r < static_cast<int>(rows))
        acc[r] += quant_dot_scalar(a.x, a.x_dt, x_index + static_cast<size_t>(r) * a.x_row_stride, k_vec, a.k, prow, a.scales, a.biases, a.p_dt, grow, BITS, a.group_size, lane);
  }
#pragma unroll
  for (int r = 0; r < QM; ++r) acc[r] = warp_sum(acc[r]);
}

template <int BITS>
__global__ void __launch_bounds__(256) quant_matmul_kernel(QuantArgs a, void* out, int out_dt, unsigned m) {
  const int lane = threadIdx.x & 31;
  const unsigned col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= a.n) return;
  for (unsigned r0 = blockIdx.y * QM; r0 < m; r0 += gridDim.y * QM) {
    float acc[QM];
#pragma unroll
    for (int r = 0; r < QM; ++r) acc[r] = 0.0f;
    const unsigned rows = min(static_cast<unsigned>(QM), m - r0);
    quant_column<BITS>(a, static_cast<size_t>(r0) * a.x_row_stride, rows, 0, 0, col, lane, acc);
    if (lane == 0)
      for (unsigned r = 0; r < rows; ++r) store_from_f32(out, out_dt, static_cast<size_t>(r0 + r) * a.n + col, acc[r]);
  }
}

__device__ inline float sigmoid_ref(float v) { return 1.0f / (1.0f + expf(-v)); }

// Gathered projection: grid.y = rows * routes; each route uses the expert named by indices.
template <int BITS>
__global__ void __launch_bounds__(256) gather_quant_kernel(QuantArgs a, QuantArgs b, int paired, const unsigned* __restrict__ indices,
                                                           void* out, int out_dt, unsigned routes, size_t total_routes, unsigned experts,
                                                           int epilogue, ErrorRecord* err) {
  const int lane = threadIdx.x & 31;
  const unsigned col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= a.n) return;
  for (size_t route = blockIdx.y; route < total_routes; route += gridDim.y) {
  const size_t row = route / routes;
  const unsigned expert = indices[route];
  const size_t out_index = route * a.n + col;
  if (expert >= experts) {  // zero row + lowest bad index (lib.rs:1078-1088)
    if (lane == 0) { store_from_f32(out, out_dt, out_index, 0.0f); if (col == 0) report_error(err, ERR_INDEX, expert); }
    continue;
  }
  const size_t packed_base = static_cast<size_t>(expert) * a.n * (a.k * BITS / 32);
  const size_t group_base = static_cast<size_t>(expert) * a.n * (a.k / a.group_size);
  float acc[QM];
#pragma unroll
  for (int r = 0; r < QM; ++r) acc[r] = 0.0f;
  quant_column<BITS>(a, row * a.x_row_stride, 1, packed_base, group_base, col, lane, acc);
  float value = acc[0];
  if (paired) {
    float acc2[QM];
#pragma unroll
    for (int r = 0; r < QM; ++r) acc2[r] = 0.0f;
    quant_column<BITS>(b, row * b.x_row_stride, 1, packed_base, group_base, col, lane, acc2);
    // only the gate*sigmoid(gate)*up epilogue is defined for the pair form
    value = epilogue == 1 ? value * sigmoid_ref(value) * acc2[0] : value;
  }
  if (lane == 0) store_from_f32(out, out_dt, out_index, value);
  }
}

// Weighted sum over routes: out[row, col] = (epilogue 2: extra[row, col] +) sum_j w[row,j] * (act[row,j,:] . W[idx[row,j]][col]).
// Routes are accumulated in ascending j like the reference (lib.rs:1153-1199).
template <int BITS>
__global__ void __launch_bounds__(256) gather_weighted_kernel(QuantArgs a, const unsigned* __restrict__ indices, const void* weights,
                                                              int w_dt, const void* extra, int e_dt, void* out, int out_dt,
                                                              unsigned rows, unsigned routes, unsigned experts, int epilogue, ErrorRecord* err) {
  const int lane = threadIdx.x & 31;
  const unsigned col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= a.n) return;
  for (unsigned row = blockIdx.y; row < rows; row += gridDim.y) {
  float total = 0.0f;
  for (unsigned j = 0; j < routes; ++j) {
    const size_t route = static_cast<size_t>(row) * routes + j;
    const unsigned expert = indices[route];
    if (expert >= experts) {
      if (lane == 0 && col == 0) report_error(err, ERR_INDEX, expert);
      continue;
    }
    const size_t packed_base = static_cast<size_t>(expert) * a.n * (a.k * BITS / 32);
    const size_t group_base = static_cast<size_t>(expert) * a.n * (a.k / a.group_size);
    float acc[QM];
#pragma unroll
    for (int r = 0; r < QM; ++r) acc[r] = 0.0f;
    quant_column<BITS>(a, route * a.x_row_stride, 1, packed_base, group_base, col, lane, acc);
    total += load_as_f32(weights, w_dt, route) * acc[0];
  }
  if (lane == 0) {
    const size_t o = static_cast<size_t>(row) * a.n + col;
    if (epilogue == 2) total = total + load_as_f32(extra, e_dt, o);
    store_from_f32(out, out_dt, o, total);
  }
  }
}

}  // namespace

void launch_quant_matmul(Ctx& ctx, const void* x, int x_dt, const unsigned* packed, const void* scales, const void* biases,
                         int p_dt, void* out, int out_dt, unsigned m, unsigned k, unsigned n, unsigned bits,
                         unsigned group_size) {
  if (m == 0 || n == 0) return;
  QuantArgs a{x, x_dt, k, packed, scales, biases, p_dt, k, n, bits, group_size};
  unsigned row_groups = (m + QM - 1) / QM;
  dim3 grid((n + 7) / 8, min(row_groups, 65535u));
  if (bits == 4) quant_matmul_kernel<4><<<grid, 256, 0, ctx.stream>>>(a, out, out_dt, m);
  else quant_matmul_kernel<8><<<grid, 256, 0, ctx.stream>>>(a, out, out_dt, m);
  ctx.launches++;
}

void launch_gather_quant_matmul(Ctx& ctx, const void* x, int x_dt, const unsigned* packed, const void* scales,
                                const void* biases, int p_dt, const unsigned* packed2, const void* scales2,
                                const void* biases2, const unsigned* indices, void* out, int out_dt, unsigned rows,
                                unsigned k, unsigned experts, unsigned n, unsigned routes, unsigned bits, unsigned group_size,
                                int epilogue, ErrorRecord* err) {
  if (rows == 0 || routes == 0 || n == 0) return;
  QuantArgs a{x, x_dt, k, packed, scales, biases, p_dt, k, n, bits, group_size};
  QuantArgs b{x, x_dt, k, packed2, scales2, biases2, p_dt, k, n, bits, group_size};
  const int paired = packed2 != nullptr;
  const size_t total_routes = static_cast<size_t>(rows) * routes;
  dim3 grid((n + 7) / 8, static_cast<unsigned>(total_routes < 65535 ? total_routes : 65535));
  if (bits == 4) gather_quant_kernel<4><<<grid, 256, 0, ctx.stream>>>(a, b, paired, indices, out, out_dt, routes, total_routes, experts, epilogue, err);
  else gather_quant_kernel<8><<<grid, 256, 0, ctx.stream>>>(a, b, paired, indices, out, out_dt, routes, total_routes, experts, epilogue, err);
  ctx.launches++;
}

void launch_gather_quant_weighted_sum(Ctx& ctx, const void* act, int a_dt, const unsigned* packed, const void* scales,
                                      const void* biases, int p_dt, const unsigned* indices, const void* weights, int w_dt,
                                      const void* extra, int e_dt, void* out, int out_dt, unsigned rows, unsigned routes,
                                      unsigned k, unsigned experts, unsigned n, unsigned bits, unsigned group_size,
                                      int epilogue, ErrorRecord* err) {
  if (rows == 0 || n == 0) return;
  QuantArgs a{act, a_dt, k, packed, scales, biases, p_dt, k, n, bits, group_size};
  dim3 grid((n + 7) / 8, min(rows, 65535u));
  if (bits == 4) gather_weighted_kernel<4><<<grid, 256, 0, ctx.stream>>>(a, indices, weights, w_dt, extra, e_dt, out, out_dt, rows, routes, experts, epilogue, err);
  else gather_weighted_kernel<8><<<grid, 256, 0, ctx.stream>>>(a, indices, weights, w_dt, extra, e_dt, out, out_dt, rows, routes, experts, epilogue, err);
  ctx.launches++;
}

}  // namespace fj
