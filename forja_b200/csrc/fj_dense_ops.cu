// Operators next to the paged path that unchanged engines also record: attention over a contiguous
// (unpaged) cache and the dense-expert gathered matmul.
//
//   Op::Sdpa         crates/forja-core/src/ops.rs:270, CPU crates/forja-cpu/src/lib.rs:1206-1273
//   Op::GatherMatmul crates/forja-core/src/ops.rs:254, CPU crates/forja-cpu/src/lib.rs:850-912
//
// Both take arbitrary strided views and any float dtype, compute in f32 and round once on store.
#include "fj_kernels.h"

namespace fj {
namespace {

constexpr int kSdpaThreads = 256;
constexpr int kSdpaTile = 256;

struct SdpaParams {
  View q, k, v, out;  // q [hq, T, d], k [kvh, L, d], v [kvh, L, dv], out [hq, T, dv]
  unsigned q_heads, kv_heads, q_len, kv_len, head_dim, value_dim, q_start;
  int causal;
  float scale;
};

// One CTA per (head, query row). Keys are walked in tiles of 256: scores (q . k) * scale with the sum over the
// head dimension in index order, running maximum and denominator rescaled per tile, output column `tid`
// accumulated in key order. Rows that attend to nothing (kv_len 0) produce zeros.
__global__ void __launch_bounds__(kSdpaThreads) sdpa_kernel(SdpaParams p) {
  __shared__ float q_s[256];
  __shared__ float scores[kSdpaTile];
  __shared__ float red[32];
  const unsigned qrow = blockIdx.x % p.q_len, head = blockIdx.x / p.q_len;
  const unsigned tid = threadIdx.x;
  const unsigned kv_head = head / (p.q_heads / p.kv_heads);
  unsigned long long limit = p.causal ? static_cast<unsigned long long>(p.q_start) + qrow + 1 : p.kv_len;
  const unsigned attended = static_cast<unsigned>(limit < p.kv_len ? limit : p.kv_len);
  const size_t q_off = head * p.q.strides[0] + qrow * p.q.strides[1];
  for (unsigned c = tid; c < p.head_dim; c += kSdpaThreads) q_s[c] = load_as_f32(p.q.base, p.q.dtype, q_off + c * p.q.strides[2]);
  __syncthreads();
  float m = -INFINITY, l = 0.0f, acc = 0.0f;
  for (unsigned tile = 0; tile < attended; tile += kSdpaTile) {
    const unsigned n = min(static_cast<unsigned>(kSdpaTile), attended - tile);
    float local_max = -INFINITY;
    for (unsigned i = tid; i < n; i += kSdpaThreads) {
      const size_t base = kv_head * p.k.strides[0] + static_cast<size_t>(tile + i) * p.k.strides[1];
      float dot = 0.0f;
      for (unsigned c = 0; c < p.head_dim; ++c) dot += q_s[c] * load_as_f32(p.k.base, p.k.dtype, base + c * p.k.strides[2]);
      const float sc = dot * p.scale;
      scores[i] = sc;
      local_max = fmaxf(local_max, sc);
    }
    local_max = warp_max(local_max);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = local_max;
    __syncthreads();
    float tile_max = -INFINITY;
    for (int w = 0; w < kSdpaThreads / 32; ++w) tile_max = fmaxf(tile_max, red[w]);
    const float m_new = fmaxf(m, tile_max);
    const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
    const float alpha = m == -INFINITY ? 0.0f : expf(m - m_safe);
    float local_sum = 0.0f;
    for (unsigned i = tid; i < n; i += kSdpaThreads) {
      const float pr = expf(scores[i] - m_safe);
      scores[i] = pr;
      local_sum += pr;
    }
    const float tile_sum = block_sum(local_sum, red);  // its barriers also publish scores[]
    l = l * alpha + tile_sum;
    m = m_new;
    if (tid < p.value_dim) {
      acc *= alpha;
      const size_t base = kv_head * p.v.strides[0] + static_cast<size_t>(tile) * p.v.strides[1] + tid * p.v.strides[2];
      for (unsigned i = 0; i < n; ++i) acc += scores[i] * load_as_f32(p.v.base, p.v.dtype, base + i * p.v.strides[1]);
    }
    __syncthreads();
  }
  if (tid < p.value_dim)
    store_from_f32(p.out.base, p.out.dtype, head * p.out.strides[0] + qrow * p.out.strides[1] + tid * p.out.strides[2], l > 0.0f ? acc / l : 0.0f);
}

struct GatherMatmulParams {
  View x, w, idx, out;  // x [rows, inner], w [experts, inner, cols], idx [rows, routes], out [rows, routes, cols]
  unsigned rows, inner, experts, cols, routes;
  ErrorRecord* err;
};

// One CTA per route (row, j); thread c owns output column c (columns are the fastest axis of the stored expert,
// so a warp reads 32 neighbouring weights per k). The sum over `inner` runs in index order with a separate
// multiply and add, which reproduces the reference's sequential f32 fold bit for bit.
__global__ void __launch_bounds__(256) gather_matmul_kernel(GatherMatmulParams p) {
  extern __shared__ float x_s[];
  const unsigned route = blockIdx.x;
  const unsigned row = route / p.routes, j = route % p.routes;
  const unsigned expert = static_cast<const unsigned*>(p.idx.base)[row * p.idx.strides[0] + j * p.idx.strides[1]];
  const size_t out_base = row * p.out.strides[0] + j * p.out.strides[1];
  if (expert >= p.experts) {
    if (threadIdx.x == 0) report_error(p.err, ERR_INDEX, expert);
    for (unsigned c = threadIdx.x; c < p.cols; c += blockDim.x) store_from_f32(p.out.base, p.out.dtype, out_base + c * p.out.strides[2], 0.0f);
    return;
  }
  for (unsigned i = threadIdx.x; i < p.inner; i += blockDim.x) x_s[i] = load_as_f32(p.x.base, p.x.dtype, row * p.x.strides[0] + i * p.x.strides[1]);
  __syncthreads();
  const size_t w_base = expert * p.w.strides[0];
  for (unsigned c = threadIdx.x; c < p.cols; c += blockDim.x) {
    float sum = 0.0f;
    const size_t col = w_base + c * p.w.strides[2];
    for (unsigned i = 0; i < p.inner; ++i) sum = __fadd_rn(sum, __fmul_rn(x_s[i], load_as_f32(p.w.base, p.w.dtype, col + i * p.w.strides[1])));
    store_from_f32(p.out.base, p.out.dtype, out_base + c * p.out.strides[2], sum);
  }
}

}  // namespace

bool launch_sdpa(Ctx& ctx, const View& q, const View& k, const View& v, const View& out, float scale, bool causal, unsigned q_start) {
  SdpaParams p;
  p.q = q; p.k = k; p.v = v; p.out = out;
  p.q_heads = q.shape[0]; p.q_len = q.shape[1]; p.head_dim = q.shape[2];
  p.kv_heads = k.shape[0]; p.kv_len = k.shape[1]; p.value_dim = v.shape[2];
  p.q_start = q_start; p.causal = causal ? 1 : 0; p.scale = scale;
  if (p.head_dim > 256 || p.value_dim > kSdpaThreads || p.kv_heads == 0 || p.q_heads % p.kv_heads != 0) return false;
  const unsigned long long blocks = static_cast<unsigned long long>(p.q_heads) * p.q_len;
  if (blocks == 0 || p.value_dim == 0) return true;
  if (blocks > 0x7FFFFFFFull) return false;
  sdpa_kernel<<<static_cast<unsigned>(blocks), kSdpaThreads, 0, ctx.stream>>>(p);
  ctx.launches++;
  return true;
}

bool launch_gather_matmul(Ctx& ctx, const View& x, const View& w, const View& idx, const View& out, ErrorRecord* err) {
  GatherMatmulParams p;
  p.x = x; p.w = w; p.idx = idx; p.out = out;
  p.rows = x.shape[0]; p.inner = x.shape[1]; p.experts = w.shape[0]; p.cols = w.shape[2]; p.routes = idx.shape[1];
  p.err = err;
  const unsigned long long blocks = static_cast<unsigned long long>(p.rows) * p.routes;
  if (blocks == 0 || p.cols == 0) return true;
  const size_t smem = static_cast<size_t>(p.inner) * sizeof(float);
  if (blocks > 0x7FFFFFFFull || smem > 48 * 1024) return false;
  gather_matmul_kernel<<<static_cast<unsigned>(blocks), 256, smem, ctx.stream>>>(p);
  ctx.launches++;
  return true;
}

}  // namespace fj
