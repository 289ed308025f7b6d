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
#include "fj_q4_i8.cuh"

#include <algorithm>

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
  pdl_sync();
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

// ---------------------------------------------------------------------------------------------
// q4 decode projection on tensor cores (M <= 16 rows, 16-bit activations, group 64 or 128)
// ---------------------------------------------------------------------------------------------
// At HBM speed a B200 delivers ~13 T nibbles/s, more than its FP32 lanes can unpack and multiply
// one by one, so the weights go through mma.sync m16n8k16 with the roles swapped: the 16 rows of
// the A operand are 16 output columns of W, the 8 columns of the B operand are up to 8 activation
// rows. Nibbles become exact bf16/f16 values by OR-ing them into the mantissa of 128.0 / 1024.0
// (value = offset + q); the mma accumulates sum_k x (offset + q) in f32 per 64-k group and the
// affine part is applied per group afterwards:
//   y += s * acc + (b - offset * s) * sum_k x.
// Inside a group the k order seen by the mma is permuted (lane t of a quad owns 16 consecutive k,
// and a register pairs k = i with k = i + 4 so that one mask extracts two nibbles), which is
// harmless because both operands use the same permutation. The per-group sum of x comes from a
// second mma against an all-ones A operand. One warp owns 16 columns over
// a slice of K; the 4 warps of a CTA split K and combine through shared memory. Per 64-k block a
// lane issues two 8-byte weight loads, 4 mma per 8 activation rows and ~1 integer op per nibble.

template <bool kBF16>
__device__ inline void mma_q4(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  if (kBF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

struct Q4MmaArgs {
  const unsigned short* x; size_t x_row_stride;   // activations, 16-bit
  const unsigned* packed; const unsigned short* scales; const unsigned short* biases;  // one matrix [n, k/8], [n, k/group]
  void* out; int out_dt; size_t out_row_stride;
  unsigned m, k, n, group_size;
};

constexpr int Q4_UNROLL = 4;  // 64-k blocks whose weight loads are in flight together per lane

// NB = number of 8-row activation tiles (1: m <= 8, 2: m <= 16); WARPS split K inside the CTA.
// A B200 needs ~5 MB in flight to cover DRAM latency at full bandwidth, about the size of one
// decode projection, so every lane issues the loads of all its blocks (up to Q4_UNROLL at a
// time, 16 bytes of weights each) before it touches the first one.
template <bool kBF16, int NB, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 768 / (WARPS * 32)) q4_mma_gemv_kernel(Q4MmaArgs a) {
  pdl_sync();
  __shared__ float partial[WARPS][16][8 * NB];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned g = lane >> 2, t = lane & 3;
  const unsigned col0 = blockIdx.x * 16;
  const unsigned blocks = a.k / 64, per_warp = (blocks + WARPS - 1) / WARPS;
  const unsigned b_begin = min(blocks, warp * per_warp), b_end = min(blocks, b_begin + per_warp);
  const unsigned words_per_row = a.k / 8, groups_per_row = a.k / a.group_size;
  const unsigned group_shift = a.group_size == 64 ? 0 : 1;  // blocks per group: 1 or 2
  const float offset = kBF16 ? 128.0f : 1024.0f;
  // this lane's two weight columns (rows g and g + 8 of the A operand); out-of-range columns read column 0 and are dropped at the end
  const unsigned ca = col0 + g < a.n ? col0 + g : 0, cb = col0 + g + 8 < a.n ? col0 + g + 8 : 0;
  const unsigned* wa = a.packed + static_cast<size_t>(ca) * words_per_row + 2 * t;
  const unsigned* wb = a.packed + static_cast<size_t>(cb) * words_per_row + 2 * t;
  const unsigned short* sa = a.scales + static_cast<size_t>(ca) * groups_per_row;
  const unsigned short* sb = a.scales + static_cast<size_t>(cb) * groups_per_row;
  const unsigned short* ba = a.biases + static_cast<size_t>(ca) * groups_per_row;
  const unsigned short* bb = a.biases + static_cast<size_t>(cb) * groups_per_row;
  // activation rows supplied by this lane to the B operand: row g of each 8-row tile
  const unsigned short* xr[NB];
  bool xok[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) { xok[nb] = g + 8 * nb < a.m; xr[nb] = a.x + static_cast<size_t>(xok[nb] ? g + 8 * nb : 0) * a.x_row_stride + 16 * t; }

  float y[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) y[nb][0] = y[nb][1] = y[nb][2] = y[nb][3] = 0.0f;

  auto to_f = [](unsigned short h) { return kBF16 ? __bfloat162float(__ushort_as_bfloat16(h)) : __half2float(__ushort_as_half(h)); };

  // scale/bias pairs of 4 consecutive groups come in one 8-byte load when the warp's block range is 4-aligned
  const bool vec_params = group_shift == 0 && per_warp % 4 == 0 && groups_per_row % 4 == 0 && Q4_UNROLL == 4;
  const unsigned ones = kBF16 ? 0x3F803F80u : 0x3C003C00u, magic = kBF16 ? 0x43004300u : 0x64006400u;

  for (unsigned blk0 = b_begin; blk0 < b_end; blk0 += Q4_UNROLL) {
    uint2 qa[Q4_UNROLL], qb[Q4_UNROLL];
    unsigned short hs_a[Q4_UNROLL], hs_b[Q4_UNROLL], hb_a[Q4_UNROLL], hb_b[Q4_UNROLL];
#pragma unroll
    for (int u = 0; u < Q4_UNROLL; ++u) {
      const unsigned blk = min(blk0 + u, b_end - 1);  // the tail re-reads the last block and is skipped below
      qa[u] = __ldg(reinterpret_cast<const uint2*>(wa + blk * 8));
      qb[u] = __ldg(reinterpret_cast<const uint2*>(wb + blk * 8));
    }
    if (vec_params) {
      const uint2 v0 = __ldg(reinterpret_cast<const uint2*>(sa + blk0)), v1 = __ldg(reinterpret_cast<const uint2*>(sb + blk0));
      const uint2 v2 = __ldg(reinterpret_cast<const uint2*>(ba + blk0)), v3 = __ldg(reinterpret_cast<const uint2*>(bb + blk0));
      hs_a[0] = v0.x & 0xFFFFu; hs_a[1] = v0.x >> 16; hs_a[2] = v0.y & 0xFFFFu; hs_a[3] = v0.y >> 16;
      hs_b[0] = v1.x & 0xFFFFu; hs_b[1] = v1.x >> 16; hs_b[2] = v1.y & 0xFFFFu; hs_b[3] = v1.y >> 16;
      hb_a[0] = v2.x & 0xFFFFu; hb_a[1] = v2.x >> 16; hb_a[2] = v2.y & 0xFFFFu; hb_a[3] = v2.y >> 16;
      hb_b[0] = v3.x & 0xFFFFu; hb_b[1] = v3.x >> 16; hb_b[2] = v3.y & 0xFFFFu; hb_b[3] = v3.y >> 16;
    } else {
#pragma unroll
      for (int u = 0; u < Q4_UNROLL; ++u) {
        const unsigned grp = min(blk0 + u, b_end - 1) >> group_shift;
        hs_a[u] = __ldg(sa + grp); hs_b[u] = __ldg(sb + grp);
        hb_a[u] = __ldg(ba + grp); hb_b[u] = __ldg(bb + grp);
      }
    }
#pragma unroll
    for (int u = 0; u < Q4_UNROLL; ++u) {
      const unsigned blk = blk0 + u;
      if (blk >= b_end) break;  // uniform across the warp
      const float s_a = to_f(hs_a[u]), s_b = to_f(hs_b[u]);
      const float o_a = to_f(hb_a[u]) - offset * s_a, o_b = to_f(hb_b[u]) - offset * s_b;
      // A fragments: one mask per register yields nibbles i and i + 4 of a word as {offset + q_i, offset + q_(i+4)},
      // so a register pairs k = i with k = i + 4; the activations below are paired the same way.
      unsigned fa[2][4], fb[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        fa[0][i] = ((qa[u].x >> (4 * i)) & 0x000F000Fu) | magic; fa[1][i] = ((qa[u].y >> (4 * i)) & 0x000F000Fu) | magic;
        fb[0][i] = ((qb[u].x >> (4 * i)) & 0x000F000Fu) | magic; fb[1][i] = ((qb[u].y >> (4 * i)) & 0x000F000Fu) | magic;
      }
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        // 16 activations of row g for this lane's k slice: 32 bytes, re-paired as (x_i, x_(i+4)) per 8
        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
        if (xok[nb]) {
          x0 = *reinterpret_cast<const uint4*>(xr[nb] + blk * 64);
          x1 = *reinterpret_cast<const uint4*>(xr[nb] + blk * 64 + 8);
        }
        const unsigned p0 = __byte_perm(x0.x, x0.z, 0x5410), p1 = __byte_perm(x0.x, x0.z, 0x7632);
        const unsigned p2 = __byte_perm(x0.y, x0.w, 0x5410), p3 = __byte_perm(x0.y, x0.w, 0x7632);
        const unsigned p4 = __byte_perm(x1.x, x1.z, 0x5410), p5 = __byte_perm(x1.x, x1.z, 0x7632);
        const unsigned p6 = __byte_perm(x1.y, x1.w, 0x5410), p7 = __byte_perm(x1.y, x1.w, 0x7632);
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        mma_q4<kBF16>(acc, fa[0][0], fb[0][0], fa[0][1], fb[0][1], p0, p1);
        mma_q4<kBF16>(acc, fa[0][2], fb[0][2], fa[0][3], fb[0][3], p2, p3);
        mma_q4<kBF16>(acc, fa[1][0], fb[1][0], fa[1][1], fb[1][1], p4, p5);
        mma_q4<kBF16>(acc, fa[1][2], fb[1][2], fa[1][3], fb[1][3], p6, p7);
        // sum of the block's activations per row through the same pipe: A = all ones, so every
        // accumulator row holds sum_k x[row 2t / 2t+1][k], already in this lane's output layout
        mma_q4<kBF16>(sum, ones, ones, ones, ones, p0, p1);
        mma_q4<kBF16>(sum, ones, ones, ones, ones, p2, p3);
        mma_q4<kBF16>(sum, ones, ones, ones, ones, p4, p5);
        mma_q4<kBF16>(sum, ones, ones, ones, ones, p6, p7);
        y[nb][0] += s_a * acc[0] + o_a * sum[0];
        y[nb][1] += s_a * acc[1] + o_a * sum[1];
        y[nb][2] += s_b * acc[2] + o_b * sum[0];
        y[nb][3] += s_b * acc[3] + o_b * sum[1];
      }
    }
  }
  // combine the K slices of the warps; layout [warp][column in tile][activation row]
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    partial[warp][g][8 * nb + 2 * t] = y[nb][0];
    partial[warp][g][8 * nb + 2 * t + 1] = y[nb][1];
    partial[warp][g + 8][8 * nb + 2 * t] = y[nb][2];
    partial[warp][g + 8][8 * nb + 2 * t + 1] = y[nb][3];
  }
  __syncthreads();
  for (unsigned idx = threadIdx.x; idx < 16 * 8 * NB; idx += blockDim.x) {
    const unsigned row = idx / 16, c = idx % 16;  // consecutive threads write consecutive columns
    if (row < a.m && col0 + c < a.n) {
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += partial[w][c][row];
      store_from_f32(a.out, a.out_dt, static_cast<size_t>(row) * a.out_row_stride + col0 + c, v);
    }
  }
}

bool q4_mma_supported(int x_dt, int p_dt, unsigned m, unsigned k, unsigned bits, unsigned group_size, const void* x, size_t x_row_stride,
                      const void* packed) {
  return bits == 4 && (x_dt == BF16 || x_dt == F16) && p_dt == x_dt && m >= 1 && m <= 16 && (group_size == 64 || group_size == 128) &&
         k % 64 == 0 && k >= 64 && x_row_stride % 8 == 0 && reinterpret_cast<size_t>(x) % 16 == 0 && reinterpret_cast<size_t>(packed) % 8 == 0;
}

template <bool kBF16, int NB>
void run_q4_mma_warps(Ctx& ctx, const Q4MmaArgs& a) {
  const unsigned grid = (a.n + 15) / 16, blocks = a.k / 64;
  if (blocks >= 64) launch_pdl(q4_mma_gemv_kernel<kBF16, NB, 16>, dim3(grid), dim3(16 * 32), 0, ctx.stream, a);
  else if (blocks >= 32) launch_pdl(q4_mma_gemv_kernel<kBF16, NB, 8>, dim3(grid), dim3(8 * 32), 0, ctx.stream, a);
  else launch_pdl(q4_mma_gemv_kernel<kBF16, NB, 4>, dim3(grid), dim3(4 * 32), 0, ctx.stream, a);
  ctx.launches++;
}

void run_q4_mma(Ctx& ctx, const Q4MmaArgs& a, int x_dt) {
  const bool bf = x_dt == BF16;
  if (a.m <= 8) {
    if (bf) run_q4_mma_warps<true, 1>(ctx, a); else run_q4_mma_warps<false, 1>(ctx, a);
  } else {
    if (bf) run_q4_mma_warps<true, 2>(ctx, a); else run_q4_mma_warps<false, 2>(ctx, a);
  }
}

// ---------------------------------------------------------------------------------------------
// Streaming q4 decode projection: persistent CTAs, per-warp cp.async rings, integer tensor cores
// ---------------------------------------------------------------------------------------------
// Unpacking nibbles into 16-bit floats costs 7 integer instructions per packed word, and the
// integer pipe (16 lanes per scheduler) then caps the kernel near a third of HBM bandwidth. Here
// the nibbles stay integers: `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are already the u8 A
// operands of mma.sync m16n8k32 (3 instructions per word). The activations are turned, once per
// CTA, into block fixed point: per (row, 64-k block) a power-of-two step S = 2^(E-11) with E the
// exponent of the block's largest |x|, and x / S rounded to a 13-bit integer that is split into a
// signed high byte and an unsigned low byte. A bf16 activation has 8 significant bits, so every
// element within 2^4 of the block maximum is represented exactly and the rest to within S/2,
// i.e. 2^-12 of the block maximum. The integer dot products are exact and, with 64 terms of at
// most 15 * 4095, stay below 2^22; the low accumulator starts at 0x4B400000 so that the bit
// pattern of 256 * hi + lo read as f32 is 12582912 + sum, which makes the int -> float
// conversion a single subtraction. Per block:
//   y += (s * S) * (256 * hi + lo) + b * sum_k x        (sum_k x is taken from the original values)
// Layout and pipeline:
//  * activations (fixed-point bytes in fragment order, block sums and steps) live in shared
//    memory for the whole kernel: K * 17 bytes per 8 rows;
//  * every warp owns whole 16-column tiles (or a 1/ksplit slice of K when there are too few tiles
//    to go round) and streams them in units of 256 k = 2 KB of nibbles + 256 B of scales and
//    biases through its own ring of cp.async stages, so the steady state has no CTA barrier;
//  * a unit's rows are 128 bytes apart in memory and 160 bytes apart in shared memory, which
//    keeps the copies coalesced and the 8-byte fragment reads of 4 rows x 4 lanes conflict-free.
// Tiles [tile_base, tile_end) are dealt out in `rounds` rounds of (WARPS / ksplit) tiles per CTA, each tile
// shared by ksplit warps along K. Phase 0 gives every warp of the grid the same number of whole tiles;
// phase 1 spreads the remainder over as many warps as possible so that the tail costs a fraction of a tile.
struct Q4Phase {
  unsigned ksplit, rounds, tile_base, tile_end;
};
struct Q4WarpArgs {
  Q4MmaArgs base;
  Q4Phase phase[2];
};

// bf16 activations and parameters only (f16 callers use the mantissa-offset kernel above).
template <bool kG64, int NB, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) q4_i8_stream_kernel(Q4WarpArgs args) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  extern __shared__ __align__(128) unsigned char q4_smem[];
  const Q4MmaArgs& a = args.base;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned g = lane >> 2, t = lane & 3;
  const unsigned blocks = a.k / 64, groups_per_row = a.k / a.group_size;
  constexpr bool g64 = kG64;
  auto half_to_f = [](unsigned h) { return __uint_as_float(h << 16); };

  uint4* xq = reinterpret_cast<uint4*>(q4_smem);                                                  // [blocks][NB][2][32]
  float2* xmeta = reinterpret_cast<float2*>(q4_smem + static_cast<size_t>(blocks) * NB * 1024);    // [blocks][NB][8] {sum, step}
  unsigned char* ring = q4_smem + static_cast<size_t>(blocks) * NB * Q4W_X_BYTES + warp * (STAGES * Q4W_UNIT_BYTES);
  float* partial = reinterpret_cast<float*>(q4_smem + static_cast<size_t>(blocks) * NB * Q4W_X_BYTES + WARPS * STAGES * Q4W_UNIT_BYTES);  // [warp][16][8 NB]
  const unsigned ring_base = static_cast<unsigned>(__cvta_generic_to_shared(ring));

  bool x_ready = false;
  for (int phase_index = 0; phase_index < 2; ++phase_index) {
  const Q4Phase ph = phase_index == 0 ? args.phase[0] : args.phase[1];
  if (ph.rounds == 0) continue;  // uniform across the grid
  const unsigned ksplit = ph.ksplit, group = warp / ksplit, ks = warp % ksplit, tile_groups = WARPS / ksplit;
  const unsigned upt = (a.k / 256) / ksplit;  // units of this warp per tile
  const unsigned items = ph.rounds * upt;
  const unsigned tile_step = tile_groups * gridDim.x, tile_first = ph.tile_base + group * gridDim.x + blockIdx.x;
  const unsigned char* wbase = reinterpret_cast<const unsigned char*>(a.packed);
  const size_t row_bytes = a.k / 2;
  const unsigned copy_row = lane >> 3, copy_col = (lane & 7) * 16;
  const unsigned param_which = lane >> 4, param_col = lane & 15;
  const unsigned copy_dst = copy_row * Q4W_ROW_STRIDE + copy_col, param_dst = Q4W_PARAM_OFFSET + param_which * 128 + param_col * 8;
  const unsigned short* param_base = param_which ? a.biases : a.scales;

  // ---- producer side: the unit after the last one issued (tile, unit in tile, stage), advanced without divisions ----
  unsigned in_tile = tile_first, in_u = 0, in_stage = 0, in_count = 0;
  const unsigned char* in_rows[4];
  const unsigned short* in_param = nullptr;
  auto issue = [&]() {
    if (in_count < items && in_tile < ph.tile_end) {
      if (in_u == 0) {  // new tile: row pointers of this lane's 4 copies and of its parameter slot
#pragma unroll
        for (int i = 0; i < 4; ++i) in_rows[i] = wbase + min(in_tile * 16 + copy_row + 4 * i, a.n - 1) * row_bytes + (ks * upt) * 128 + copy_col;
        in_param = param_base + static_cast<size_t>(min(in_tile * 16 + param_col, a.n - 1)) * groups_per_row + (ks * upt) * (256 / (g64 ? 64 : 128));
      }
      const unsigned stage = ring_base + in_stage * Q4W_UNIT_BYTES;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(stage + copy_dst + i * (4 * Q4W_ROW_STRIDE)), "l"(in_rows[i] + in_u * 128) : "memory");
      if (g64) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(stage + param_dst), "l"(in_param + in_u * 4) : "memory");
      else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(stage + param_dst), "l"(in_param + in_u * 2) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    ++in_count;
    in_stage = in_stage + 1 == STAGES ? 0 : in_stage + 1;
    if (++in_u == upt) { in_u = 0; in_tile += tile_step; }
  };

  for (int q = 0; q + 1 < STAGES; ++q) issue();  // the first weight units are already on their way while the activations are converted

  // ---- activations -> block fixed point in fragment order, once per CTA ----
  // (programmatic dependent launch: the weight copies above do not depend on the previous kernel; the activations do)
  if (!x_ready) asm volatile("griddepcontrol.wait;\n" ::: "memory");
  for (unsigned b = x_ready ? blocks : warp; b < blocks; b += WARPS) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
      if (g + 8 * nb < a.m) {
        const unsigned short* xr = a.x + static_cast<size_t>(g + 8 * nb) * a.x_row_stride + b * 64 + 16 * t;
        x0 = *reinterpret_cast<const uint4*>(xr);
        x1 = *reinterpret_cast<const uint4*>(xr + 8);
      }
      const unsigned raw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
      float f[16];
      float sum = 0.0f, biggest = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f[2 * i] = half_to_f(raw[i] & 0xFFFFu);
        f[2 * i + 1] = half_to_f(raw[i] >> 16);
        sum += f[2 * i] + f[2 * i + 1];
        biggest = fmaxf(biggest, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, 1));
      biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, 2));
      // step = 2^(E - 11); blocks of zeros, subnormals, infinities or NaNs keep a harmless step of 1
      const unsigned exponent = __float_as_uint(biggest) & 0x7F800000u;
      const bool usable = exponent >= (12u << 23) && exponent < (255u << 23);
      const float step = usable ? __uint_as_float(exponent - (11u << 23)) : 1.0f;
      const float inv_step = usable ? __uint_as_float((254u << 23) - (exponent - (11u << 23))) : 1.0f;
      int fixed[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) fixed[i] = usable ? __float2int_rn(f[i] * inv_step) : 0;
      // byte order of a B register: k = 0,2,4,6 | 1,3,5,7 | 8,10,12,14 | 9,11,13,15 (matches the nibble masks)
      unsigned hi[4], lo[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int base = (r >> 1) * 8 + (r & 1);
        hi[r] = lo[r] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int v = fixed[base + 2 * j];
          hi[r] |= (static_cast<unsigned>(v >> 8) & 0xFFu) << (8 * j);
          lo[r] |= (static_cast<unsigned>(v) & 0xFFu) << (8 * j);
        }
      }
      xq[((b * NB + nb) * 2 + 0) * 32 + lane] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      xq[((b * NB + nb) * 2 + 1) * 32 + lane] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      // a block without a usable step (all zeros, or values below 2^-115) keeps only its b * sum term
      if (t == 0) xmeta[(b * NB + nb) * 8 + g] = make_float2(sum, usable ? step : 0.0f);
    }
  }
  x_ready = true;
  __syncthreads();

  constexpr int kMagic = 0x4B400000;        // bit pattern of 12582912.0f
  constexpr float kMagicF = 12582912.0f;
  float y[NB][4];
  unsigned tile = tile_first, u = 0, out_stage = 0;
  for (unsigned q = 0; q < items; ++q) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2) : "memory");
    __syncwarp();  // unit q is visible to the whole warp, and the warp is done with unit q - 1
    issue();
    const bool live = tile < ph.tile_end;
    if (u == 0) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) y[nb][0] = y[nb][1] = y[nb][2] = y[nb][3] = 0.0f;
    }
    if (live) {
      const unsigned char* stage = ring + out_stage * Q4W_UNIT_BYTES;
      // scales and biases of this lane's two columns for the unit's 4 blocks (group 128: 2 slots used)
      const uint2 sa = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + g * 8);
      const uint2 sb = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + (g + 8) * 8);
      const uint2 ba = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + 128 + g * 8);
      const uint2 bb = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + 128 + (g + 8) * 8);
      float s_a[4], s_b[4], b_a[4], b_b[4];
      {
        const unsigned w[8] = {sa.x, sa.y, sb.x, sb.y, ba.x, ba.y, bb.x, bb.y};
        float v[8][2];
#pragma unroll
        for (int i = 0; i < 8; ++i) { v[i][0] = __uint_as_float(w[i] << 16); v[i][1] = __uint_as_float(w[i] & 0xFFFF0000u); }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int slot = g64 ? j : j >> 1;
          s_a[j] = v[0 + (slot >> 1)][slot & 1]; s_b[j] = v[2 + (slot >> 1)][slot & 1];
          b_a[j] = v[4 + (slot >> 1)][slot & 1]; b_b[j] = v[6 + (slot >> 1)][slot & 1];
        }
      }
      const uint4* xq_unit = xq + static_cast<size_t>((ks * upt + u) * 4) * (NB * 2 * 32) + lane;
      const float2* meta_unit = xmeta + static_cast<size_t>((ks * upt + u) * 4) * (NB * 8) + 2 * t;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint2 qa = *reinterpret_cast<const uint2*>(stage + g * Q4W_ROW_STRIDE + j * 32 + t * 8);
        const uint2 qb = *reinterpret_cast<const uint2*>(stage + (g + 8) * Q4W_ROW_STRIDE + j * 32 + t * 8);
        const unsigned ea0 = qa.x & 0x0F0F0F0Fu, oa0 = (qa.x >> 4) & 0x0F0F0F0Fu, ea1 = qa.y & 0x0F0F0F0Fu, oa1 = (qa.y >> 4) & 0x0F0F0F0Fu;
        const unsigned eb0 = qb.x & 0x0F0F0F0Fu, ob0 = (qb.x >> 4) & 0x0F0F0F0Fu, eb1 = qb.y & 0x0F0F0F0Fu, ob1 = (qb.y >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const uint4 xh = xq_unit[((j * NB + nb) * 2 + 0) * 32];
          const uint4 xl = xq_unit[((j * NB + nb) * 2 + 1) * 32];
          const float4 meta = *reinterpret_cast<const float4*>(meta_unit + (j * NB + nb) * 8);  // rows 2t, 2t+1: {sum, step} x 2
          int hi[4] = {0, 0, 0, 0}, lo[4] = {kMagic, kMagic, kMagic, kMagic};
          mma_u8<true>(hi, ea0, eb0, oa0, ob0, xh.x, xh.y);
          mma_u8<false>(lo, ea0, eb0, oa0, ob0, xl.x, xl.y);
          mma_u8<true>(hi, ea1, eb1, oa1, ob1, xh.z, xh.w);
          mma_u8<false>(lo, ea1, eb1, oa1, ob1, xl.z, xl.w);
          // |256 * hi + lo| < 2^22, so the combined integer keeps the magic exponent
          float v[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] = __int_as_float(hi[i] * 256 + lo[i]) - kMagicF;
          y[nb][0] += (s_a[j] * meta.y) * v[0] + b_a[j] * meta.x;
          y[nb][1] += (s_a[j] * meta.w) * v[1] + b_a[j] * meta.z;
          y[nb][2] += (s_b[j] * meta.y) * v[2] + b_b[j] * meta.x;
          y[nb][3] += (s_b[j] * meta.w) * v[3] + b_b[j] * meta.z;
        }
      }
    }
    out_stage = out_stage + 1 == STAGES ? 0 : out_stage + 1;
    if (u + 1 == upt) {
      if (ksplit == 1) {
        if (live) {
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const unsigned row = 8 * nb + 2 * t + (i & 1), col = tile * 16 + g + (i >> 1) * 8;
              if (row < a.m && col < a.n) store_from_f32(a.out, a.out_dt, static_cast<size_t>(row) * a.out_row_stride + col, y[nb][i]);
            }
          }
        }
      } else {
        // the warps sharing a tile combine their K slices; every warp of the CTA reaches both barriers
        float* mine = partial + warp * (16 * 8 * NB);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          mine[g * (8 * NB) + 8 * nb + 2 * t] = y[nb][0];
          mine[g * (8 * NB) + 8 * nb + 2 * t + 1] = y[nb][1];
          mine[(g + 8) * (8 * NB) + 8 * nb + 2 * t] = y[nb][2];
          mine[(g + 8) * (8 * NB) + 8 * nb + 2 * t + 1] = y[nb][3];
        }
        __syncthreads();
        if (live) {
          const float* first = partial + (group * ksplit) * (16 * 8 * NB);
          for (unsigned idx = ks * 32 + lane; idx < 16 * 8 * NB; idx += ksplit * 32) {
            const unsigned row = idx / 16, c = idx % 16;
            if (row < a.m && tile * 16 + c < a.n) {
              float v = 0.0f;
              for (unsigned w = 0; w < ksplit; ++w) v += first[w * (16 * 8 * NB) + c * (8 * NB) + row];
              store_from_f32(a.out, a.out_dt, static_cast<size_t>(row) * a.out_row_stride + tile * 16 + c, v);
            }
          }
        }
        __syncthreads();
      }
    }
    if (++u == upt) { u = 0; tile += tile_step; }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  __syncwarp();
  }  // phase
}

template <bool kG64, int NB, int STAGES, int WARPS>
bool launch_q4_i8_stream(Ctx& ctx, const Q4WarpArgs& args, unsigned grid, size_t smem) {
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64) return false;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(q4_i8_stream_kernel<kG64, NB, STAGES, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) { cudaGetLastError(); return false; }
    configured[device] = true;
  }
  launch_pdl(q4_i8_stream_kernel<kG64, NB, STAGES, WARPS>, dim3(grid), dim3(WARPS * 32), smem, ctx.stream, args);
  ctx.launches++;
  return true;
}

// Shared-memory need of one CTA and the two-phase tile split for a given warp count; false when it cannot run.
template <int STAGES, int WARPS>
bool plan_q4_i8(const Q4MmaArgs& a, unsigned sms, unsigned nb, Q4WarpArgs* args, unsigned* grid, size_t* smem) {
  const unsigned blocks = a.k / 64, units = a.k / 256, tiles = (a.n + 15) / 16;
  *grid = std::min(tiles, sms);
  const unsigned warps_total = *grid * WARPS, whole = tiles / warps_total;
  args->phase[0] = Q4Phase{1, whole, 0, whole * warps_total};
  args->phase[1] = Q4Phase{1, 0, whole * warps_total, tiles};
  const unsigned rest = tiles - whole * warps_total;
  if (rest != 0) {
    // too few tiles left for every warp to own one: let 2, 4, ... warps share a tile along K
    const unsigned per_cta = (rest + *grid - 1) / *grid;
    unsigned tile_groups = 1;
    while (tile_groups < WARPS && tile_groups < per_cta) tile_groups *= 2;
    unsigned ksplit = WARPS / tile_groups;
    while (ksplit > 1 && units % ksplit != 0) ksplit /= 2;
    tile_groups = WARPS / ksplit;
    args->phase[1].ksplit = ksplit;
    args->phase[1].rounds = (rest + tile_groups * *grid - 1) / (tile_groups * *grid);
  }
  *smem = static_cast<size_t>(blocks) * nb * Q4W_X_BYTES + static_cast<size_t>(WARPS) * STAGES * Q4W_UNIT_BYTES +
          (args->phase[1].ksplit > 1 ? static_cast<size_t>(WARPS) * 16 * 8 * nb * sizeof(float) : 0);
  return *smem <= 227 * 1024;
}

template <bool kG64, int NB>
bool run_q4_i8_config(Ctx& ctx, const Q4MmaArgs& a, unsigned sms) {
  Q4WarpArgs args{a, {}};
  unsigned grid = 0;
  size_t smem = 0;
  if (plan_q4_i8<4, 16>(a, sms, NB, &args, &grid, &smem)) return launch_q4_i8_stream<kG64, NB, 4, 16>(ctx, args, grid, smem);
  if (plan_q4_i8<3, 16>(a, sms, NB, &args, &grid, &smem)) return launch_q4_i8_stream<kG64, NB, 3, 16>(ctx, args, grid, smem);
  if (plan_q4_i8<3, 8>(a, sms, NB, &args, &grid, &smem)) return launch_q4_i8_stream<kG64, NB, 3, 8>(ctx, args, grid, smem);
  return false;
}

// Tries the streaming kernel; false when dtype, shape or alignment rule it out (the caller falls back).
bool run_q4_stream(Ctx& ctx, const Q4MmaArgs& a, int x_dt) {
  const unsigned param_align = a.group_size == 64 ? 8 : 4;
  if (x_dt != BF16 || a.k % 256 != 0 || reinterpret_cast<size_t>(a.packed) % 16 != 0 || reinterpret_cast<size_t>(a.scales) % param_align != 0 ||
      reinterpret_cast<size_t>(a.biases) % param_align != 0) return false;
  const unsigned sms = static_cast<unsigned>(ctx.sm_count > 0 ? ctx.sm_count : 148);
  if (a.group_size == 64) return a.m <= 8 ? run_q4_i8_config<true, 1>(ctx, a, sms) : run_q4_i8_config<true, 2>(ctx, a, sms);
  return a.m <= 8 ? run_q4_i8_config<false, 1>(ctx, a, sms) : run_q4_i8_config<false, 2>(ctx, a, sms);
}

// ---- one or two rows: integer dot products from registers ---------------------------------------------------
// q4, group 64, bf16 activations, k a multiple of 1024 up to 4096. A warp owns whole weight rows (output columns): lane l
// takes the four packed words l*4 .. l*4+3 of every 1024-k slice (one 16-byte load, 32 weights, half a group), so a warp
// reads a row as contiguous 512-byte pieces. The lane's activations never leave its registers: converted once per CTA
// pass to the same block fixed point as the tensor-core form above (per 64-k block a power-of-two step, 13-bit integers
// split into a signed high and an unsigned low byte), packed in the byte order of the nibble masks (`w & 0x0F0F0F0F`
// holds k = 0,2,4,6 of a word, `(w >> 4) & 0x0F0F0F0F` k = 1,3,5,7) and multiplied with dp4a: 3 mask/shift and 4 dp4a
// instructions per packed word and row, no shared memory, no tensor-core tile that is 15/16 zero rows.
// y = sum over the lane's half groups of (s * S) * (256 * hi + lo) + b * (sum of the lane's 32 activations), then a warp sum.
// The loads of the two rows after the current one are in flight while it is reduced.
__device__ inline int dp4a_us(unsigned a, unsigned b, int c) {  // unsigned bytes of a x signed bytes of b
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ inline int dp4a_uu(unsigned a, unsigned b, int c) {  // unsigned x unsigned
  int d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <int SLICES, int ROWS>
__global__ void __launch_bounds__(256) q4_dp4a_gemv_kernel(Q4MmaArgs a) {
  const unsigned lane = threadIdx.x & 31;
  const unsigned warps_total = gridDim.x * (blockDim.x >> 5), warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const unsigned groups_per_row = a.k / 64;
  const uint4* packed = reinterpret_cast<const uint4*>(a.packed);
  const size_t row_vectors = a.k / 32;  // 16-byte vectors per weight row

  // the first row's weights are requested before the activations are touched (they do not depend on the previous kernel)
  unsigned n = warp_global;
  constexpr int SP = (SLICES + 1) / 2;  // a lane keeps the scale and bias of groups lane and lane + 32
  uint4 q[SLICES], q_next[SLICES], q_after[SLICES];  // the row being reduced and the two rows behind it, already requested
  unsigned short scale_raw[SP], bias_raw[SP], scale_next[SP], bias_next[SP], scale_after[SP], bias_after[SP];
#pragma unroll
  for (int i = 0; i < SP; ++i) scale_raw[i] = bias_raw[i] = scale_next[i] = bias_next[i] = scale_after[i] = bias_after[i] = 0;
  auto request = [&](unsigned row, uint4 (&dst)[SLICES], unsigned short (&sr)[SP], unsigned short (&br)[SP]) {
    if (row < a.n) {
#pragma unroll
      for (int it = 0; it < SLICES; ++it) dst[it] = __ldcs(packed + static_cast<size_t>(row) * row_vectors + it * 32 + lane);
#pragma unroll
      for (int i = 0; i < SP; ++i) {
        if (lane + 32 * i < groups_per_row) {
          sr[i] = __ldcs(a.scales + static_cast<size_t>(row) * groups_per_row + lane + 32 * i);
          br[i] = __ldcs(a.biases + static_cast<size_t>(row) * groups_per_row + lane + 32 * i);
        }
      }
    }
  };
  request(n, q, scale_raw, bias_raw);
  request(n + warps_total, q_next, scale_next, bias_next);
  pdl_sync();

  // activations of this lane: k = it * 1024 + lane * 32 .. + 31 for every slice
  unsigned xh[ROWS][SLICES][8], xl[ROWS][SLICES][8];  // [word][even | odd] packed bytes
  float xsum[ROWS][SLICES], xstep[ROWS][SLICES];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int it = 0; it < SLICES; ++it) {
      float f[32];
      float sum = 0.0f, biggest = 0.0f;
      if (static_cast<unsigned>(r) < a.m) {
        const uint4* src = reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(r) * a.x_row_stride + it * 1024 + lane * 32);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 raw = src[v];
          const unsigned words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            f[v * 8 + 2 * i] = __uint_as_float(words[i] << 16);
            f[v * 8 + 2 * i + 1] = __uint_as_float(words[i] & 0xFFFF0000u);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) { sum += f[i]; biggest = fmaxf(biggest, fabsf(f[i])); }
      biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, 1));  // the 64-k block spans this lane and its neighbour
      const unsigned exponent = __float_as_uint(biggest) & 0x7F800000u;
      const bool usable = exponent >= (12u << 23) && exponent < (255u << 23);
      const float inv_step = usable ? __uint_as_float((254u << 23) - (exponent - (11u << 23))) : 1.0f;
      xstep[r][it] = usable ? __uint_as_float(exponent - (11u << 23)) : 0.0f;  // a block without a usable step keeps only its bias term
      xsum[r][it] = sum;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        unsigned he = 0, ho = 0, le = 0, lo = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int even = usable ? __float2int_rn(f[w * 8 + 2 * j] * inv_step) : 0, odd = usable ? __float2int_rn(f[w * 8 + 2 * j + 1] * inv_step) : 0;
          he |= (static_cast<unsigned>(even >> 8) & 0xFFu) << (8 * j);
          le |= (static_cast<unsigned>(even) & 0xFFu) << (8 * j);
          ho |= (static_cast<unsigned>(odd >> 8) & 0xFFu) << (8 * j);
          lo |= (static_cast<unsigned>(odd) & 0xFFu) << (8 * j);
        }
        xh[r][it][2 * w] = he; xh[r][it][2 * w + 1] = ho;
        xl[r][it][2 * w] = le; xl[r][it][2 * w + 1] = lo;
      }
    }
  }

  for (; n < a.n; n += warps_total) {
    request(n + 2 * warps_total, q_after, scale_after, bias_after);
    float y[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) y[r] = 0.0f;
#pragma unroll
    for (int it = 0; it < SLICES; ++it) {
      // scale and bias of this lane's group g = it * 16 + lane / 2 sit in lane g % 32, slot g / 32
      const unsigned holder = (it * 16 + (lane >> 1)) & 31u;
      const float s = __uint_as_float(__shfl_sync(0xffffffffu, static_cast<unsigned>(scale_raw[it / 2]), holder) << 16);
      const float b = __uint_as_float(__shfl_sync(0xffffffffu, static_cast<unsigned>(bias_raw[it / 2]), holder) << 16);
      const unsigned words[4] = {q[it].x, q[it].y, q[it].z, q[it].w};
      int hi[ROWS], lo[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) { hi[r] = 0; lo[r] = 0; }
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const unsigned even = words[w] & 0x0F0F0F0Fu, odd = (words[w] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          hi[r] = dp4a_us(even, xh[r][it][2 * w], hi[r]);
          hi[r] = dp4a_us(odd, xh[r][it][2 * w + 1], hi[r]);
          lo[r] = dp4a_uu(even, xl[r][it][2 * w], lo[r]);
          lo[r] = dp4a_uu(odd, xl[r][it][2 * w + 1], lo[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) y[r] += (s * xstep[r][it]) * static_cast<float>(hi[r] * 256 + lo[r]) + b * xsum[r][it];
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float total = warp_sum(y[r]);
      if (lane == 0 && static_cast<unsigned>(r) < a.m) store_from_f32(a.out, a.out_dt, static_cast<size_t>(r) * a.out_row_stride + n, total);
    }
#pragma unroll
    for (int it = 0; it < SLICES; ++it) { q[it] = q_next[it]; q_next[it] = q_after[it]; }
#pragma unroll
    for (int i = 0; i < SP; ++i) { scale_raw[i] = scale_next[i]; bias_raw[i] = bias_next[i]; scale_next[i] = scale_after[i]; bias_next[i] = bias_after[i]; }
  }
}

template <int SLICES, int ROWS>
void launch_q4_dp4a(Ctx& ctx, const Q4MmaArgs& a) {
  const unsigned sms = static_cast<unsigned>(ctx.sm_count > 0 ? ctx.sm_count : 148);
  const unsigned row_warps = (a.n + 7) / 8;  // CTAs if every warp took a single row
  // CTAs per SM that the register file holds at once (256 threads each), so that the whole grid is resident and the rows stay interleaved
  constexpr unsigned per_sm = ROWS > 1 ? 2u : (SLICES == 1 ? 4u : (SLICES == 2 ? 3u : (SLICES == 3 ? 2u : 1u)));
  const unsigned grid = std::min(row_warps, sms * per_sm);
  launch_pdl(q4_dp4a_gemv_kernel<SLICES, ROWS>, dim3(grid), dim3(256), 0, ctx.stream, a);
  ctx.launches++;
}

// A single row of bf16 activations against a large q4 / group-64 matrix whose k is 1024, 2048, 3072 or 4096. Measured
// against the tensor-core streaming form: 2048 x 151936 (an lm_head) 38.2 us against 41.9 with one row in flight fewer; on
// matrices of a few MB (5 us either way, launch and one DRAM round trip) and with two rows (54 against 44 us: the dp4a count
// doubles while the loads stay) it is not faster, so those stay with the tensor-core form.
constexpr uint64_t kDp4aMinWeights = 32ull << 20;
bool run_q4_dp4a(Ctx& ctx, const Q4MmaArgs& a, int x_dt) {
  if (x_dt != BF16 || a.group_size != 64 || a.m != 1 || a.k % 1024 != 0 || a.k > 4096 || static_cast<uint64_t>(a.n) * a.k < kDp4aMinWeights) return false;
  if (reinterpret_cast<size_t>(a.packed) % 16 != 0 || reinterpret_cast<size_t>(a.x) % 16 != 0 || (a.x_row_stride * 2) % 16 != 0) return false;
  switch (a.k / 1024) {
    case 1: launch_q4_dp4a<1, 1>(ctx, a); break;
    case 2: launch_q4_dp4a<2, 1>(ctx, a); break;
    case 3: launch_q4_dp4a<3, 1>(ctx, a); break;
    default: launch_q4_dp4a<4, 1>(ctx, a); break;
  }
  return true;
}

// Dequantises `cols` weight rows (columns of the projection) starting at absolute row `row0` of
// the scale/bias tables into a dense [cols, k] matrix of dtype out_dt; one thread per packed word.
__global__ void dequant_rows_kernel(const unsigned* __restrict__ packed, const void* scales, const void* biases, int p_dt, void* out, int out_dt,
                                    unsigned cols, unsigned k, unsigned bits, unsigned group_size, unsigned row0) {
  pdl_sync();
  const unsigned vpw = 32 / bits, mask = (1u << bits) - 1, words_per_row = k / vpw, groups = k / group_size;
  const size_t total = static_cast<size_t>(cols) * words_per_row;
  // 4-bit weights into a 16-bit slab: one packed word becomes one 16-byte store
  const bool wide = bits == 4 && (out_dt == BF16 || out_dt == F16) && reinterpret_cast<size_t>(out) % 16 == 0;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const unsigned row = static_cast<unsigned>(idx / words_per_row), wi = static_cast<unsigned>(idx % words_per_row);
    const unsigned word = __ldg(packed + idx);
    const size_t g = static_cast<size_t>(row0 + row) * groups + (wi * vpw) / group_size;
    const float s = load_as_f32(scales, p_dt, g), b = load_as_f32(biases, p_dt, g);
    if (wide) {
      unsigned o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = __fadd_rn(__fmul_rn(s, static_cast<float>((word >> (8 * i)) & 15u)), b), hi = __fadd_rn(__fmul_rn(s, static_cast<float>((word >> (8 * i + 4)) & 15u)), b);
        o[i] = out_dt == BF16 ? (static_cast<unsigned>(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) | (static_cast<unsigned>(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16))
                              : (static_cast<unsigned>(__half_as_ushort(__float2half_rn(lo))) | (static_cast<unsigned>(__half_as_ushort(__float2half_rn(hi))) << 16));
      }
      *reinterpret_cast<uint4*>(static_cast<unsigned short*>(out) + idx * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      continue;
    }
    for (unsigned i = 0; i < vpw; ++i)
      store_from_f32(out, out_dt, static_cast<size_t>(row) * k + wi * vpw + i, __fadd_rn(__fmul_rn(s, static_cast<float>((word >> (i * bits)) & mask)), b));
  }
}

__device__ inline float sigmoid_ref(float v) { return 1.0f / (1.0f + expf(-v)); }

// Gathered projection: grid.y = rows * routes; each route uses the expert named by indices.
template <int BITS>
__global__ void __launch_bounds__(256) gather_quant_kernel(QuantArgs a, QuantArgs b, int paired, const unsigned* __restrict__ indices,
                                                           void* out, int out_dt, unsigned routes, size_t total_routes, unsigned experts,
                                                           int epilogue, ErrorRecord* err) {
  pdl_sync();
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
  pdl_sync();
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
    total = __fadd_rn(total, __fmul_rn(load_as_f32(weights, w_dt, route), acc[0]));  // product rounded, then added (lib.rs:1153-1199)
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
                         unsigned group_size, void* workspace, size_t workspace_bytes, void* gemm_scratch, size_t gemm_scratch_bytes) {
  if (m == 0 || n == 0) return;
  // 17 to 64 rows: passes of 16 rows through the decode kernels (the weights of the later passes come from L2 for
  // all but the largest matrices), cheaper than expanding the matrix for a GEMM of so few rows
  if (m > 16 && m <= 64 && out_dt == x_dt && q4_mma_supported(x_dt, p_dt, 16, k, bits, group_size, x, k, packed) && (k * 2) % 16 == 0) {
    for (unsigned r0 = 0; r0 < m; r0 += 16) {
      const unsigned rows = std::min(16u, m - r0);
      Q4MmaArgs a{static_cast<const unsigned short*>(x) + static_cast<size_t>(r0) * k, k, packed, static_cast<const unsigned short*>(scales), static_cast<const unsigned short*>(biases),
                  static_cast<char*>(out) + static_cast<size_t>(r0) * n * 2, out_dt, n, rows, k, n, group_size};
      if (!run_q4_stream(ctx, a, x_dt)) run_q4_mma(ctx, a, x_dt);
    }
    return;
  }
  if (q4_mma_supported(x_dt, p_dt, m, k, bits, group_size, x, k, packed)) {
    Q4MmaArgs a{static_cast<const unsigned short*>(x), k, packed, static_cast<const unsigned short*>(scales), static_cast<const unsigned short*>(biases),
                out, out_dt, n, m, k, n, group_size};
    if (run_q4_dp4a(ctx, a, x_dt)) return;
    if (!run_q4_stream(ctx, a, x_dt)) run_q4_mma(ctx, a, x_dt);
    return;
  }
  // More than 16 rows of 16-bit activations: dequantise a slab of columns into the workspace in
  // the activation dtype and run the dense tensor-core GEMM on it (the weights are rounded to
  // 16 bits once, which stays inside the quantised tolerance).
  const size_t esz = 2;
  if (m > 16 && (x_dt == BF16 || x_dt == F16) && out_dt == x_dt && workspace != nullptr && k % 8 == 0 && workspace_bytes >= static_cast<size_t>(k) * 64 * esz) {
    unsigned slab = static_cast<unsigned>(std::min<size_t>(n, workspace_bytes / (static_cast<size_t>(k) * esz)));
    if (slab < n) slab = slab / 64 * 64;
    for (unsigned n0 = 0; n0 < n; n0 += slab) {
      const unsigned cols = std::min(slab, n - n0);
      const size_t total = static_cast<size_t>(cols) * k / 8;
      dequant_rows_kernel<<<static_cast<unsigned>(std::min<size_t>((total + 255) / 256, 65535u * 8)), 256, 0, ctx.stream>>>(
          packed + static_cast<size_t>(n0) * (k * bits / 32), scales, biases, p_dt, workspace, x_dt, cols, k, bits, group_size, n0);
      ctx.launches++;
      launch_gemm_nt(ctx, x, x_dt, k, workspace, x_dt, k, static_cast<char*>(out) + static_cast<size_t>(n0) * esz, out_dt, n, m, cols, k, gemm_scratch, gemm_scratch_bytes);
    }
    return;
  }
  QuantArgs a{x, x_dt, k, packed, scales, biases, p_dt, k, n, bits, group_size};
  unsigned row_groups = (m + QM - 1) / QM;
  dim3 grid((n + 7) / 8, min(row_groups, 65535u));
  if (bits == 4) launch_pdl(quant_matmul_kernel<4>, grid, dim3(256), 0, ctx.stream, a, out, out_dt, m);
  else launch_pdl(quant_matmul_kernel<8>, grid, dim3(256), 0, ctx.stream, a, out, out_dt, m);
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
  if (bits == 4) launch_pdl(gather_quant_kernel<4>, grid, dim3(256), 0, ctx.stream, a, b, paired, indices, out, out_dt, routes, total_routes, experts, epilogue, err);
  else launch_pdl(gather_quant_kernel<8>, grid, dim3(256), 0, ctx.stream, a, b, paired, indices, out, out_dt, routes, total_routes, experts, epilogue, err);
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
  if (bits == 4) launch_pdl(gather_weighted_kernel<4>, grid, dim3(256), 0, ctx.stream, a, indices, weights, w_dt, extra, e_dt, out, out_dt, rows, routes, experts, epilogue, err);
  else launch_pdl(gather_weighted_kernel<8>, grid, dim3(256), 0, ctx.stream, a, indices, weights, w_dt, extra, e_dt, out, out_dt, rows, routes, experts, epilogue, err);
  ctx.launches++;
}

}  // namespace fj
