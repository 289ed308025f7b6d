// Building blocks of the int8 tensor-core form of the MLX 4-bit projections, shared by the
// streaming kernel of plain projections (fj_quant.cu) and the per-expert one (fj_grouped.cu).
// Reference semantics: affine group quantisation, w = scale * q + bias with 8 nibbles per u32,
// lowest nibble first (crates/forja-cpu/src/lib.rs:878-962).
//
// The nibbles stay integers (`w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are u8 A operands of
// mma.sync m16n8k32); the activations become block fixed point, per (row, 64-k block) a
// power-of-two step S = 2^(E-11) and x / S as a 13-bit integer split into a signed high byte and
// an unsigned low byte. Per block: y += (s * S) * (256 * hi + lo) + b * sum_k x.
#pragma once

#include "fj_common.cuh"

namespace fj {

constexpr int Q4W_ROW_STRIDE = 160;                     // bytes between the rows of a unit in shared memory (128 of data)
constexpr int Q4W_PARAM_OFFSET = 16 * Q4W_ROW_STRIDE;
constexpr int Q4W_UNIT_BYTES = Q4W_PARAM_OFFSET + 256;  // 16 rows x 256 k of nibbles, then scales [16][4] u16, biases [16][4] u16
constexpr int Q4W_X_BYTES = 1024 + 64;                  // per (64-k block, 8-row tile): fragments + {sum, step} per row

template <bool kSignedB>
__device__ inline void mma_u8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  if (kSignedB) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// One warp turns 64 k of 8 activation rows into fragment order. Lane (g, t) reads the 16 values
// k = 16 t .. 16 t + 15 of row g (`row` points at them, nullptr for a row that does not exist) and
// writes its hi and lo B registers to `hi_out[lane]`, `lo_out[lane]`; lane t == 0 writes {sum, step}
// of row g to `meta[g]`. A block without a usable step (all zeros, subnormals, infinities or
// NaNs) keeps only its bias term.
__device__ inline void q4_i8_convert_block(const unsigned short* row, uint4* hi_out, uint4* lo_out, float2* meta, unsigned lane) {
  const unsigned g = lane >> 2, t = lane & 3;
  uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
  if (row != nullptr) {
    x0 = *reinterpret_cast<const uint4*>(row);
    x1 = *reinterpret_cast<const uint4*>(row + 8);
  }
  const unsigned raw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
  float f[16];
  float sum = 0.0f, biggest = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    f[2 * i] = __uint_as_float((raw[i] & 0xFFFFu) << 16);
    f[2 * i + 1] = __uint_as_float(raw[i] & 0xFFFF0000u);
    sum += f[2 * i] + f[2 * i + 1];
    biggest = fmaxf(biggest, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, 1));
  biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, 2));
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
  hi_out[lane] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  lo_out[lane] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  if (t == 0) meta[g] = make_float2(sum, usable ? step : 0.0f);
}

// One unit (16 weight rows x 256 k, group size 64) of a ring stage against NB 8-row activation tiles:
// y[nb] = {(row 2t, col g), (row 2t+1, col g), (row 2t, col g+8), (row 2t+1, col g+8)} accumulates.
// `xq_unit` / `meta_unit` point at the unit's first 64-k block of the converted activations
// ([block][NB][2][32] uint4 and [block][NB][8] float2).
template <int NB>
__device__ inline void q4_i8_unit_g64(const unsigned char* stage, const uint4* xq_unit, const float2* meta_unit, unsigned lane, float (&y)[NB][4]) {
  constexpr int kMagic = 0x4B400000;  // bit pattern of 12582912.0f: the low accumulator starts there, so 256 * hi + lo read as f32 is 12582912 + sum
  constexpr float kMagicF = 12582912.0f;
  const unsigned g = lane >> 2, t = lane & 3;
  const uint2 sa = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + g * 8);
  const uint2 sb = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + (g + 8) * 8);
  const uint2 ba = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + 128 + g * 8);
  const uint2 bb = *reinterpret_cast<const uint2*>(stage + Q4W_PARAM_OFFSET + 128 + (g + 8) * 8);
  const unsigned w[8] = {sa.x, sa.y, sb.x, sb.y, ba.x, ba.y, bb.x, bb.y};
  float v8[8][2];
#pragma unroll
  for (int i = 0; i < 8; ++i) { v8[i][0] = __uint_as_float(w[i] << 16); v8[i][1] = __uint_as_float(w[i] & 0xFFFF0000u); }
  xq_unit += lane;
  meta_unit += 2 * t;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float s_a = v8[0 + (j >> 1)][j & 1], s_b = v8[2 + (j >> 1)][j & 1], b_a = v8[4 + (j >> 1)][j & 1], b_b = v8[6 + (j >> 1)][j & 1];
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
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = __int_as_float(hi[i] * 256 + lo[i]) - kMagicF;  // |256 * hi + lo| < 2^22
      y[nb][0] += (s_a * meta.y) * v[0] + b_a * meta.x;
      y[nb][1] += (s_a * meta.w) * v[1] + b_a * meta.z;
      y[nb][2] += (s_b * meta.y) * v[2] + b_b * meta.x;
      y[nb][3] += (s_b * meta.w) * v[3] + b_b * meta.z;
    }
  }
}

}  // namespace fj
