// Grouped expert projections for many routed rows (reference counterparts: the sorted MoE path of
// crates/forja-metal/kernels/quant_matmul.metal: count_expert_routes :1217, plan_expert_routes
// :1255, arrange_expert_routes :1312, grouped_quantized_pair_32x32_2x2_blocked :1615; operator
// semantics: Op::GatherQuantMatmul, crates/forja-cpu/src/lib.rs:964-1204).
//
// The per-route kernels read an expert's whole matrix for every route, which is right for a few
// decode rows and hopeless beyond. Here the routes are bucketed by expert (histogram, scan,
// arrange; one CTA, like the reference) and cut into tiles of one expert's rows; three forms run
// the tiles, chosen by the average number of rows per expert:
//  * 16-row tiles streamed through the int8 tensor-core q4 form (expert_q4_stream_kernel below):
//    every active expert's nibbles are read once per tile, activations in block fixed point;
//  * 128-row tiles on tcgen05 with TMEM accumulators (fj_grouped_tc5.cu);
//  * 64- or 128-row mma.sync tiles (grouped_q4_gemm_kernel below) for shapes the other two refuse:
//    per 64-k step (= one quantisation group) the CTA copies 64 columns x 32 bytes of nibbles with
//    cp.async, expands them to bf16 (one bf16x2 fma per pair of weights) into a swizzled shared
//    tile and feeds mma.sync m16n8k16 through ldmatrix; rows of A are gathered through the sorted
//    route list.
//  pair mode: gate and up tiles share the A tile; epilogue silu(gate) * up -> act[route] (bf16)
//  single mode: f32 result per route (the weighted combine adds them in route order afterwards)
// The order of rows inside an expert's bucket is whatever the atomics give; it only decides which
// tile a row lands in, never its value.
#include "fj_kernels.h"
#include "fj_q4_i8.cuh"
#include "fj_grouped.cuh"

#include <algorithm>

namespace fj {

namespace {

constexpr int GT_BN = 64, GT_BK = 64;  // columns and k per tile step; rows per tile: 64 or 128 (template parameter)

// One CTA: histogram of routes per expert, exclusive scan, arrange, tile list.
// slab_counts != nullptr: the routes come in slabs that start slab_cap entries apart; of slab s only the slab_counts[s]
// entries (at most slab_limit) from slab_offset on are in use (the rows one chunk received from peer s); nothing else is read.
__global__ void __launch_bounds__(1024) route_plan_kernel(const unsigned* __restrict__ indices, unsigned total, unsigned experts, unsigned* offsets /*[experts + 1]*/,
                                                          unsigned* sorted /*[total]*/, RouteTile* tiles, unsigned* n_tiles, unsigned tiles_cap, unsigned tile_rows, ErrorRecord* err,
                                                          const unsigned* __restrict__ slab_counts, unsigned slab_cap, unsigned slab_offset, unsigned slab_limit) {
  extern __shared__ unsigned plan_smem[];
  pdl_sync();
  unsigned* count = plan_smem;           // [experts]
  unsigned* cursor = plan_smem + experts;  // [experts]
  for (unsigned e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  const unsigned slabs = slab_counts ? total / slab_cap : 1u, slab_len = slab_counts ? slab_cap : total;
  for (unsigned s = 0; s < slabs; ++s) {
    const unsigned used = slab_counts ? min(slab_counts[s], slab_limit) : total;
    for (unsigned i = threadIdx.x; i < used; i += blockDim.x) {
      const unsigned e = indices[s * slab_len + slab_offset + i];
      if (e < experts) atomicAdd(&count[e], 1u);
      else report_error(err, ERR_INDEX, e);  // left out of every bucket; the lowest bad id is reported (lib.rs:1078-1088)
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned running = 0, made = 0;
    for (unsigned e = 0; e < experts; ++e) {
      offsets[e] = running;
      cursor[e] = running;
      for (unsigned f = 0; f < count[e]; f += tile_rows) {
        if (made < tiles_cap) tiles[made] = RouteTile{e, running + f, min(tile_rows, count[e] - f)};
        ++made;
      }
      running += count[e];
    }
    offsets[experts] = running;
    *n_tiles = min(made, tiles_cap);
  }
  __syncthreads();
  for (unsigned s = 0; s < slabs; ++s) {
    const unsigned used = slab_counts ? min(slab_counts[s], slab_limit) : total;
    for (unsigned i = threadIdx.x; i < used; i += blockDim.x) {
      const unsigned r = s * slab_len + slab_offset + i, e = indices[r];
      if (e < experts) sorted[atomicAdd(&cursor[e], 1u)] = r;
    }
  }
}

__device__ inline void g_cp_async_16(unsigned smem_addr, const void* gmem, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void g_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ inline void g_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ inline unsigned pack_bf16(float lo, float hi) {
  return static_cast<unsigned>(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) | (static_cast<unsigned>(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
}

// Shared memory of one CTA: A stages, the expanded B tile(s), nibble stages, scales and biases, route ids.
template <bool kPair, int BM>
constexpr size_t grouped_smem_bytes() {
  return 2 * BM * 128 + (kPair ? 2 : 1) * (GT_BN * 128 + 2 * GT_BN * 32 + 2 * GT_BN * 2 * 2) + BM * 4;
}

// BM rows of one expert x 64 columns per CTA, BM / 32 x 2 warps of 32 x 32.
template <bool kPair, int BM>
__global__ void __launch_bounds__(BM * 2) grouped_q4_gemm_kernel(GroupedArgs p) {
  constexpr int NW = kPair ? 2 : 1, THREADS = BM * 2, PARTS = THREADS / GT_BN, WORDS = 8 / PARTS;  // a thread expands WORDS packed words of one column per matrix
  extern __shared__ __align__(128) unsigned char g_smem[];
  unsigned char* s_a = g_smem;                                   // [2][BM * 128]
  unsigned char* s_b = s_a + 2 * BM * 128;                        // [NW][GT_BN * 128]
  unsigned char* s_q = s_b + NW * GT_BN * 128;                    // [2][NW][GT_BN * 32]
  unsigned short* s_scale = reinterpret_cast<unsigned short*>(s_q + 2 * NW * GT_BN * 32);  // [2][NW][GT_BN]
  unsigned short* s_bias = s_scale + 2 * NW * GT_BN;              // [2][NW][GT_BN]
  unsigned* s_route = reinterpret_cast<unsigned*>(s_bias + 2 * NW * GT_BN);  // [BM]
  pdl_sync();
  if (blockIdx.y >= *p.n_tiles) return;
  const RouteTile tile = p.tiles[blockIdx.y];
  const unsigned col0 = blockIdx.x * GT_BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp >> 1, warp_n = warp & 1;
  const bool rows_live = static_cast<unsigned>(warp_m) * 32 < tile.count;  // a warp whose 32 rows are all padding only helps with the copies
  const unsigned k_iters = p.k / GT_BK, words_per_row = p.k / 8, groups_per_row = p.k / 64;
  for (unsigned i = threadIdx.x; i < BM; i += THREADS) s_route[i] = i < tile.count ? p.sorted[tile.first + i] : 0xFFFFFFFFu;
  __syncthreads();
  const unsigned a_base = static_cast<unsigned>(__cvta_generic_to_shared(s_a));
  const unsigned b_base = static_cast<unsigned>(__cvta_generic_to_shared(s_b));
  const unsigned q_base = static_cast<unsigned>(__cvta_generic_to_shared(s_q));
  const size_t expert_rows = static_cast<size_t>(tile.expert) * p.n;

  float acc[NW][2][4][4];
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[w][i][j][0] = acc[w][i][j][1] = acc[w][i][j][2] = acc[w][i][j][3] = 0.0f;

  // source row of this thread's A chunks (4 chunks of 16 bytes per thread and stage: rows r, r + THREADS / 8, ...)
  const unsigned a_c8 = threadIdx.x & 7;
  const unsigned short* a_src[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const unsigned route = s_route[(threadIdx.x >> 3) + i * (THREADS / 8)];
    a_src[i] = route != 0xFFFFFFFFu ? p.x + static_cast<size_t>(route / p.src_div) * p.k + a_c8 * 8 : nullptr;
  }

  auto issue = [&](unsigned it) {
    if (it < k_iters) {
      const unsigned stage = it & 1, kk = it * GT_BK;
      // A: BM rows x 8 chunks of 16 bytes, gathered through the route list
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const unsigned r = (threadIdx.x >> 3) + i * (THREADS / 8);
        const bool ok = a_src[i] != nullptr;
        g_cp_async_16(a_base + stage * (BM * 128) + r * 128 + ((a_c8 ^ (r & 7)) << 4), ok ? static_cast<const void*>(a_src[i] + kk) : static_cast<const void*>(p.x), ok ? 16u : 0u);
      }
      // packed weights: 64 columns x 2 chunks of 16 bytes per matrix; scales / biases: one u16 each
      if (threadIdx.x < 128) {
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          const unsigned c = threadIdx.x >> 1, half = threadIdx.x & 1;
          const bool ok = col0 + c < p.n;
          const size_t row = expert_rows + (ok ? col0 + c : 0);
          g_cp_async_16(q_base + ((stage * NW + w) * GT_BN + c) * 32 + half * 16, p.packed[w] + row * words_per_row + (kk / 8) + half * 4, ok ? 16u : 0u);
          if (half == 0) s_scale[(stage * NW + w) * GT_BN + c] = ok ? p.scales[w][row * groups_per_row + it] : static_cast<unsigned short>(0);
          else s_bias[(stage * NW + w) * GT_BN + c] = ok ? p.biases[w][row * groups_per_row + it] : static_cast<unsigned short>(0);
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  issue(0);
  for (unsigned it = 0; it < k_iters; ++it) {
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();  // stage `it` landed; everyone finished the previous step's mma (s_b and the other stage are free)
    issue(it + 1);
    const unsigned stage = it & 1;
    // expand this step's nibbles: thread -> (column, part of the 64-k step). Nibbles j and j + 4 of a word are OR-ed
    // into the mantissa of bf16 128.0, 128 is subtracted (exact), one bf16x2 fma gives bf16(s * q + b) with a
    // single rounding, and two byte permutes put the eight results back in k order.
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const unsigned c = threadIdx.x / PARTS, part = threadIdx.x % PARTS;
      const unsigned sc = s_scale[(stage * NW + w) * GT_BN + c], bi = s_bias[(stage * NW + w) * GT_BN + c];
      const unsigned s2 = sc | (sc << 16), b2 = bi | (bi << 16);
      const __nv_bfloat162 scale2 = *reinterpret_cast<const __nv_bfloat162*>(&s2), bias2 = *reinterpret_cast<const __nv_bfloat162*>(&b2);
      const unsigned offset_bits = 0x43004300u;
      const __nv_bfloat162 offset2 = *reinterpret_cast<const __nv_bfloat162*>(&offset_bits);
      const unsigned* q = reinterpret_cast<const unsigned*>(s_q + ((stage * NW + w) * GT_BN + c) * 32 + part * (WORDS * 4));
#pragma unroll
      for (int i = 0; i < WORDS; ++i) {
        const unsigned word = q[i];
        unsigned r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const unsigned pair_bits = ((word >> (4 * j)) & 0x000F000Fu) | 0x43004300u;  // {128 + nibble j, 128 + nibble j + 4}
          const __nv_bfloat162 value = __hfma2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pair_bits), offset2), scale2, bias2);
          r[j] = *reinterpret_cast<const unsigned*>(&value);
        }
        const uint4 packed = make_uint4(__byte_perm(r[0], r[1], 0x5410), __byte_perm(r[2], r[3], 0x5410), __byte_perm(r[0], r[1], 0x7632), __byte_perm(r[2], r[3], 0x7632));
        const unsigned chunk = part * WORDS + i;
        *reinterpret_cast<uint4*>(s_b + w * (GT_BN * 128) + c * 128 + ((chunk ^ (c & 7)) << 4)) = packed;
      }
    }
    __syncthreads();
    if (!rows_live) continue;
#pragma unroll
    for (int ks = 0; ks < GT_BK / 16; ++ks) {
      unsigned af[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const unsigned mi = lane >> 3, rr = lane & 7;
        const unsigned r = warp_m * 32 + i * 16 + (mi & 1) * 8 + rr;
        const unsigned chunk = ks * 2 + (mi >> 1);
        g_ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], a_base + stage * (BM * 128) + r * 128 + ((chunk ^ (r & 7)) << 4));
      }
#pragma unroll
      for (int w = 0; w < NW; ++w)
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
          const unsigned mi = lane >> 3, rr = lane & 7;
          const unsigned r = warp_n * 32 + j * 8 + (mi >> 1) * 8 + rr;
          const unsigned chunk = ks * 2 + (mi & 1);
          unsigned b0, b1, b2, b3;
          g_ldmatrix_x4(b0, b1, b2, b3, b_base + w * (GT_BN * 128) + r * 128 + ((chunk ^ (r & 7)) << 4));
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            g_mma(acc[w][i][j], af[i], b0, b1);
            g_mma(acc[w][i][j + 1], af[i], b2, b3);
          }
        }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");

  const unsigned gr = lane >> 2, gc = (lane & 3) * 2;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int e = 0; e < 4; e += 2) {
      const unsigned r = warp_m * 32 + i * 16 + gr + (e >> 1) * 8;
      const unsigned route = s_route[r];
      if (route == 0xFFFFFFFFu) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned col = col0 + warp_n * 32 + j * 8 + gc;
        if (col >= p.n) continue;
        float v0 = acc[0][i][j][e], v1 = acc[0][i][j][e + 1];
        if (kPair) {
          v0 = v0 * (1.0f / (1.0f + expf(-v0))) * acc[NW - 1][i][j][e];
          v1 = v1 * (1.0f / (1.0f + expf(-v1))) * acc[NW - 1][i][j][e + 1];
          unsigned short* o = static_cast<unsigned short*>(p.out) + static_cast<size_t>(route) * p.n + col;
          if (col + 1 < p.n) *reinterpret_cast<unsigned*>(o) = pack_bf16(v0, v1);
          else *o = __bfloat16_as_ushort(__float2bfloat16_rn(v0));
        } else if (p.out_bf16) {
          unsigned short* o = static_cast<unsigned short*>(p.out) + static_cast<size_t>(route) * p.n + col;
          if (col + 1 < p.n) *reinterpret_cast<unsigned*>(o) = pack_bf16(v0, v1);
          else *o = __bfloat16_as_ushort(__float2bfloat16_rn(v0));
        } else {
          float* o = static_cast<float*>(p.out) + static_cast<size_t>(route) * p.n + col;
          if (col + 1 < p.n) *reinterpret_cast<float2*>(o) = make_float2(v0, v1);
          else *o = v0;
        }
      }
    }
}

// ---- streaming form for few rows per expert (decode) ----
// With a handful of rows per expert the projections are bound by reading every active expert's
// nibbles once. The routes are bucketed as above but cut into tiles of 16 rows; CTA (chunk, tile)
// converts the tile's rows to block fixed point in shared memory once and its warps stream
// 16-column weight tiles of that expert (units of 256 k through a per-warp cp.async ring) into
// int8 tensor-core products, exactly like the plain decode projections. Pair mode streams the
// gate tile and then the up tile of the same columns and stores silu(gate) * up.
struct ExpertStreamArgs {
  const unsigned short* x;
  const unsigned* packed[2];
  const unsigned short* scales[2];
  const unsigned short* biases[2];
  const unsigned* sorted;
  const RouteTile* tiles;
  const unsigned* n_tiles;
  void* out;  // [routes][n]: pair bf16; single f32 (bf16 when out_bf16)
  unsigned k, n, src_div, cols_per_cta;  // cols_per_cta: 16-column tiles per chunk
  int out_bf16;
};

template <bool kPair, int NB, int STAGES, int WARPS>
__device__ __forceinline__ void expert_stream_body(const ExpertStreamArgs& a, const RouteTile tile, unsigned char* smem, const unsigned* s_route) {
  constexpr int MATS = kPair ? 2 : 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned g = lane >> 2, t = lane & 3;
  const unsigned blocks = a.k / 64, upt = a.k / 256;
  uint4* xq = reinterpret_cast<uint4*>(smem);                                              // [blocks][NB][2][32]
  float2* xmeta = reinterpret_cast<float2*>(smem + static_cast<size_t>(blocks) * NB * 1024);  // [blocks][NB][8] {sum, step}
  unsigned char* ring = smem + static_cast<size_t>(blocks) * 2 * Q4W_X_BYTES + warp * (STAGES * Q4W_UNIT_BYTES);
  const unsigned ring_base = static_cast<unsigned>(__cvta_generic_to_shared(ring));

  const unsigned col_tiles = (a.n + 15) / 16, c_begin = blockIdx.x * a.cols_per_cta, c_end = min(c_begin + a.cols_per_cta, col_tiles);
  const unsigned c_first = c_begin + warp;
  const unsigned my_cols = c_first < c_end ? (c_end - c_first + WARPS - 1) / WARPS : 0;
  const unsigned items = my_cols * MATS * upt;
  const size_t row_bytes = a.k / 2, expert_row0 = static_cast<size_t>(tile.expert) * a.n;
  const unsigned copy_row = lane >> 3, copy_col = (lane & 7) * 16;
  const unsigned param_which = lane >> 4, param_col = lane & 15;
  const unsigned copy_dst = copy_row * Q4W_ROW_STRIDE + copy_col, param_dst = Q4W_PARAM_OFFSET + param_which * 128 + param_col * 8;

  unsigned in_c = c_first, in_mat = 0, in_u = 0, in_stage = 0, in_count = 0;
  const unsigned char* in_rows[4];
  const unsigned short* in_param = nullptr;
  auto issue = [&]() {
    if (in_count < items) {
      if (in_u == 0) {
        const unsigned char* wbase = reinterpret_cast<const unsigned char*>(in_mat == 0 ? a.packed[0] : a.packed[MATS - 1]);
        const unsigned short* pbase = param_which ? (in_mat == 0 ? a.biases[0] : a.biases[MATS - 1]) : (in_mat == 0 ? a.scales[0] : a.scales[MATS - 1]);
#pragma unroll
        for (int i = 0; i < 4; ++i) in_rows[i] = wbase + (expert_row0 + min(in_c * 16 + copy_row + 4 * i, a.n - 1)) * row_bytes + copy_col;
        in_param = pbase + (expert_row0 + min(in_c * 16 + param_col, a.n - 1)) * blocks;
      }
      const unsigned stage = ring_base + in_stage * Q4W_UNIT_BYTES;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(stage + copy_dst + i * (4 * Q4W_ROW_STRIDE)), "l"(in_rows[i] + in_u * 128) : "memory");
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(stage + param_dst), "l"(in_param + in_u * 4) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    ++in_count;
    in_stage = in_stage + 1 == STAGES ? 0 : in_stage + 1;
    if (++in_u == upt) {
      in_u = 0;
      if (++in_mat == MATS) { in_mat = 0; in_c += WARPS; }
    }
  };
  for (int q = 0; q + 1 < STAGES; ++q) issue();  // weights are on their way while the rows are converted

  const unsigned short* x_row[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const unsigned route = s_route[g + 8 * nb];
    x_row[nb] = route == 0xFFFFFFFFu ? nullptr : a.x + static_cast<size_t>(route / a.src_div) * a.k + 16 * t;
  }
  for (unsigned b = warp; b < blocks; b += WARPS) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
      q4_i8_convert_block(x_row[nb] ? x_row[nb] + b * 64 : nullptr, xq + ((b * NB + nb) * 2 + 0) * 32, xq + ((b * NB + nb) * 2 + 1) * 32, xmeta + (b * NB + nb) * 8, lane);
  }
  __syncthreads();

  float y[NB][4], gate[NB][4];
  unsigned c = c_first, mat = 0, u = 0, out_stage = 0;
  for (unsigned q = 0; q < items; ++q) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2) : "memory");
    __syncwarp();  // unit q is visible to the whole warp, and the warp is done with unit q - 1
    issue();
    if (u == 0) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) y[nb][0] = y[nb][1] = y[nb][2] = y[nb][3] = 0.0f;
    }
    q4_i8_unit_g64<NB>(ring + out_stage * Q4W_UNIT_BYTES, xq + static_cast<size_t>(u * 4) * (NB * 2 * 32), xmeta + static_cast<size_t>(u * 4) * (NB * 8), lane, y);
    out_stage = out_stage + 1 == STAGES ? 0 : out_stage + 1;
    if (++u == upt) {
      u = 0;
      if (kPair && mat == 0) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int i = 0; i < 4; ++i) gate[nb][i] = y[nb][i];
        mat = 1;
      } else {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const unsigned route = s_route[8 * nb + 2 * t + (i & 1)], col = c * 16 + g + (i >> 1) * 8;
            if (route == 0xFFFFFFFFu || col >= a.n) continue;
            const size_t o = static_cast<size_t>(route) * a.n + col;
            float v = y[nb][i];
            if (kPair) v = gate[nb][i] * (1.0f / (1.0f + expf(-gate[nb][i]))) * v;
            if (kPair || a.out_bf16) static_cast<unsigned short*>(a.out)[o] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
            else static_cast<float*>(a.out)[o] = v;
          }
        mat = 0;
        c += WARPS;
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <bool kPair, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) expert_q4_stream_kernel(ExpertStreamArgs a) {
  extern __shared__ __align__(128) unsigned char es_smem[];
  unsigned* s_route = reinterpret_cast<unsigned*>(es_smem + static_cast<size_t>(a.k / 64) * 2 * Q4W_X_BYTES + static_cast<size_t>(WARPS) * STAGES * Q4W_UNIT_BYTES);  // [16]
  pdl_sync();  // the plan and the rows come from the kernels before
  if (blockIdx.y >= *a.n_tiles) return;
  const RouteTile tile = a.tiles[blockIdx.y];
  if (threadIdx.x < 16) s_route[threadIdx.x] = threadIdx.x < tile.count ? a.sorted[tile.first + threadIdx.x] : 0xFFFFFFFFu;
  __syncthreads();
  if (tile.count <= 8) expert_stream_body<kPair, 1, STAGES, WARPS>(a, tile, es_smem, s_route);
  else expert_stream_body<kPair, 2, STAGES, WARPS>(a, tile, es_smem, s_route);
}

template <bool kPair, int STAGES, int WARPS>
bool launch_expert_stream(Ctx& ctx, ExpertStreamArgs a, unsigned tiles_cap, unsigned est_tiles) {
  const size_t smem = static_cast<size_t>(a.k / 64) * 2 * Q4W_X_BYTES + static_cast<size_t>(WARPS) * STAGES * Q4W_UNIT_BYTES + 64;  // + the tile's 16 route ids
  if (smem > 227 * 1024) return false;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64) return false;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(expert_q4_stream_kernel<kPair, STAGES, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) { cudaGetLastError(); return false; }
    configured[device] = true;
  }
  // enough CTAs for about three per SM, never less than one 16-column tile per warp
  const unsigned sms = static_cast<unsigned>(ctx.sm_count > 0 ? ctx.sm_count : 148), col_tiles = (a.n + 15) / 16;
  unsigned chunks = (3 * sms + est_tiles - 1) / std::max(est_tiles, 1u);
  chunks = std::max(1u, std::min(chunks, std::max(1u, col_tiles / WARPS)));
  a.cols_per_cta = (col_tiles + chunks - 1) / chunks;
  chunks = (col_tiles + a.cols_per_cta - 1) / a.cols_per_cta;
  launch_pdl(expert_q4_stream_kernel<kPair, STAGES, WARPS>, dim3(chunks, tiles_cap), dim3(WARPS * 32), smem, ctx.stream, a);
  ctx.launches++;
  return true;
}

template <bool kPair>
bool run_expert_stream(Ctx& ctx, const ExpertStreamArgs& a, unsigned tiles_cap, unsigned est_tiles) {
  return launch_expert_stream<kPair, 4, 16>(ctx, a, tiles_cap, est_tiles) || launch_expert_stream<kPair, 3, 16>(ctx, a, tiles_cap, est_tiles) ||
         launch_expert_stream<kPair, 3, 8>(ctx, a, tiles_cap, est_tiles);
}

}  // namespace

size_t route_plan_bytes(unsigned total_routes, unsigned experts) {
  const size_t tiles_cap = total_routes / 16 + experts + 1;  // sized for the smallest tile height (16 rows)
  return (static_cast<size_t>(experts) + 1 + total_routes + 4) * sizeof(unsigned) + tiles_cap * sizeof(RouteTile) + 64;
}

namespace {
struct PlanLayout {
  unsigned *offsets, *sorted, *n_tiles;
  RouteTile* tiles;
  unsigned tiles_cap;
};
PlanLayout plan_layout(void* plan, unsigned total_routes, unsigned experts) {
  PlanLayout l;
  unsigned* base = static_cast<unsigned*>(plan);
  l.n_tiles = base;  // 4 words reserved
  l.offsets = base + 4;
  l.sorted = l.offsets + experts + 1;
  size_t words = 4 + static_cast<size_t>(experts) + 1 + total_routes;
  words = (words + 3) / 4 * 4;
  l.tiles = reinterpret_cast<RouteTile*>(base + words);
  l.tiles_cap = total_routes / 16 + experts + 1;
  return l;
}
}  // namespace

void launch_route_plan(Ctx& ctx, const unsigned* indices, unsigned total_routes, unsigned experts, void* plan, ErrorRecord* err, unsigned tile_rows, const unsigned* slab_counts,
                       unsigned slab_cap, unsigned slab_offset, unsigned slab_limit) {
  const PlanLayout l = plan_layout(plan, total_routes, experts);
  if (slab_counts && (slab_cap == 0 || total_routes % slab_cap != 0 || slab_offset >= slab_cap)) slab_counts = nullptr;
  if (slab_limit == 0 || slab_limit > slab_cap - slab_offset) slab_limit = slab_cap - slab_offset;
  launch_pdl(route_plan_kernel, dim3(1), dim3(1024), 2 * experts * sizeof(unsigned), ctx.stream, indices, total_routes, experts, l.offsets, l.sorted, l.tiles, l.n_tiles, l.tiles_cap,
             tile_rows, err, slab_counts, slab_cap, slab_counts ? slab_offset : 0u, slab_limit);
  ctx.launches++;
}

// 128-row tiles (tcgen05) once the average expert fills half of one, else 64-row tiles.
unsigned grouped_tile_rows(unsigned total_routes, unsigned experts) { return total_routes >= 64ull * experts ? 128u : 64u; }

bool grouped_q4_supported(unsigned k, unsigned n, unsigned bits, unsigned group_size, unsigned experts, const void* x, const void* packed) {
  return bits == 4 && group_size == 64 && k % 64 == 0 && n % 2 == 0 && experts <= 4096 && reinterpret_cast<size_t>(x) % 16 == 0 && reinterpret_cast<size_t>(packed) % 16 == 0;
}

namespace {
template <bool kPair, int BM>
void launch_grouped(Ctx& ctx, const GroupedArgs& a, unsigned tiles) {
  constexpr size_t smem = grouped_smem_bytes<kPair, BM>();
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    cudaFuncSetAttribute(grouped_q4_gemm_kernel<kPair, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    configured[device] = true;
  }
  launch_pdl(grouped_q4_gemm_kernel<kPair, BM>, dim3((a.n + GT_BN - 1) / GT_BN, tiles), dim3(BM * 2), smem, ctx.stream, a);
  ctx.launches++;
}
// tile_rows must be the value the plan was made with (64 or 128); the grid covers the most tiles such a plan can hold
template <bool kPair>
void run_grouped(Ctx& ctx, const GroupedArgs& a, unsigned tile_rows, unsigned total_routes, unsigned experts) {
  const unsigned tiles = total_routes / tile_rows + experts + 1;
  if (tile_rows == 128 && grouped_tc5_supported(a)) launch_grouped_tc5(ctx, a, kPair, tiles);  // tcgen05 tiles with TMEM accumulators
  else if (tile_rows == 128) launch_grouped<kPair, 128>(ctx, a, tiles);
  else launch_grouped<kPair, 64>(ctx, a, tiles);
}
}  // namespace

void launch_grouped_q4_pair(Ctx& ctx, const void* x, const unsigned* gate, const void* gate_scales, const void* gate_biases, const unsigned* up, const void* up_scales,
                            const void* up_biases, const void* plan, unsigned total_routes, unsigned experts, unsigned src_div, void* act_out, unsigned k, unsigned n, unsigned tile_rows) {
  const PlanLayout l = plan_layout(const_cast<void*>(plan), total_routes, experts);
  GroupedArgs a{static_cast<const unsigned short*>(x), {gate, up}, {static_cast<const unsigned short*>(gate_scales), static_cast<const unsigned short*>(up_scales)},
                {static_cast<const unsigned short*>(gate_biases), static_cast<const unsigned short*>(up_biases)}, l.sorted, l.tiles, l.n_tiles, act_out, k, n, src_div, 1};
  run_grouped<true>(ctx, a, tile_rows, total_routes, experts);
}

void launch_grouped_q4_single(Ctx& ctx, const void* x, const unsigned* packed, const void* scales, const void* biases, const void* plan, unsigned total_routes, unsigned experts,
                              unsigned src_div, void* out, bool out_bf16, unsigned k, unsigned n, unsigned tile_rows) {
  const PlanLayout l = plan_layout(const_cast<void*>(plan), total_routes, experts);
  GroupedArgs a{static_cast<const unsigned short*>(x), {packed, packed}, {static_cast<const unsigned short*>(scales), static_cast<const unsigned short*>(scales)},
                {static_cast<const unsigned short*>(biases), static_cast<const unsigned short*>(biases)}, l.sorted, l.tiles, l.n_tiles, out, k, n, src_div, out_bf16 ? 1 : 0};
  run_grouped<false>(ctx, a, tile_rows, total_routes, experts);
}

bool expert_stream_supported(unsigned k, unsigned n, unsigned bits, unsigned group_size, unsigned experts, const void* x, const void* packed, const void* scales, const void* biases) {
  return bits == 4 && group_size == 64 && k % 256 == 0 && k <= 4096 && n >= 1 && experts <= 4096 && reinterpret_cast<size_t>(x) % 16 == 0 && reinterpret_cast<size_t>(packed) % 16 == 0 &&
         reinterpret_cast<size_t>(scales) % 8 == 0 && reinterpret_cast<size_t>(biases) % 8 == 0;
}

// The plan must have been made with 16-row tiles. live_routes: how many of the routes are expected to carry a valid
// expert id (padded exchanges); it only sizes the grid.
bool launch_expert_stream_pair(Ctx& ctx, const void* x, const unsigned* gate, const void* gate_scales, const void* gate_biases, const unsigned* up, const void* up_scales,
                               const void* up_biases, const void* plan, unsigned total_routes, unsigned experts, unsigned src_div, void* act_out, unsigned k, unsigned n, unsigned live_routes) {
  const PlanLayout l = plan_layout(const_cast<void*>(plan), total_routes, experts);
  live_routes = std::min(live_routes, total_routes);
  ExpertStreamArgs a{static_cast<const unsigned short*>(x), {gate, up}, {static_cast<const unsigned short*>(gate_scales), static_cast<const unsigned short*>(up_scales)},
                     {static_cast<const unsigned short*>(gate_biases), static_cast<const unsigned short*>(up_biases)}, l.sorted, l.tiles, l.n_tiles, act_out, k, n, src_div, 0, 1};
  return run_expert_stream<true>(ctx, a, l.tiles_cap, std::min(experts, live_routes) + live_routes / 16);
}

bool launch_expert_stream_single(Ctx& ctx, const void* x, const unsigned* packed, const void* scales, const void* biases, const void* plan, unsigned total_routes, unsigned experts,
                                 unsigned src_div, void* out, bool out_bf16, unsigned k, unsigned n, unsigned live_routes) {
  const PlanLayout l = plan_layout(const_cast<void*>(plan), total_routes, experts);
  live_routes = std::min(live_routes, total_routes);
  ExpertStreamArgs a{static_cast<const unsigned short*>(x), {packed, packed}, {static_cast<const unsigned short*>(scales), static_cast<const unsigned short*>(scales)},
                     {static_cast<const unsigned short*>(biases), static_cast<const unsigned short*>(biases)}, l.sorted, l.tiles, l.n_tiles, out, k, n, src_div, 0, out_bf16 ? 1 : 0};
  return run_expert_stream<false>(ctx, a, l.tiles_cap, std::min(experts, live_routes) + live_routes / 16);
}

unsigned grouped_tcgen05_giveups() { return grouped_tc5_giveups(); }

namespace {
// out[row] = (extra[row] +) sum_j weights[row, j] * per_route[slot(row, j)], j ascending, f32, each product rounded
// before it is added: the arithmetic of the fused weighted-sum projection (lib.rs:1153-1199). route_slot == nullptr:
// the result of route r sits in row r and routes whose expert id is out of range are skipped.
__global__ void routes_combine_kernel(const void* __restrict__ per_route_any, int p_dt, const unsigned* __restrict__ route_slot, const unsigned* __restrict__ expert_ids, unsigned experts,
                                      const void* __restrict__ weights, int w_dt, const void* __restrict__ extra, int e_dt, void* out, int out_dt, unsigned rows, unsigned top_k,
                                      unsigned width) {
  pdl_sync();
  // four columns per thread (16-byte loads of f32 per-route rows, 8-byte loads of bf16 ones) when the row width and the pointer allow it
  const float* per_route = static_cast<const float*>(per_route_any);
  const unsigned short* per_route_h = static_cast<const unsigned short*>(per_route_any);
  const bool wide = width % 4 == 0 && reinterpret_cast<size_t>(per_route_any) % 16 == 0 && (p_dt == F32 || p_dt == BF16);
  for (unsigned row = blockIdx.x; row < rows; row += gridDim.x) {
    if (wide) {
      for (unsigned c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < width; c += gridDim.y * blockDim.x * 4) {
        float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (unsigned j = 0; j < top_k; ++j) {
          const unsigned slot = route_slot ? route_slot[row * top_k + j] : (expert_ids[row * top_k + j] < experts ? row * top_k + j : 0xFFFFFFFFu);
          if (slot == 0xFFFFFFFFu) continue;
          const float w = load_as_f32(weights, w_dt, row * top_k + j);
          float4 v;
          if (p_dt == F32) {
            v = *reinterpret_cast<const float4*>(per_route + static_cast<size_t>(slot) * width + c);
          } else {
            const uint2 h = *reinterpret_cast<const uint2*>(per_route_h + static_cast<size_t>(slot) * width + c);
            v = make_float4(__uint_as_float(h.x << 16), __uint_as_float(h.x & 0xFFFF0000u), __uint_as_float(h.y << 16), __uint_as_float(h.y & 0xFFFF0000u));
          }
          total[0] = __fadd_rn(total[0], __fmul_rn(w, v.x));
          total[1] = __fadd_rn(total[1], __fmul_rn(w, v.y));
          total[2] = __fadd_rn(total[2], __fmul_rn(w, v.z));
          total[3] = __fadd_rn(total[3], __fmul_rn(w, v.w));
        }
        const size_t o = static_cast<size_t>(row) * width + c;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (extra) total[i] = total[i] + load_as_f32(extra, e_dt, o + i);
          store_from_f32(out, out_dt, o + i, total[i]);
        }
      }
      continue;
    }
    for (unsigned c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
      float total = 0.0f;
      for (unsigned j = 0; j < top_k; ++j) {
        const unsigned slot = route_slot ? route_slot[row * top_k + j] : (expert_ids[row * top_k + j] < experts ? row * top_k + j : 0xFFFFFFFFu);
        if (slot == 0xFFFFFFFFu) continue;
        total = __fadd_rn(total, __fmul_rn(load_as_f32(weights, w_dt, row * top_k + j), load_as_f32(per_route_any, p_dt, static_cast<size_t>(slot) * width + c)));
      }
      const size_t o = static_cast<size_t>(row) * width + c;
      if (extra) total = total + load_as_f32(extra, e_dt, o);
      store_from_f32(out, out_dt, o, total);
    }
  }
}
}  // namespace

void launch_routes_combine(Ctx& ctx, const void* per_route, int p_dt, const unsigned* route_slot, const unsigned* expert_ids, unsigned experts, const void* weights, int w_dt, const void* extra,
                           int e_dt, void* out, int out_dt, unsigned rows, unsigned top_k, unsigned width) {
  if (rows == 0) return;
  // few rows: spread the columns of a row over several CTAs so that the grid still fills the GPU
  const unsigned col_ctas = rows >= 1024u ? 1u : std::min((width + 1023u) / 1024u, (1024u + rows - 1) / rows);
  launch_pdl(routes_combine_kernel, dim3(rows < 1024u ? rows : 1024u, col_ctas), dim3(256), 0, ctx.stream, per_route, p_dt, route_slot, expert_ids, experts, weights, w_dt, extra, e_dt, out, out_dt, rows,
             top_k, width);
  ctx.launches++;
}

}  // namespace fj
