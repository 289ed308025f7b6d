// Dense projections of the forward step: C[M,N] = A[M,K] * W[N,K]^T with f32 accumulation and one
// rounding of each output (reference: Op::Matmul, crates/forja-cpu/src/lib.rs:815-848, with the
// weight stored [out, in] and viewed transposed, test :3041-3077).
//
// Three kernels:
//  * gemv_nt: M <= 16 rows, one warp per output column, 16-byte weight loads; HBM-bound on the
//    weight stream (N*K*sizeof(T) bytes per launch).
//  * gemm_nt_mma: 16-bit operands, 128 x BN x 64 tiles, cp.async 3-stage pipeline, ldmatrix +
//    mma.sync m16n8k16, optional split-K through an f32 scratch with last-CTA reduction.
//  * gemm_nt_f32: f32 operands, one thread owns each output and accumulates k in ascending order
//    with separate multiply and add (no FMA contraction), which reproduces the reference's
//    sequential sum bit for bit.
#include "fj_kernels.h"

namespace fj {

namespace {

// ---------------------------------------------------------------------------------------------
// GEMV (M <= 16)
// ---------------------------------------------------------------------------------------------

template <typename T> struct Vec16;  // 16-byte vector of T
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__half> { static constexpr int N = 8; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T, int MAX_M>
__global__ void __launch_bounds__(256) gemv_nt_kernel(const T* __restrict__ a, size_t lda, const T* __restrict__ w, size_t ldw, void* c,
                                                      int c_dt, size_t ldc, unsigned m, unsigned n, unsigned k) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const unsigned col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= n) return;
  float acc[MAX_M];
#pragma unroll
  for (int r = 0; r < MAX_M; ++r) acc[r] = 0.0f;
  const T* wrow = w + static_cast<size_t>(col) * ldw;
  const bool vec_ok = (k % V == 0) && (ldw % V == 0) && (lda % V == 0) &&
                      ((reinterpret_cast<size_t>(w) | reinterpret_cast<size_t>(a)) % 16 == 0);
  if (vec_ok) {
    for (unsigned k0 = lane * V; k0 < k; k0 += 32 * V) {
      uint4 wv = *reinterpret_cast<const uint4*>(wrow + k0);
      const T* wp = reinterpret_cast<const T*>(&wv);
      float wf[V];
#pragma unroll
      for (int i = 0; i < V; ++i) wf[i] = to_f32(wp[i]);
#pragma unroll
      for (int r = 0; r < MAX_M; ++r) {
        if (r < static_cast<int>(m)) {
          uint4 av = *reinterpret_cast<const uint4*>(a + static_cast<size_t>(r) * lda + k0);
          const T* ap = reinterpret_cast<const T*>(&av);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[r] += to_f32(ap[i]) * wf[i];
        }
      }
    }
  } else {
    for (unsigned k0 = lane; k0 < k; k0 += 32) {
      float wf = to_f32(wrow[k0]);
#pragma unroll
      for (int r = 0; r < MAX_M; ++r)
        if (r < static_cast<int>(m)) acc[r] += to_f32(a[static_cast<size_t>(r) * lda + k0]) * wf;
    }
  }
#pragma unroll
  for (int r = 0; r < MAX_M; ++r) {
    if (r < static_cast<int>(m)) {
      float v = warp_sum(acc[r]);
      if (lane == 0) store_from_f32(c, c_dt, static_cast<size_t>(r) * ldc + col, v);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// f32 GEMM, sequential k per output, no FMA contraction
// ---------------------------------------------------------------------------------------------

constexpr int F32_TILE = 32, F32_BK = 32;

__global__ void __launch_bounds__(F32_TILE* F32_TILE) gemm_nt_f32_kernel(const float* __restrict__ a, size_t lda,
                                                                         const float* __restrict__ w, size_t ldw, void* c, int c_dt,
                                                                         size_t ldc, unsigned m, unsigned n, unsigned k) {
  __shared__ float as[F32_TILE][F32_BK + 1];
  __shared__ float ws[F32_TILE][F32_BK + 1];
  const unsigned tx = threadIdx.x % F32_TILE, ty = threadIdx.x / F32_TILE;
  const unsigned row = blockIdx.y * F32_TILE + ty, col = blockIdx.x * F32_TILE + tx;
  float sum = 0.0f;
  for (unsigned k0 = 0; k0 < k; k0 += F32_BK) {
    // each thread loads one element of each tile: (ty, tx) -> a[row_tile + ty][k0 + tx], w[col_tile + ty][k0 + tx]
    unsigned ar = blockIdx.y * F32_TILE + ty, wr = blockIdx.x * F32_TILE + ty, kk = k0 + tx;
    as[ty][tx] = (ar < m && kk < k) ? a[static_cast<size_t>(ar) * lda + kk] : 0.0f;
    ws[ty][tx] = (wr < n && kk < k) ? w[static_cast<size_t>(wr) * ldw + kk] : 0.0f;
    __syncthreads();
    const unsigned lim = min(static_cast<unsigned>(F32_BK), k - k0);
    for (unsigned i = 0; i < lim; ++i) sum = __fadd_rn(sum, __fmul_rn(as[ty][i], ws[tx][i]));
    __syncthreads();
  }
  if (row < m && col < n) store_from_f32(c, c_dt, static_cast<size_t>(row) * ldc + col, sum);
}

// ---------------------------------------------------------------------------------------------
// 16-bit tensor-core GEMM (mma.sync), NT
// ---------------------------------------------------------------------------------------------

constexpr int BM = 128, BK = 64, GEMM_THREADS = 256;
// cp.async pipeline depth: decode-sized grids leave one CTA per SM, so the tile stream itself has
// to keep enough bytes in flight (BN 64: 6 x 24 KB, BN 128: 4 x 32 KB).
template <int BN> constexpr int kPipelineDepth = BN == 128 ? 4 : 6;

__device__ inline void cp_async_16(unsigned smem_addr, const void* gmem, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ inline void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ inline void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <bool kBF16>
__device__ inline void mma_16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  if (kBF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

struct GemmParams {
  const unsigned short* a; size_t lda;
  const unsigned short* w; size_t ldw;
  void* c; int c_dt; size_t ldc;
  unsigned m, n, k;
  unsigned splits, k_per_split;   // k_per_split is a multiple of BK
  float* partial;                 // [splits][m][n] when splits > 1
  unsigned* counters;             // [tiles]
};

template <int BN, bool kBF16>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_nt_mma_kernel(GemmParams p) {
  constexpr int WARPS_N = BN == 128 ? 4 : 2;
  constexpr int WARPS_M = 8 / WARPS_N;
  constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
  constexpr int MT = WM / 16, NT = WN / 8;
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ unsigned s_ticket;
  pdl_sync();
  const unsigned smem_base = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp % WARPS_N;
  const unsigned row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  const unsigned k_begin = blockIdx.z * p.k_per_split;
  const unsigned k_end = min(p.k, k_begin + p.k_per_split);
  const unsigned k_iters = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

  auto issue = [&](unsigned it) {
    if (it < k_iters) {
      const unsigned stage = smem_base + (it % kPipelineDepth<BN>) * STAGE_BYTES;
      const unsigned kk = k_begin + it * BK;
      // A tile: BM rows x 8 chunks; W tile: BN rows x 8 chunks (16 B = 8 elements each)
#pragma unroll
      for (int i = 0; i < (BM * 8) / GEMM_THREADS; ++i) {
        const unsigned chunk = threadIdx.x + i * GEMM_THREADS, r = chunk >> 3, c8 = chunk & 7;
        const unsigned gk = kk + c8 * 8;
        const bool ok = (row0 + r < p.m) && (gk + 8 <= k_end);
        const void* src = ok ? static_cast<const void*>(p.a + static_cast<size_t>(row0 + r) * p.lda + gk) : static_cast<const void*>(p.a);
        cp_async_16(stage + r * 128 + ((c8 ^ (r & 7)) << 4), src, ok ? 16u : 0u);
      }
#pragma unroll
      for (int i = 0; i < (BN * 8) / GEMM_THREADS; ++i) {
        const unsigned chunk = threadIdx.x + i * GEMM_THREADS, r = chunk >> 3, c8 = chunk & 7;
        const unsigned gk = kk + c8 * 8;
        const bool ok = (col0 + r < p.n) && (gk + 8 <= k_end);
        const void* src = ok ? static_cast<const void*>(p.w + static_cast<size_t>(col0 + r) * p.ldw + gk) : static_cast<const void*>(p.w);
        cp_async_16(stage + A_BYTES + r * 128 + ((c8 ^ (r & 7)) << 4), src, ok ? 16u : 0u);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < kPipelineDepth<BN> - 1; ++s) issue(s);

  for (unsigned it = 0; it < k_iters; ++it) {
    cp_async_wait<kPipelineDepth<BN> - 2>();
    __syncthreads();  // stage `it` has landed for every thread; stage it-1 is free for refill
    issue(it + kPipelineDepth<BN> - 1);
    const unsigned stage = smem_base + (it % kPipelineDepth<BN>) * STAGE_BYTES;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      unsigned af[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        // A fragment: matrices (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi)
        const unsigned mi = lane >> 3, rr = lane & 7;
        const unsigned r = warp_m * WM + i * 16 + (mi & 1) * 8 + rr;
        const unsigned chunk = ks * 2 + (mi >> 1);
        ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], stage + r * 128 + ((chunk ^ (r & 7)) << 4));
      }
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        // B fragments for two n-tiles: (n 0-7, k lo), (n 0-7, k hi), (n 8-15, k lo), (n 8-15, k hi)
        const unsigned mi = lane >> 3, rr = lane & 7;
        const unsigned r = warp_n * WN + j * 8 + (mi >> 1) * 8 + rr;
        const unsigned chunk = ks * 2 + (mi & 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, stage + A_BYTES + r * 128 + ((chunk ^ (r & 7)) << 4));
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          mma_16816<kBF16>(acc[i][j], af[i], b0, b1);
          mma_16816<kBF16>(acc[i][j + 1], af[i], b2, b3);
        }
      }
    }
  }
  cp_async_wait<0>();

  const unsigned gr = lane >> 2, gc = (lane & 3) * 2;
  if (p.splits == 1) {
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
          const unsigned r = row0 + warp_m * WM + i * 16 + gr + (e >> 1) * 8;
          const unsigned c = col0 + warp_n * WN + j * 8 + gc;
          if (r >= p.m) continue;
          const size_t off = static_cast<size_t>(r) * p.ldc + c;
          if (c + 1 < p.n && p.c_dt != F32 && (p.ldc & 1) == 0 && (reinterpret_cast<size_t>(p.c) & 3) == 0) {
            unsigned packed;
            if (p.c_dt == BF16) { __nv_bfloat162 v = __floats2bfloat162_rn(acc[i][j][e], acc[i][j][e + 1]); packed = *reinterpret_cast<unsigned*>(&v); }
            else { __half2 v = __floats2half2_rn(acc[i][j][e], acc[i][j][e + 1]); packed = *reinterpret_cast<unsigned*>(&v); }
            *reinterpret_cast<unsigned*>(static_cast<unsigned short*>(p.c) + off) = packed;
          } else {
            if (c < p.n) store_from_f32(p.c, p.c_dt, off, acc[i][j][e]);
            if (c + 1 < p.n) store_from_f32(p.c, p.c_dt, off + 1, acc[i][j][e + 1]);
          }
        }
    return;
  }
  // split-K: write the f32 partial, last CTA of the tile sums the splits in split order
  float* mine = p.partial + static_cast<size_t>(blockIdx.z) * p.m * p.n;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const unsigned r = row0 + warp_m * WM + i * 16 + gr + (e >> 1) * 8;
        const unsigned c = col0 + warp_n * WN + j * 8 + gc;
        if (r < p.m && c + 1 < p.n && (p.n & 1) == 0) {
          *reinterpret_cast<float2*>(mine + static_cast<size_t>(r) * p.n + c) = make_float2(acc[i][j][e], acc[i][j][e + 1]);
        } else if (r < p.m) {
          if (c < p.n) mine[static_cast<size_t>(r) * p.n + c] = acc[i][j][e];
          if (c + 1 < p.n) mine[static_cast<size_t>(r) * p.n + c + 1] = acc[i][j][e + 1];
        }
      }
  __threadfence();
  __syncthreads();
  const unsigned tile = blockIdx.y * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) s_ticket = atomicAdd(&p.counters[tile], 1u);
  __syncthreads();
  if (s_ticket != p.splits - 1) return;
  __threadfence();
  const bool vec4 = (p.n % 4 == 0) && (p.ldc % 4 == 0) && (reinterpret_cast<size_t>(p.c) % 8 == 0) && p.c_dt != F32;
  if (vec4) {
    // four columns per thread, all splits' loads of an element group issued back to back
    for (unsigned idx = threadIdx.x; idx < BM * (BN / 4); idx += GEMM_THREADS) {
      const unsigned r = row0 + idx / (BN / 4), c = col0 + (idx % (BN / 4)) * 4;
      if (r < p.m && c < p.n) {
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
        for (unsigned s = 0; s < p.splits; ++s) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(p.partial + (static_cast<size_t>(s) * p.m + r) * p.n + c));
          sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        unsigned short h[4];
        if (p.c_dt == BF16) {
          h[0] = __bfloat16_as_ushort(__float2bfloat16_rn(sum.x)); h[1] = __bfloat16_as_ushort(__float2bfloat16_rn(sum.y));
          h[2] = __bfloat16_as_ushort(__float2bfloat16_rn(sum.z)); h[3] = __bfloat16_as_ushort(__float2bfloat16_rn(sum.w));
        } else {
          h[0] = __half_as_ushort(__float2half_rn(sum.x)); h[1] = __half_as_ushort(__float2half_rn(sum.y));
          h[2] = __half_as_ushort(__float2half_rn(sum.z)); h[3] = __half_as_ushort(__float2half_rn(sum.w));
        }
        uint2 packed = make_uint2(h[0] | (static_cast<unsigned>(h[1]) << 16), h[2] | (static_cast<unsigned>(h[3]) << 16));
        *reinterpret_cast<uint2*>(static_cast<unsigned short*>(p.c) + static_cast<size_t>(r) * p.ldc + c) = packed;
      }
    }
  } else {
    for (unsigned idx = threadIdx.x; idx < BM * BN; idx += GEMM_THREADS) {
      const unsigned r = row0 + idx / BN, c = col0 + idx % BN;
      if (r < p.m && c < p.n) {
        float sum = 0.0f;
        for (unsigned s = 0; s < p.splits; ++s) sum += __ldcg(p.partial + (static_cast<size_t>(s) * p.m + r) * p.n + c);
        store_from_f32(p.c, p.c_dt, static_cast<size_t>(r) * p.ldc + c, sum);
      }
    }
  }
  if (threadIdx.x == 0) p.counters[tile] = 0;
}

__global__ void matmul_generic_kernel(View a, View b, View c, unsigned batch, unsigned m, unsigned n, unsigned k) {
  const size_t total = static_cast<size_t>(batch) * m * n;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t bi = idx / (static_cast<size_t>(m) * n);
    const unsigned r = static_cast<unsigned>((idx / n) % m), col = static_cast<unsigned>(idx % n);
    float sum = 0.0f;
    for (unsigned kk = 0; kk < k; ++kk) {
      float x = load_as_f32(a.base, a.dtype, view_offset(a, (bi * m + r) * k + kk));
      float y = load_as_f32(b.base, b.dtype, view_offset(b, (bi * k + kk) * n + col));
      sum = __fadd_rn(sum, __fmul_rn(x, y));
    }
    store_from_f32(c.base, c.dtype, view_offset(c, idx), sum);
  }
}

struct SplitPlan { unsigned bn, splits, k_per_split, tiles; };

SplitPlan plan_gemm(unsigned m, unsigned n, unsigned k, int sm_count) {
  SplitPlan s;
  // Wide tiles only when they alone fill the GPU (lm_head); otherwise BN 64 gives twice the CTAs.
  unsigned tiles_m = (m + BM - 1) / BM;
  s.bn = (tiles_m * ((n + 127) / 128) >= 2u * static_cast<unsigned>(sm_count)) ? 128 : 64;
  unsigned tiles_n = (n + s.bn - 1) / s.bn;
  s.tiles = tiles_m * tiles_n;
  unsigned k_iters = (k + BK - 1) / BK;
  unsigned splits = 1;
  // Split K only for grids that would leave most SMs idle: every split costs an f32 partial
  // round trip and a serial reduction by the last CTA of the tile.
  // (measured on the decode projections, 128 rows: asking for more CTAs or allowing shorter splits only adds time -
  // 14.7 -> 16-24 us for 1024 x 4096 - the tile's own tensor-core work and the reduction, not the weight stream, set the pace)
  const unsigned want_ctas = static_cast<unsigned>(sm_count) / 2;
  if (s.tiles < want_ctas) {
    splits = (want_ctas + s.tiles - 1) / s.tiles;
    unsigned max_by_k = k_iters / 8;  // at least 8 k-iterations per split
    if (splits > max_by_k) splits = max_by_k;
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
  }
  unsigned iters_per = (k_iters + splits - 1) / splits;
  s.k_per_split = iters_per * BK;
  s.splits = (k_iters + iters_per - 1) / iters_per;
  return s;
}

template <int BN, bool kBF16>
void run_mma(Ctx& ctx, const GemmParams& p, unsigned tiles_m, unsigned tiles_n) {
  constexpr int smem = kPipelineDepth<BN> * (BM * BK * 2 + BN * BK * 2);
  static SmemOptIn opted;
  opt_in_smem(opted, gemm_nt_mma_kernel<BN, kBF16>, smem);
  launch_pdl(gemm_nt_mma_kernel<BN, kBF16>, dim3(tiles_n, tiles_m, p.splits), dim3(GEMM_THREADS), smem, ctx.stream, p);
  ctx.launches++;
}

}  // namespace

size_t gemm_scratch_bytes(unsigned m, unsigned n, unsigned k) {
  // f32 partials for up to 16 splits + one counter per tile (tiles <= sm_count when splitting)
  return static_cast<size_t>(16) * m * n * sizeof(float) + 4096 * sizeof(unsigned);
}

void launch_gemm_nt(Ctx& ctx, const void* a, int a_dt, size_t lda, const void* w, int w_dt, size_t ldw, void* c, int c_dt,
                    size_t ldc, unsigned m, unsigned n, unsigned k, void* scratch, size_t scratch_bytes) {
  if (m == 0 || n == 0) return;
  if (a_dt == F32) {
    dim3 grid((n + F32_TILE - 1) / F32_TILE, (m + F32_TILE - 1) / F32_TILE);
    gemm_nt_f32_kernel<<<grid, F32_TILE * F32_TILE, 0, ctx.stream>>>(static_cast<const float*>(a), lda, static_cast<const float*>(w), ldw, c, c_dt, ldc, m, n, k);
    ctx.launches++;
    return;
  }
  const bool aligned = (k % 8 == 0) && (lda % 8 == 0) && (ldw % 8 == 0) && ((reinterpret_cast<size_t>(a) | reinterpret_cast<size_t>(w)) % 16 == 0);
  if (m <= 16 || !aligned) {
    for (unsigned r0 = 0; r0 < m; r0 += 16) {
      unsigned rows = min(16u, m - r0);
      unsigned blocks = (n + 7) / 8;
      const char* ap = static_cast<const char*>(a) + static_cast<size_t>(r0) * lda * 2;
      char* cp = static_cast<char*>(c) + static_cast<size_t>(r0) * ldc * dtype_size(c_dt);
      if (a_dt == BF16)
        gemv_nt_kernel<__nv_bfloat16, 16><<<blocks, 256, 0, ctx.stream>>>(reinterpret_cast<const __nv_bfloat16*>(ap), lda, static_cast<const __nv_bfloat16*>(w), ldw, cp, c_dt, ldc, rows, n, k);
      else
        gemv_nt_kernel<__half, 16><<<blocks, 256, 0, ctx.stream>>>(reinterpret_cast<const __half*>(ap), lda, static_cast<const __half*>(w), ldw, cp, c_dt, ldc, rows, n, k);
      ctx.launches++;
    }
    return;
  }
  // 17 rows or more: the TMA-fed tcgen05 kernel (TMEM accumulators; 128 x 32..256 tiles chosen from the grid it gives).
  // Measured against the mma.sync split-K kernel below on the 128-row decode projections: 1024 x 4096 in 7.6 us instead of
  // 14.7, 1024 x 6144 in 8.5 instead of 12.0, 2048 x 1024 in 11.5 instead of 13.4; 4096^3 at 1343 TFLOP/s.
  if (gemm_nt_tma_supported(a_dt, w_dt, m, n, k, lda, ldw, a, w) && launch_gemm_nt_tma(ctx, a, a_dt, lda, w, ldw, c, c_dt, ldc, m, n, k)) return;
  SplitPlan plan = plan_gemm(m, n, k, ctx.sm_count);
  const size_t need = static_cast<size_t>(plan.splits) * m * n * sizeof(float) + static_cast<size_t>(plan.tiles) * sizeof(unsigned);
  if (plan.splits > 1 && (scratch == nullptr || scratch_bytes < need || plan.tiles > 4096)) {
    plan.splits = 1;
    plan.k_per_split = ((k + BK - 1) / BK) * BK;
  }
  GemmParams p;
  p.a = static_cast<const unsigned short*>(a); p.lda = lda;
  p.w = static_cast<const unsigned short*>(w); p.ldw = ldw;
  p.c = c; p.c_dt = c_dt; p.ldc = ldc; p.m = m; p.n = n; p.k = k;
  p.splits = plan.splits; p.k_per_split = plan.k_per_split;
  // counters live at the start of the scratch (zero on first use, kernels leave them zero)
  p.counters = static_cast<unsigned*>(scratch);
  p.partial = scratch ? reinterpret_cast<float*>(static_cast<char*>(scratch) + 4096 * sizeof(unsigned)) : nullptr;
  unsigned tiles_m = (m + BM - 1) / BM, tiles_n = (n + plan.bn - 1) / plan.bn;
  const bool bf16 = a_dt == BF16;
  if (plan.bn == 128) { if (bf16) run_mma<128, true>(ctx, p, tiles_m, tiles_n); else run_mma<128, false>(ctx, p, tiles_m, tiles_n); }
  else { if (bf16) run_mma<64, true>(ctx, p, tiles_m, tiles_n); else run_mma<64, false>(ctx, p, tiles_m, tiles_n); }
}

void launch_matmul_generic(Ctx& ctx, const View& a, const View& b, const View& c, unsigned batch, unsigned m, unsigned n,
                           unsigned k) {
  size_t total = static_cast<size_t>(batch) * m * n;
  if (total == 0) return;
  size_t blocks = (total + 255) / 256;
  if (blocks > 65535u * 16) blocks = 65535u * 16;
  matmul_generic_kernel<<<static_cast<unsigned>(blocks), 256, 0, ctx.stream>>>(a, b, c, batch, m, n, k);
  ctx.launches++;
}

}  // namespace fj
