// Dense 16-bit GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T ("NT", both
// operands K-major), f32 accumulation in tensor memory, output rounded once (reference operator:
// Op::Matmul, crates/forja-cpu/src/lib.rs:815-848; used here for prefill-sized projections and
// for the dequantised-slab path of Op::QuantMatmul).
//
// One CTA owns a 128 x 128 output tile. Operand tiles of 128 rows x 64 k (128 bytes per row) are
// copied with cp.async into shared memory in the 128-byte-swizzle layout the tensor core expects
// for K-major operands (16-byte chunk c of row r at chunk c ^ (r & 7), 8-row groups 1024 bytes
// apart), three stages deep with two CTAs per SM. When a stage has landed, one elected thread issues four
// tcgen05.mma.cta_group::1.kind::f16 (M 128, N 128, K 16 each) whose accumulator is a 128-lane x
// 128-column f32 block of TMEM, then tcgen05.commit arrives on that stage's mbarrier once the
// tensor core is done reading it, which is what lets the stage be refilled. After the last k step
// a final commit signals the epilogue: each of the four warps reads its 32 TMEM lanes (= 32 rows)
// with tcgen05.ld, 32 columns at a time, rounds and stores rows of 64 bytes.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the kernel records the give-up in a
// device counter, skips the rest of its work, frees its tensor memory and returns.
#include "fj_kernels.h"

namespace fj {

namespace {

constexpr int T5_BM = 128, T5_BN = 128, T5_BK = 64, T5_STAGES = 3, T5_THREADS = 128;  // 3 stages = 97 KB: two CTAs per SM
constexpr int T5_TILE_BYTES = 128 * 128;                       // 128 rows x 128 bytes
constexpr int T5_STAGE_BYTES = 2 * T5_TILE_BYTES;              // A then W
constexpr int T5_SMEM = T5_STAGES * T5_STAGE_BYTES + 1024;     // + slack to align the base to 1024 bytes
constexpr unsigned kSpinLimit = 1u << 24;

__device__ unsigned g_tc5_giveups = 0;

__device__ inline void t5_cp_async_16(unsigned smem_addr, const void* gmem, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void mbar_init(unsigned addr, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count) : "memory"); }
// Polls until the phase with the given parity has completed; false when the limit ran out.
__device__ inline bool mbar_wait(unsigned addr, unsigned parity) {
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// K-major operand tile in the 128-byte swizzle: start address, 8-row group stride 1024 bytes,
// descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ inline unsigned long long smem_desc(unsigned smem_addr) {
  unsigned long long d = 0;
  d |= static_cast<unsigned long long>((smem_addr & 0x3FFFFu) >> 4);         // bits 0-13: address >> 4
  d |= static_cast<unsigned long long>(1) << 16;                              // bits 16-29: leading byte offset (unused for swizzled K-major)
  d |= static_cast<unsigned long long>(1024 >> 4) << 32;                      // bits 32-45: stride byte offset >> 4
  d |= static_cast<unsigned long long>(1) << 46;                              // bits 46-47: descriptor version
  d |= static_cast<unsigned long long>(2) << 61;                              // bits 61-63: 128-byte swizzle
  return d;
}
// kind::f16 instruction descriptor: D f32, A and B of the given 16-bit format, both K-major, N 128, M 128.
__device__ inline unsigned instr_desc(bool bf16) {
  const unsigned fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<unsigned>(T5_BN >> 3) << 17) | (static_cast<unsigned>(T5_BM >> 4) << 24);
}

struct Tc5Params {
  const unsigned short* a; size_t lda;
  const unsigned short* w; size_t ldw;
  void* c; int c_dt; size_t ldc;
  unsigned m, n, k;
  int bf16;
};

__global__ void __launch_bounds__(T5_THREADS, 2) gemm_nt_tcgen05_kernel(Tc5Params p) {
  extern __shared__ unsigned char t5_smem_raw[];
  __shared__ __align__(8) unsigned long long s_bar[T5_STAGES + 1];  // stage released by the tensor core; [STAGES]: all MMAs done
  __shared__ unsigned s_tmem;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned row0 = blockIdx.y * T5_BM, col0 = blockIdx.x * T5_BN;
  const unsigned k_iters = p.k / T5_BK;
  const unsigned raw = static_cast<unsigned>(__cvta_generic_to_shared(t5_smem_raw));
  const unsigned smem_base = (raw + 1023u) & ~1023u;
  const unsigned bar_base = static_cast<unsigned>(__cvta_generic_to_shared(&s_bar[0]));

  if (threadIdx.x == 0) {
    for (int i = 0; i <= T5_STAGES; ++i) mbar_init(bar_base + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(&s_tmem));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst), "r"(static_cast<unsigned>(T5_BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem = s_tmem;
  pdl_sync();  // barriers and tensor memory are set up while the previous kernel drains; its results are read from here on

  auto issue_loads = [&](unsigned it) {
    if (it < k_iters) {
      const unsigned stage = smem_base + (it % T5_STAGES) * T5_STAGE_BYTES;
      const unsigned kk = it * T5_BK;
#pragma unroll
      for (int i = 0; i < (T5_BM * 8) / T5_THREADS; ++i) {
        const unsigned chunk = threadIdx.x + i * T5_THREADS, r = chunk >> 3, c8 = chunk & 7;
        const bool ok = row0 + r < p.m;
        const void* src = ok ? static_cast<const void*>(p.a + static_cast<size_t>(row0 + r) * p.lda + kk + c8 * 8) : static_cast<const void*>(p.a);
        t5_cp_async_16(stage + r * 128 + ((c8 ^ (r & 7)) << 4), src, ok ? 16u : 0u);
      }
#pragma unroll
      for (int i = 0; i < (T5_BN * 8) / T5_THREADS; ++i) {
        const unsigned chunk = threadIdx.x + i * T5_THREADS, r = chunk >> 3, c8 = chunk & 7;
        const bool ok = col0 + r < p.n;
        const void* src = ok ? static_cast<const void*>(p.w + static_cast<size_t>(col0 + r) * p.ldw + kk + c8 * 8) : static_cast<const void*>(p.w);
        t5_cp_async_16(stage + T5_TILE_BYTES + r * 128 + ((c8 ^ (r & 7)) << 4), src, ok ? 16u : 0u);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

#pragma unroll
  for (int s = 0; s < T5_STAGES - 1; ++s) issue_loads(s);

  const unsigned idesc = instr_desc(p.bf16 != 0);
  bool failed = false;
  for (unsigned it = 0; it < k_iters; ++it) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(T5_STAGES - 2) : "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // cp.async wrote through the generic proxy; the tensor core reads through the async proxy
    if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }  // stage `it` has landed for every thread
    if (threadIdx.x == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const unsigned stage = smem_base + (it % T5_STAGES) * T5_STAGE_BYTES;
      const unsigned long long a_desc = smem_desc(stage), b_desc = smem_desc(stage + T5_TILE_BYTES);
#pragma unroll
      for (int ks = 0; ks < T5_BK / 16; ++ks) {
        // 16 k = 32 bytes further along the swizzled row: +2 in the descriptor's 16-byte address units
        const unsigned accumulate = (it != 0 || ks != 0) ? 1u : 0u;
        asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem), "l"(a_desc + 2ull * ks),
                     "l"(b_desc + 2ull * ks), "r"(idesc), "r"(accumulate)
                     : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_base + 8 * (it % T5_STAGES)) : "memory");
      if (it + 1 == k_iters) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_base + 8 * T5_STAGES) : "memory");
    }
    // With this step's MMAs queued, refill the stage the previous step read, once the tensor core has released it.
    if (it >= 1) {
      const unsigned prev = it - 1;
      if (!mbar_wait(bar_base + 8 * (prev % T5_STAGES), (prev / T5_STAGES) & 1u)) failed = true;
    }
    if (!failed) issue_loads(it + T5_STAGES - 1);
    else asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  if (!failed && k_iters != 0 && !mbar_wait(bar_base + 8 * T5_STAGES, 0)) failed = true;
  if (__syncthreads_or(failed ? 1 : 0)) {
    failed = true;
    if (threadIdx.x == 0) atomicAdd(&g_tc5_giveups, 1u);
  }
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  if (!failed) {
    // warp w owns TMEM lanes 32 w .. 32 w + 31 = rows; 32 columns per load
    const unsigned row = row0 + warp * 32 + lane;
#pragma unroll 1
    for (int cb = 0; cb < T5_BN / 32; ++cb) {
      unsigned v[32];
      const unsigned taddr = tmem + (static_cast<unsigned>(warp * 32) << 16) + cb * 32;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
            "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
            "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      if (row < p.m) {
        const unsigned c_first = col0 + cb * 32;
        const size_t base = static_cast<size_t>(row) * p.ldc + c_first;
        if (p.c_dt != F32 && c_first + 32 <= p.n && base % 8 == 0 && reinterpret_cast<size_t>(p.c) % 16 == 0) {
          // 32 columns of one row = 64 bytes: four 16-byte stores
          unsigned short* dst = static_cast<unsigned short*>(p.c) + base;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            unsigned packed[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lo = __uint_as_float(v[q * 8 + 2 * j]), hi = __uint_as_float(v[q * 8 + 2 * j + 1]);
              if (p.c_dt == BF16) {
                __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
                packed[j] = *reinterpret_cast<unsigned*>(&t);
              } else {
                __half2 t = __floats2half2_rn(lo, hi);
                packed[j] = *reinterpret_cast<unsigned*>(&t);
              }
            }
            *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c_first + j < p.n) store_from_f32(p.c, p.c_dt, base + j, __uint_as_float(v[j]));
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(static_cast<unsigned>(T5_BN)) : "memory");
}

}  // namespace

bool gemm_nt_tcgen05_supported(int a_dt, int w_dt, unsigned m, unsigned n, unsigned k, size_t lda, size_t ldw, const void* a, const void* w) {
  return (a_dt == BF16 || a_dt == F16) && a_dt == w_dt && m >= 64 && n >= 64 && k >= T5_BK && k % T5_BK == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
         (reinterpret_cast<size_t>(a) | reinterpret_cast<size_t>(w)) % 16 == 0;
}

void launch_gemm_nt_tcgen05(Ctx& ctx, const void* a, int a_dt, size_t lda, const void* w, size_t ldw, void* c, int c_dt, size_t ldc, unsigned m, unsigned n, unsigned k) {
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    cudaFuncSetAttribute(gemm_nt_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T5_SMEM);
    configured[device] = true;
  }
  Tc5Params p{static_cast<const unsigned short*>(a), lda, static_cast<const unsigned short*>(w), ldw, c, c_dt, ldc, m, n, k, a_dt == BF16 ? 1 : 0};
  dim3 grid((n + T5_BN - 1) / T5_BN, (m + T5_BM - 1) / T5_BM);
  launch_pdl(gemm_nt_tcgen05_kernel, grid, dim3(T5_THREADS), T5_SMEM, ctx.stream, p);
  ctx.launches++;
}

unsigned gemm_tcgen05_giveups() {
  unsigned value = 0;
  cudaMemcpyFromSymbol(&value, g_tc5_giveups, sizeof(value));
  return value;
}

}  // namespace fj
