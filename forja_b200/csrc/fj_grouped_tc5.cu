// Expert-bucketed q4 projections for prefill-sized route counts on the 5th-generation tensor cores
// (operator: Op::GatherQuantMatmul, crates/forja-cpu/src/lib.rs:964-1204; the reference's sorted MoE
// path is crates/forja-metal/kernels/quant_matmul.metal:1217-1615).
//
// One CTA owns a route tile (up to 128 rows of one expert) x 64 output columns, for the gate and up
// matrices together in pair mode. Per 64-k step (= one quantisation group):
//  * 256 producer threads copy, with cp.async and two steps ahead, the 128 gathered activation rows
//    into shared memory in the 128-byte-swizzle K-major layout, and each its own 8 bytes of nibbles
//    per matrix (column c = thread / 4, quarter of the step = thread % 4) into a private slot; the
//    column's scale and bias travel in registers, fetched one step ahead;
//  * each producer expands its nibbles to bf16 (pairs of nibbles OR-ed into the mantissa of bf16
//    128.0, minus 128, one bf16x2 fma = bf16(s * q + b) with a single rounding) straight into the
//    swizzled B tile of the step's stage and arrives on the stage's "filled" mbarrier: no CTA-wide
//    barrier in the loop, warps may run up to two steps apart;
//  * the elected thread of a ninth warp waits for "filled", issues tcgen05.mma.cta_group::1.kind::f16
//    (M 128, N 64, K 16, four per matrix) into f32 accumulators in tensor memory (64 columns per
//    matrix) and commits to the step's "done" mbarrier; a producer starts step it once the MMAs
//    of step it - 2 are done (4 A slots, 2 B slots), so the tensor core always has a step queued.
// Epilogue: the eight producer warps read their TMEM lanes (warp % 4 selects the 32 rows, warp / 4 the 32
// columns) with tcgen05.ld; pair mode stores silu(gate) * up as bf16, single mode f32 or bf16 rows,
// scattered to out[route].
// Every mbarrier wait is bounded; a wait that runs out is counted, the CTA skips its output, frees
// its tensor memory and returns.
#include "fj_grouped.cuh"

namespace fj {

namespace {

constexpr int G5_BM = 128, G5_BN = 64, G5_BK = 64, G5_PRODUCERS = 256, G5_THREADS = G5_PRODUCERS + 32;
// Copies run two steps ahead of their use; a producer may start step it once the MMAs of step it - 2 are done, which frees
// A slot (it + 2) % 4 and B slot it % 2. The nibble slots are private to a thread (3: two in flight, one being read).
constexpr int G5_A_STAGES = 4, G5_B_STAGES = 2, G5_RAW_STAGES = 3, G5_AHEAD = 2;
constexpr int G5_A_BYTES = G5_BM * 128, G5_B_BYTES = G5_BN * 128, G5_RAW_BYTES = G5_BN * 32;
constexpr unsigned kG5SpinLimit = 1u << 24;

__device__ unsigned g_grouped_tc5_giveups = 0;

// kPair: gate and up matrices, 64 columns each. kWide (single matrix only): 128 columns, handled as two 64-column halves
// so that a CTA reads its 128 activation rows once for twice the output.
template <bool kPair, bool kWide>
struct G5Layout {
  static constexpr int NW = (kPair || kWide) ? 2 : 1;
  static constexpr int B = G5_A_STAGES * G5_A_BYTES;                       // [A_STAGES] A tiles, then [B_STAGES][NW] expanded B tiles; all 1024-byte aligned
  static constexpr int RAW = B + G5_B_STAGES * NW * G5_B_BYTES;            // [RAW_STAGES][NW][256 threads x 8 B] nibbles, private to the thread that copied them
  static constexpr int ROUTES = RAW + G5_RAW_STAGES * NW * G5_RAW_BYTES;   // [128] route ids
  static constexpr int TOTAL = ROUTES + G5_BM * 4 + 1024;                  // + slack to align the base to 1024 bytes
};

__device__ inline void g5_cp_async_16(unsigned smem_addr, const void* gmem, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void g5_cp_async_8(unsigned smem_addr, const void* gmem, unsigned src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void g5_mbar_init(unsigned addr, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count) : "memory"); }
// Polls until the phase with the given parity has completed; false when the limit ran out or another thread of the CTA gave up.
__device__ inline bool g5_mbar_wait(unsigned addr, unsigned parity, volatile int* gave_up) {
  for (unsigned spin = 0; spin < kG5SpinLimit; ++spin) {
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 1023u) == 1023u && *gave_up != 0) return false;
  }
  return false;
}
// K-major operand tile in the 128-byte swizzle: start address, 8-row group stride 1024 bytes, descriptor version 1, SWIZZLE_128B.
__device__ inline unsigned long long g5_smem_desc(unsigned smem_addr) {
  unsigned long long d = 0;
  d |= static_cast<unsigned long long>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<unsigned long long>(1) << 16;
  d |= static_cast<unsigned long long>(1024 >> 4) << 32;
  d |= static_cast<unsigned long long>(1) << 46;
  d |= static_cast<unsigned long long>(2) << 61;
  return d;
}
// kind::f16: D f32, A and B bf16, both K-major, N 64, M 128.
__device__ inline unsigned g5_instr_desc() { return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<unsigned>(G5_BN >> 3) << 17) | (static_cast<unsigned>(G5_BM >> 4) << 24); }

__device__ inline void g5_tmem_load32(unsigned taddr, unsigned (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]),
        "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

template <bool kPair, bool kWide>
__global__ void __launch_bounds__(G5_THREADS, 2) grouped_q4_tc5_kernel(GroupedArgs p) {
  using L = G5Layout<kPair, kWide>;
  constexpr int NW = L::NW;
  constexpr unsigned TMEM_COLS = NW * G5_BN;
  extern __shared__ unsigned char g5_smem_raw[];
  __shared__ __align__(8) unsigned long long s_bar[2 * G5_B_STAGES + 1];  // [0, 2): step filled by the 256 producers; [2, 4): step's MMAs done; [4]: all MMAs done
  __shared__ unsigned s_tmem;
  __shared__ volatile int s_failed;
  pdl_sync();  // the route plan and the rows come from the kernels before
  if (blockIdx.y >= *p.n_tiles) return;
  const RouteTile tile = p.tiles[blockIdx.y];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned col0 = blockIdx.x * (kWide ? 2 * G5_BN : G5_BN);
  const unsigned k_iters = p.k / G5_BK, words_per_row = p.k / 8, groups_per_row = p.k / 64;
  const unsigned raw_addr = static_cast<unsigned>(__cvta_generic_to_shared(g5_smem_raw));
  const unsigned smem_base = (raw_addr + 1023u) & ~1023u;
  unsigned char* smem = g5_smem_raw + (smem_base - raw_addr);
  const unsigned bar_base = static_cast<unsigned>(__cvta_generic_to_shared(&s_bar[0]));
  unsigned* s_route = reinterpret_cast<unsigned*>(smem + L::ROUTES);

  if (threadIdx.x == 0) {
    for (int i = 0; i < G5_B_STAGES; ++i) g5_mbar_init(bar_base + 8 * i, G5_PRODUCERS);
    for (int i = G5_B_STAGES; i <= 2 * G5_B_STAGES; ++i) g5_mbar_init(bar_base + 8 * i, 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(&s_tmem));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  for (unsigned i = threadIdx.x; i < G5_BM; i += G5_THREADS) s_route[i] = i < tile.count ? p.sorted[tile.first + i] : 0xFFFFFFFFu;
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem = s_tmem;
  const size_t expert_rows = static_cast<size_t>(tile.expert) * p.n;

  const bool producer = threadIdx.x < G5_PRODUCERS;
  bool failed = false;
  if (producer) {
    // this thread's four A chunks per stage: rows r, r + 32, r + 64, r + 96, 16-byte chunk a_c8
    const unsigned a_c8 = threadIdx.x & 7;
    const unsigned short* a_src[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const unsigned route = s_route[(threadIdx.x >> 3) + i * (G5_PRODUCERS / 8)];
      a_src[i] = route != 0xFFFFFFFFu ? p.x + static_cast<size_t>(route / p.src_div) * p.k + a_c8 * 8 : nullptr;
    }
    // ... and its own slice of the weights: column c, quarter `part` of every 64-k step (8 bytes of nibbles per matrix)
    const unsigned c = threadIdx.x >> 2, part = threadIdx.x & 3;
    bool col_ok[NW];
    size_t w_row[NW];
    const unsigned* w_packed[NW];
    const unsigned short *w_scales[NW], *w_biases[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const unsigned col = col0 + (kWide ? w * G5_BN : 0) + c;
      col_ok[w] = col < p.n;
      w_row[w] = expert_rows + (col_ok[w] ? col : 0);
      w_packed[w] = p.packed[kPair ? w : 0];
      w_scales[w] = p.scales[kPair ? w : 0];
      w_biases[w] = p.biases[kPair ? w : 0];
    }
    const unsigned own = threadIdx.x * 8;  // byte offset of this thread's private staging slot inside a stage's region

    auto issue_loads = [&](unsigned it) {
      if (it < k_iters) {
        const unsigned a_tile = smem_base + (it % G5_A_STAGES) * G5_A_BYTES, slot = it % G5_RAW_STAGES, kk = it * G5_BK;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const unsigned r = (threadIdx.x >> 3) + i * (G5_PRODUCERS / 8);
          const bool ok = a_src[i] != nullptr;
          g5_cp_async_16(a_tile + r * 128 + ((a_c8 ^ (r & 7)) << 4), ok ? static_cast<const void*>(a_src[i] + kk) : static_cast<const void*>(p.x), ok ? 16u : 0u);
        }
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          g5_cp_async_8(smem_base + L::RAW + (slot * NW + w) * (G5_PRODUCERS * 8) + own, w_packed[w] + w_row[w] * words_per_row + (kk / 8) + part * 2, col_ok[w] ? 8u : 0u);
        }
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

#pragma unroll
    for (int s = 0; s < G5_AHEAD; ++s) issue_loads(s);

    const unsigned offset_bits = 0x43004300u;
    const __nv_bfloat162 offset2 = *reinterpret_cast<const __nv_bfloat162*>(&offset_bits);
    // scale and bias of this thread's column travel in registers, fetched one step ahead
    unsigned sc_next[NW], bi_next[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      sc_next[w] = col_ok[w] && k_iters != 0 ? __ldg(w_scales[w] + w_row[w] * groups_per_row) : 0u;
      bi_next[w] = col_ok[w] && k_iters != 0 ? __ldg(w_biases[w] + w_row[w] * groups_per_row) : 0u;
    }
    for (unsigned it = 0; it < k_iters; ++it) {
      // A slot (it + 2) % 4 and B slot it % 2 were last read by the MMAs of step it - 2
      if (it >= 2) {
        const unsigned prev = it - 2;
        if (!g5_mbar_wait(bar_base + 8 * (G5_B_STAGES + prev % G5_B_STAGES), (prev / G5_B_STAGES) & 1u, &s_failed)) { failed = true; break; }
      }
      issue_loads(it + G5_AHEAD);
      unsigned sc_now[NW], bi_now[NW];
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        sc_now[w] = sc_next[w];
        bi_now[w] = bi_next[w];
        const bool more = col_ok[w] && it + 1 < k_iters;
        sc_next[w] = more ? __ldg(w_scales[w] + w_row[w] * groups_per_row + it + 1) : 0u;
        bi_next[w] = more ? __ldg(w_biases[w] + w_row[w] * groups_per_row + it + 1) : 0u;
      }
      asm volatile("cp.async.wait_group %0;\n" ::"n"(G5_AHEAD) : "memory");  // this thread's copies of step `it` have landed
      const unsigned slot = it % G5_RAW_STAGES, b_slot = it % G5_B_STAGES;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const unsigned sc = sc_now[w], bi = bi_now[w];
        const unsigned s2 = sc | (sc << 16), b2 = bi | (bi << 16);
        const __nv_bfloat162 scale2 = *reinterpret_cast<const __nv_bfloat162*>(&s2), bias2 = *reinterpret_cast<const __nv_bfloat162*>(&b2);
        const uint2 q = *reinterpret_cast<const uint2*>(smem + L::RAW + (slot * NW + w) * (G5_PRODUCERS * 8) + own);
        const unsigned words[2] = {q.x, q.y};
        unsigned char* b_tile = smem + L::B + (b_slot * NW + w) * G5_B_BYTES;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          unsigned r[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const unsigned pair_bits = ((words[i] >> (4 * j)) & 0x000F000Fu) | 0x43004300u;  // {128 + nibble j, 128 + nibble j + 4}
            const __nv_bfloat162 value = __hfma2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pair_bits), offset2), scale2, bias2);
            r[j] = *reinterpret_cast<const unsigned*>(&value);
          }
          const unsigned chunk = part * 2 + i;
          *reinterpret_cast<uint4*>(b_tile + c * 128 + ((chunk ^ (c & 7)) << 4)) =
              make_uint4(__byte_perm(r[0], r[1], 0x5410), __byte_perm(r[2], r[3], 0x5410), __byte_perm(r[0], r[1], 0x7632), __byte_perm(r[2], r[3], 0x7632));
        }
      }
      // cp.async and st.shared wrote through the generic proxy; the tensor core reads through the async proxy
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_base + 8 * b_slot) : "memory");
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  } else if (threadIdx.x == G5_PRODUCERS) {
    // the elected thread of the extra warp feeds the tensor core as stages fill up
    const unsigned idesc = g5_instr_desc();
    for (unsigned it = 0; it < k_iters; ++it) {
      const unsigned b_slot = it % G5_B_STAGES;
      if (!g5_mbar_wait(bar_base + 8 * b_slot, (it / G5_B_STAGES) & 1u, &s_failed)) { failed = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const unsigned long long a_desc = g5_smem_desc(smem_base + (it % G5_A_STAGES) * G5_A_BYTES);
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const unsigned long long b_desc = g5_smem_desc(smem_base + L::B + (b_slot * NW + w) * G5_B_BYTES);
#pragma unroll
        for (int ks = 0; ks < G5_BK / 16; ++ks) {
          const unsigned accumulate = (it != 0 || ks != 0) ? 1u : 0u;
          asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem + w * G5_BN), "l"(a_desc + 2ull * ks),
                       "l"(b_desc + 2ull * ks), "r"(idesc), "r"(accumulate)
                       : "memory");
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_base + 8 * (G5_B_STAGES + b_slot)) : "memory");
      if (it + 1 == k_iters) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_base + 8 * (2 * G5_B_STAGES)) : "memory");
    }
  }
  if (failed) s_failed = 1;
  // every thread waits for the last MMA (bounded), then the CTA agrees on whether anything gave up
  if (!failed && k_iters != 0 && !g5_mbar_wait(bar_base + 8 * (2 * G5_B_STAGES), 0, &s_failed)) { failed = true; s_failed = 1; }
  if (__syncthreads_or(failed ? 1 : 0)) {
    failed = true;
    if (threadIdx.x == 0) atomicAdd(&g_grouped_tc5_giveups, 1u);
  }
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  if (!failed && producer) {
    const unsigned quarter = warp & 3, half = warp >> 2;  // TMEM lanes 32 * quarter .., columns 32 * half .. of every 64-column block
    const unsigned route = s_route[quarter * 32 + lane];
#pragma unroll 1
    for (int pass = 0; pass < (kWide ? 2 : 1); ++pass) {
    const unsigned c_first = col0 + pass * G5_BN + half * 32;
    const unsigned taddr = tmem + ((quarter * 32) << 16) + pass * G5_BN + half * 32;
    unsigned v[32];
    g5_tmem_load32(taddr, v);
    if (kPair) {
      unsigned u[32];
      g5_tmem_load32(taddr + G5_BN, u);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float gate = __uint_as_float(v[j]);
        v[j] = __float_as_uint(gate * (1.0f / (1.0f + expf(-gate))) * __uint_as_float(u[j]));
      }
    }
    if (route != 0xFFFFFFFFu && c_first < p.n) {
      const size_t base = static_cast<size_t>(route) * p.n + c_first;
      const bool full = c_first + 32 <= p.n;
      if (kPair || p.out_bf16) {
        unsigned short* dst = static_cast<unsigned short*>(p.out) + base;
        if (full && base % 8 == 0) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            unsigned packed[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2 * j]), __uint_as_float(v[q * 8 + 2 * j + 1]));
              packed[j] = *reinterpret_cast<const unsigned*>(&t);
            }
            *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c_first + j < p.n) dst[j] = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(v[j])));
        }
      } else {
        float* dst = static_cast<float*>(p.out) + base;
        if (full && base % 4 == 0) {
#pragma unroll
          for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(dst + q * 4) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c_first + j < p.n) dst[j] = __uint_as_float(v[j]);
        }
      }
    }
    }  // pass
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

template <bool kPair, bool kWide>
void launch_g5(Ctx& ctx, const GroupedArgs& a, unsigned tiles) {
  constexpr int smem = G5Layout<kPair, kWide>::TOTAL;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    cudaFuncSetAttribute(grouped_q4_tc5_kernel<kPair, kWide>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured[device] = true;
  }
  const unsigned width = kWide ? 2 * G5_BN : G5_BN;
  launch_pdl(grouped_q4_tc5_kernel<kPair, kWide>, dim3((a.n + width - 1) / width, tiles), dim3(G5_THREADS), smem, ctx.stream, a);
  ctx.launches++;
}

}  // namespace

bool grouped_tc5_supported(const GroupedArgs& a) {
  return a.k % 64 == 0 && a.k >= 64 && a.n >= 1 && reinterpret_cast<size_t>(a.packed[0]) % 8 == 0 && reinterpret_cast<size_t>(a.packed[1]) % 8 == 0;
}

void launch_grouped_tc5(Ctx& ctx, const GroupedArgs& a, bool pair, unsigned tiles) {
  if (pair) launch_g5<true, false>(ctx, a, tiles);
  else if (a.n > G5_BN) launch_g5<false, true>(ctx, a, tiles);
  else launch_g5<false, false>(ctx, a, tiles);
}

unsigned grouped_tc5_giveups() {
  unsigned value = 0;
  cudaMemcpyFromSymbol(&value, g_grouped_tc5_giveups, sizeof(value));
  return value;
}

}  // namespace fj
