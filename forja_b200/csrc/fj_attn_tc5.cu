// Chunked-prefill paged attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Contract (reference: crates/forja-cpu/src/lib.rs:309-433 paged_sdpa; crates/forja-metal/src/paged.metal:206-298 for the
// role): one CTA takes one {sequence, first token} item and one KV head and computes 128 rows = (128 / group) query tokens x
// group query heads against the lane's pages, causal by absolute position; refused pages zero the block's rows and are reported.
//
// Per 64-key tile:
//   * K and V pages are copied with cp.async into shared memory in the 128-byte swizzle, two 64-wide halves of the head
//     dimension each ([keys][64] bf16 = 128 bytes per row), a tile ahead of their use (V in two buffers). For S = Q K^T that
//     layout is a K-major B operand (reduction over the head dimension); for O += P V the very same bytes are an MN-major B
//     operand (reduction over the keys, the head dimension contiguous), so V is never transposed.
//   * S (128 x 64, f32) is produced by 8 tcgen05.mma of K = 16 into one of two tensor-memory buffers; every thread owns one
//     row, reads it back with tcgen05.ld, applies scale and causal limit, and writes its row of P = 2^(s - m) (bf16) into
//     shared memory in the swizzled K-major layout.
//   * O += P V (128 x 128, f32) is 4 tcgen05.mma accumulating in tensor memory over all tiles. The scale m follows the row
//     maximum only when that has grown by more than 2^8, so the accumulator is read, multiplied and written back
//     (tcgen05.ld / tcgen05.st) a few times per row at most instead of once per tile; the row sum uses the same scale.
//   * one __syncthreads per tile; after it a single thread queues O += P V of this tile and S of the next, which run while
//     the threads come round to wait for that S.
// The lane's page table is authenticated into shared memory 1024 pages at a time, off the tile loop's critical path.
// Two CTAs share an SM (about 104 KB of shared memory, 256 tensor-memory columns each): while one runs its softmax the
// other's MMAs and copies proceed. Every wait on an mbarrier is bounded; a wait that runs out is counted
// (attn_prefill_tc5_giveups) and the CTA writes zeros for its rows.
#include "fj_kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace fj {
namespace {

constexpr int A5_ROWS = 128, A5_KEYS = 64, A5_D = 128, A5_PAGE = 16, A5_THREADS = 128;
constexpr int A5_ROW_BYTES = A5_D * 2;                    // one token of one KV head in a plane
constexpr int A5_Q_HALF = A5_ROWS * 128;                  // [128 rows][64 d] bf16, 128 bytes per row
constexpr int A5_KV_HALF = A5_KEYS * 128;                 // [64 keys][64 d]
constexpr int A5_V_BYTES = 2 * A5_KV_HALF;                // one V tile; two of them, used in turn
constexpr int A5_Q = 0, A5_K = A5_Q + 2 * A5_Q_HALF, A5_V = A5_K + 2 * A5_KV_HALF, A5_P = A5_V + 2 * A5_V_BYTES, A5_BAR = A5_P + A5_ROWS * 128;
constexpr int A5_SMEM = A5_BAR + 64 + 1024;               // + barriers, + slack to align the base to 1024 bytes
constexpr unsigned A5_TMEM_COLS = 256, A5_S_COL = 0, A5_O_COL = 128;  // S twice (64 columns each, used in turn), then O
constexpr unsigned kA5SpinLimit = 1u << 24;
constexpr unsigned A5_PAGE_CACHE = 1024;  // authenticated page-table entries kept in shared memory: 256 tiles
constexpr unsigned kPoison = 0xFFFFFFFFu;

__device__ unsigned g_attn_tc5_giveups = 0;

struct A5Params {
  const AttnSeq* seqs;
  const uint2* items;  // {sequence, first token of the block}
  unsigned n_items;
  const char* kpool;
  const char* vpool;
  const unsigned* generations;
  unsigned physical_pages, q_heads, kv_heads, group;
  float scale;
  int out_dtype;
  ErrorRecord* err;
};

__device__ inline void a5_cp_async_16(unsigned smem_addr, const void* gmem, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void a5_mbar_init(unsigned addr, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count) : "memory"); }
// Polls until the phase with the given parity has completed; false when the limit ran out or another thread of the CTA gave up
// (all threads of the CTA wait for the same phases, so they leave the tile loop at the same place).
__device__ inline bool a5_mbar_wait(unsigned addr, unsigned parity, volatile int* gave_up) {
  for (unsigned spin = 0; spin < kA5SpinLimit; ++spin) {
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 1023u) == 1023u && *gave_up != 0) return false;
  }
  *gave_up = 1;
  return false;
}
// Operand tile in the 128-byte swizzle. K-major: rows 128 bytes apart, 8-row groups 1024 bytes apart (stride field), the
// leading field unused. MN-major (the reduction index runs over the rows, 64 contiguous elements of the other index per
// row): 8-row groups again 1024 bytes apart (stride field), the next 64 elements of the contiguous index `leading` bytes on.
__device__ inline unsigned long long a5_desc(unsigned smem_addr, unsigned leading_bytes) {
  unsigned long long d = 0;
  d |= static_cast<unsigned long long>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<unsigned long long>((leading_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<unsigned long long>(1024 >> 4) << 32;
  d |= static_cast<unsigned long long>(1) << 46;
  d |= static_cast<unsigned long long>(2) << 61;
  return d;
}
// kind::f16: D f32; A and B of the 16-bit type; bit 16 set = B is MN-major.
template <bool kBF16>
__device__ inline unsigned a5_idesc(unsigned n, bool b_mn_major) {
  const unsigned fmt = kBF16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn_major ? (1u << 16) : 0u) | ((n >> 3) << 17) | (static_cast<unsigned>(A5_ROWS >> 4) << 24);
}
__device__ inline void a5_mma(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ inline void a5_commit(unsigned bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory"); }
__device__ inline void a5_tmem_load32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ inline void a5_tmem_store32(unsigned taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
      "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
      "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
      "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
      "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
// 2^x for x <= 8 or so; flushes results below 2^-126 to zero (a probability that small adds nothing to an f32 sum)
__device__ inline float a5_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
template <bool kBF16>
__device__ inline unsigned a5_pack2(float lo, float hi) {
  if (kBF16) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&t);
  }
  const __half2 t = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&t);
}

template <bool kBF16>
__global__ void __launch_bounds__(A5_THREADS, 2) attn_prefill_tc5_kernel(A5Params p) {
  extern __shared__ unsigned char a5_smem_raw[];
  __shared__ unsigned s_tmem;
  __shared__ int s_bad, s_gave_up;
  __shared__ unsigned s_pages[A5_PAGE_CACHE];
  const unsigned raw = static_cast<unsigned>(__cvta_generic_to_shared(a5_smem_raw));
  const unsigned smem = (raw + 1023u) & ~1023u;
  unsigned char* smem_ptr = a5_smem_raw + (smem - raw);
  const unsigned bar_s = smem + A5_BAR, bar_o = smem + A5_BAR + 8;
  const int warp = threadIdx.x >> 5;

  pdl_sync();
  if (blockIdx.x >= p.n_items) return;
  const uint2 item = p.items[blockIdx.x];
  const AttnSeq seq = p.seqs[item.x];
  const unsigned kv_head = blockIdx.y, token0 = item.y;
  const unsigned tokens_per_block = A5_ROWS / p.group;
  const unsigned block_tokens = min(tokens_per_block, seq.q_len - token0);
  const bool inactive = seq.activity != nullptr && *seq.activity == 0;

  // this thread's row of the 128-row tile
  const unsigned row = threadIdx.x;
  const unsigned tok = token0 + row / p.group, head = kv_head * p.group + row % p.group;
  const bool live = row / p.group < block_tokens;
  const unsigned limit = !live ? 0u : (seq.causal ? min(seq.key_length, seq.q_start + tok + 1) : seq.key_length);
  const size_t out_off = static_cast<size_t>(tok) * seq.o_tok_stride + static_cast<size_t>(head) * seq.o_head_stride;
  if (inactive) {  // zeros, no reads (lib.rs:319-328)
    if (live)
      for (int i = 0; i < A5_D; ++i) store_from_f32(seq.out, p.out_dtype, out_off + i, 0.0f);
    return;
  }

  if (threadIdx.x == 0) {
    a5_mbar_init(bar_s, 1);
    a5_mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    s_bad = 0;
    s_gave_up = 0;
  }
  if (warp == 0) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(&s_tmem));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst), "r"(A5_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }

  // Q: 128 rows x 256 bytes, two swizzled halves; 4-byte loads (a query view only promises 4-byte alignment); dead rows are zero
  {
    const unsigned short* qbase = static_cast<const unsigned short*>(seq.q);
    for (unsigned id = threadIdx.x; id < A5_ROWS * 16; id += A5_THREADS) {
      const unsigned r = id >> 4, c16 = id & 15;
      const unsigned t = token0 + r / p.group, h = kv_head * p.group + r % p.group;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r / p.group < block_tokens) {
        const unsigned* src = reinterpret_cast<const unsigned*>(qbase + static_cast<size_t>(t) * seq.q_tok_stride + static_cast<size_t>(h) * seq.q_head_stride + c16 * 8);
        v = make_uint4(src[0], src[1], src[2], src[3]);
      }
      *reinterpret_cast<uint4*>(smem_ptr + A5_Q + (c16 >> 3) * A5_Q_HALF + r * 128 + (((c16 & 7) ^ (r & 7)) << 4)) = v;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem = s_tmem;

  // keys this CTA has to visit: the largest limit of its rows
  const unsigned last_token = token0 + block_tokens - 1;
  const unsigned key_end = seq.causal ? min(seq.key_length, seq.q_start + last_token + 1) : seq.key_length;
  const unsigned n_tiles = (key_end + A5_KEYS - 1) / A5_KEYS;
  const size_t plane_row_bytes = static_cast<size_t>(p.kv_heads) * A5_ROW_BYTES;
  const float scale2 = p.scale * 1.4426950408889634f;  // scores are kept in the base-2 domain: p = 2^(s - m)

  // running maximum that the stored probabilities and the accumulator in tensor memory are scaled by, and the row sum in that scale
  float m = -INFINITY, l = 0.0f;
  bool failed = false;
  const unsigned idesc_s = a5_idesc<kBF16>(A5_KEYS, false), idesc_o = a5_idesc<kBF16>(A5_D, true);
  const unsigned lane_base = tmem + ((static_cast<unsigned>(warp) * 32u) << 16);

  // The lane's page table is authenticated ahead of the tile loop, 1024 pages (256 tiles) at a time, into shared memory: one
  // coalesced pass by all threads instead of two dependent global loads per page in every thread on the tile loop's critical
  // path. An entry is the physical page, or kPoison for a page past the keys this block needs or one that failed authentication.
  auto fill_pages = [&](unsigned first_page) {
    for (unsigned idx = threadIdx.x; idx < A5_PAGE_CACHE; idx += A5_THREADS) {
      const unsigned lp = first_page + idx;
      unsigned entry = kPoison;
      if (lp * A5_PAGE < key_end) {
        bool ok = lp < seq.table_pages;
        unsigned page = 0;
        if (ok) {
          page = seq.table[2 * lp];
          const unsigned generation = seq.table[2 * lp + 1];
          ok = page < p.physical_pages && generation != kPoison && p.generations[page] == generation;
        }
        if (ok) entry = page;
        else {
          s_bad = 1;
          report_error(p.err != nullptr ? p.err + seq.err_index : nullptr, ERR_PAGE, lp);
        }
      }
      s_pages[idx] = entry;
    }
  };
  // Pages of a tile as this thread sees them: it copies rows t / 16 + 8 i (i = 0..7) of the tile, i.e. page i / 2, twice each.
  // Only valid while the tile lies in the cached window.
  auto entries = [&](unsigned tile, unsigned (&pg)[4]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) pg[q] = tile < n_tiles ? s_pages[(tile * (A5_KEYS / A5_PAGE) + q) % A5_PAGE_CACHE] : kPoison;
  };
  // One cp.async group with this thread's 8 pieces of a tile of one plane (rows past key_end and refused pages are zero-filled).
  // Piece i is row t / 16 + 8 i of the tile: row (t / 16 + 8 (i & 1)) of page i / 2, and it lands 1024 bytes after piece i - 1.
  const unsigned c16 = threadIdx.x & 15, r0 = threadIdx.x >> 4;
  const size_t page_bytes = static_cast<size_t>(A5_PAGE) * plane_row_bytes;
  const size_t src_even = static_cast<size_t>(kv_head) * A5_ROW_BYTES + r0 * plane_row_bytes + c16 * 16, src_odd = src_even + 8 * plane_row_bytes;
  const unsigned dst0 = (c16 >> 3) * A5_KV_HALF + r0 * 128 + (((c16 & 7) ^ (r0 & 7)) << 4);
  auto issue = [&](unsigned tile, const unsigned (&pg)[4], const char* pool, unsigned region) {
    if (tile < n_tiles) {
      const unsigned rows_left = key_end - tile * A5_KEYS;  // rows of this tile that exist (>= 1)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const unsigned page = pg[i >> 1];
        const bool ok = page != kPoison && r0 + 8 * i < rows_left;
        const size_t src = ok ? page * page_bytes + ((i & 1) ? src_odd : src_even) : 0;
        a5_cp_async_16(smem + region + dst0 + i * 1024, pool + src, ok ? 16u : 0u);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  fill_pages(0);
  __syncthreads();
  unsigned pg[4];
  entries(0, pg);
  issue(0, pg, p.kpool, A5_K);
  issue(0, pg, p.vpool, A5_V);
  entries(1, pg);

  // S = Q K^T of one tile into S buffer (tile & 1): reduction over the head dimension, 4 steps of 16 in each half. One thread issues.
  auto issue_scores = [&](unsigned tile) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const unsigned long long a_desc = a5_desc(smem + A5_Q + half * A5_Q_HALF, 16), b_desc = a5_desc(smem + A5_K + half * A5_KV_HALF, 16);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) a5_mma(tmem + A5_S_COL + (tile & 1u) * A5_KEYS, a_desc + 2ull * ks, b_desc + 2ull * ks, idesc_s, (half != 0 || ks != 0) ? 1u : 0u);
    }
    a5_commit(bar_s);
  };
  if (n_tiles != 0) {
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");  // K of the first tile has landed
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      issue_scores(0);
    }
  }

  // The accumulator O stays in tensor memory over all tiles (P V accumulates into it). It is scaled by 2^-m like the stored
  // probabilities; m follows the row maximum only when that has grown by more than 2^8 since m was set, so the accumulator has
  // to be rescaled (read, multiplied, written back) a few times per row at most, instead of once per tile. Probabilities are
  // at most 2^8 in that scale, exact enough in bf16 and far from any overflow in the f32 sums.
  // One barrier per tile: after it the issuing thread queues O += P V of this tile and S of the next one, which then run while
  // the threads come round to wait for that S.
  constexpr float kSlack = 8.0f;
  for (unsigned tile = 0; tile < n_tiles && !failed; ++tile) {
    const unsigned key_base = tile * A5_KEYS;
    if (!a5_mbar_wait(bar_s, tile & 1u, &s_gave_up)) { failed = true; break; }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    issue(tile + 1, pg, p.kpool, A5_K);  // the tensor core is done with K: the next tile's K travels under the softmax
    const unsigned s_addr = lane_base + A5_S_COL + (tile & 1u) * A5_KEYS;

    // ---- this thread's row of S: the maximum over the keys it may see (all 64 unless the row's limit cuts the tile)
    const unsigned visible = limit > key_base ? min(limit - key_base, static_cast<unsigned>(A5_KEYS)) : 0u;
    // the row is read from tensor memory once and kept in registers for both passes
    float sc[A5_KEYS];
    {
      float part[32];
      a5_tmem_load32(s_addr, part);
#pragma unroll
      for (int i = 0; i < 32; ++i) sc[i] = part[i];
      a5_tmem_load32(s_addr + 32, part);
#pragma unroll
      for (int i = 0; i < 32; ++i) sc[32 + i] = part[i];
    }
    float row_max = -INFINITY;
    {
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (visible == A5_KEYS) {
#pragma unroll
        for (int i = 0; i < A5_KEYS; ++i) mx[i & 3] = fmaxf(mx[i & 3], sc[i]);
      } else {
#pragma unroll
        for (int i = 0; i < A5_KEYS; ++i)
          if (static_cast<unsigned>(i) < visible) mx[i & 3] = fmaxf(mx[i & 3], sc[i]);
      }
      row_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale2;  // scale2 > 0: the maximum commutes with the scaling
    }
    // the previous tile's P V is complete: P and the other V buffer are free, O is stable
    if (tile != 0 && !a5_mbar_wait(bar_o, (tile - 1) & 1u, &s_gave_up)) { failed = true; break; }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    issue(tile + 1, pg, p.vpool, A5_V + ((tile + 1) & 1u) * A5_V_BYTES);
    if ((tile + 2) % (A5_PAGE_CACHE / 4) == 0 && tile + 2 < n_tiles) {  // the next window of the page table (every 256 tiles; uniform over the CTA)
      __syncthreads();  // everyone has taken the entries of tile + 1
      fill_pages((tile + 2) * (A5_KEYS / A5_PAGE));
      __syncthreads();
    }
    entries(tile + 2, pg);
    float alpha = 1.0f;
    if (row_max > m + kSlack || (m == -INFINITY && row_max != -INFINITY)) {
      alpha = m == -INFINITY ? 0.0f : a5_exp2(m - row_max);
      m = row_max;
      l *= alpha;
    }
    if (tile != 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float part[32];
        a5_tmem_load32(lane_base + A5_O_COL + q * 32, part);
#pragma unroll
        for (int i = 0; i < 32; ++i) part[i] *= alpha;
        a5_tmem_store32(lane_base + A5_O_COL + q * 32, part);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
    }
    // ---- second pass: P = 2^(s - m) goes to shared memory as the next A operand
    const float m_safe = m == -INFINITY ? 0.0f : m;
    float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (visible == A5_KEYS) {
#pragma unroll
      for (int i = 0; i < A5_KEYS; ++i) sc[i] = a5_exp2(fmaf(sc[i], scale2, -m_safe));
    } else {
#pragma unroll
      for (int i = 0; i < A5_KEYS; ++i) sc[i] = static_cast<unsigned>(i) < visible ? a5_exp2(fmaf(sc[i], scale2, -m_safe)) : 0.0f;
    }
#pragma unroll
    for (int chunk = 0; chunk < 8; ++chunk) {
      unsigned packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sums[j] += sc[chunk * 8 + 2 * j] + sc[chunk * 8 + 2 * j + 1];
        packed[j] = a5_pack2<kBF16>(sc[chunk * 8 + 2 * j], sc[chunk * 8 + 2 * j + 1]);
      }
      *reinterpret_cast<uint4*>(smem_ptr + A5_P + row * 128 + ((chunk ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    const float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
    l += sum;
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");  // V of this tile and K of the next have landed (the newest group is the next tile's V)
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();  // every row of P is written, V and the next K are in shared memory for everyone, O is rescaled, S has been read

    // ---- O += P V: reduction over the 64 keys in 4 steps of 16; V is MN-major (the two 64-wide halves of the head dimension 8 KB apart)
    if (threadIdx.x == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const unsigned long long a_desc = a5_desc(smem + A5_P, 16);
      const unsigned v_tile = smem + A5_V + (tile & 1u) * A5_V_BYTES;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) a5_mma(tmem + A5_O_COL, a_desc + 2ull * ks, a5_desc(v_tile + ks * 16 * 128, A5_KV_HALF), idesc_o, (tile != 0 || ks != 0) ? 1u : 0u);
      a5_commit(bar_o);
      if (tile + 1 < n_tiles) issue_scores(tile + 1);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  if (!failed && n_tiles != 0 && !a5_mbar_wait(bar_o, (n_tiles - 1) & 1u, &s_gave_up)) failed = true;
  const int any_failed = __syncthreads_or(failed ? 1 : 0);  // the CTA agrees before the next warp-wide tensor-memory reads
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  float o[A5_D];
#pragma unroll
  for (int i = 0; i < A5_D; ++i) o[i] = 0.0f;
  if (!any_failed && n_tiles != 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float part[32];
      a5_tmem_load32(lane_base + A5_O_COL + q * 32, part);
#pragma unroll
      for (int i = 0; i < 32; ++i) o[q * 32 + i] = part[i];
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(A5_TMEM_COLS) : "memory");
  if (any_failed && threadIdx.x == 0) atomicAdd(&g_attn_tc5_giveups, 1u);
  if (!live) return;
  // a refused page or a wait that ran out zeroes the rows of this block
  const float inv = (any_failed || s_bad || l <= 0.0f) ? 0.0f : 1.0f / l;
  if ((p.out_dtype == BF16 || p.out_dtype == F16) && (reinterpret_cast<size_t>(seq.out) + out_off * 2) % 16 == 0) {
    unsigned short* dst = static_cast<unsigned short*>(seq.out) + out_off;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      unsigned packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float v0 = o[c * 8 + 2 * j] * inv, v1 = o[c * 8 + 2 * j + 1] * inv;
        if (p.out_dtype == BF16) packed[j] = a5_pack2<true>(v0, v1);
        else packed[j] = a5_pack2<false>(v0, v1);
      }
      *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < A5_D; ++i) store_from_f32(seq.out, p.out_dtype, out_off + i, o[i] * inv);
  }
}

}  // namespace

bool attn_prefill_tc5_supported(const AttnGeometry& g) {
  const unsigned group = g.kv_heads ? g.q_heads / g.kv_heads : 0;
  return g.head_dim == A5_D && g.value_dim == A5_D && g.page_tokens == A5_PAGE && (g.kv_dtype == BF16 || g.kv_dtype == F16) && g.q_dtype == g.kv_dtype && g.kv_heads != 0 &&
         g.q_heads % g.kv_heads == 0 && group != 0 && group <= A5_ROWS && A5_ROWS % group == 0;
}

unsigned attn_prefill_tc5_tokens_per_block(const AttnGeometry& g) { return A5_ROWS / (g.q_heads / g.kv_heads); }

void launch_attn_prefill_tc5(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, const uint2* items, unsigned n_items, const void* kpool, const void* vpool,
                             const unsigned* generations, ErrorRecord* err) {
  if (n_items == 0) return;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    cudaFuncSetAttribute(attn_prefill_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, A5_SMEM);
    cudaFuncSetAttribute(attn_prefill_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, A5_SMEM);
    configured[device] = true;
  }
  A5Params p{seqs, items, n_items, static_cast<const char*>(kpool), static_cast<const char*>(vpool), generations, g.physical_pages, g.q_heads, g.kv_heads,
             g.q_heads / g.kv_heads, g.scale, g.out_dtype, err};
  dim3 grid(n_items, g.kv_heads);
  if (g.kv_dtype == BF16) launch_pdl(attn_prefill_tc5_kernel<true>, grid, dim3(A5_THREADS), A5_SMEM, ctx.stream, p);
  else launch_pdl(attn_prefill_tc5_kernel<false>, grid, dim3(A5_THREADS), A5_SMEM, ctx.stream, p);
  ctx.launches++;
}

unsigned attn_prefill_tc5_giveups() {
  unsigned value = 0;
  cudaMemcpyFromSymbol(&value, g_attn_tc5_giveups, sizeof(value));
  return value;
}

}  // namespace fj
