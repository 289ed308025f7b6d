// Paged KV kernels: authenticated row copy, split-K GQA decode attention on tensor cores, and a
// generic f32-math attention for f32 planes and odd shapes.
//
// Reference semantics: crates/forja-cpu/src/paged.rs:77-259 (copy_in/copy_out/sdpa/softmax),
// crates/forja-cpu/src/lib.rs:189-380 (PagedCopy, PagedSdpa, PagedSdpaAppend, inactive lanes) and
// the page-table rules of crates/forja-core/src/paged.rs:68-194. score = (q . k) * scale, softmax
// with max subtraction, out = sum_t p_t v_t; causal: attended = min(key_length, q_start + row + 1).
//
// The decode kernel is HBM-bound: per 16-token page and KV head it moves 8 KB (K and V rows of
// 256 B) and spends 32 mma.sync. Algorithmic bytes per sequence and layer:
// kv_heads * L * (d + dv) * 2 + q/out rows + 12 B per page of table/generation reads.
#include "fj_kernels.h"

namespace fj {

namespace {

constexpr unsigned POISON_GENERATION = 0xFFFFFFFFu;

__device__ inline bool authenticate(unsigned page, unsigned generation, const unsigned* __restrict__ generations,
                                    unsigned physical_pages) {
  return page < physical_pages && generation != POISON_GENERATION && generations[page] == generation;
}

// ---------------------------------------------------------------------------------------------
// paged copy
// ---------------------------------------------------------------------------------------------

__global__ void paged_validate_kernel(const unsigned* __restrict__ table, unsigned table_pages,
                                      const unsigned* __restrict__ generations, unsigned physical_pages, unsigned first_page,
                                      unsigned last_page, const unsigned* activity, ErrorRecord* err) {
  if (activity != nullptr && *activity == 0) return;
  for (unsigned lp = first_page + threadIdx.x; lp <= last_page; lp += blockDim.x) {
    bool ok = lp < table_pages && authenticate(table[2 * lp], table[2 * lp + 1], generations, physical_pages);
    if (!ok) report_error(err, ERR_PAGE, lp);
  }
}

__global__ void paged_copy_kernel(int into_pages, void* ordinary, int o_dt, size_t o_row_stride, void* pool, int p_dt,
                                  const unsigned* __restrict__ table, unsigned start, unsigned tokens, unsigned page_tokens,
                                  unsigned elements, const unsigned* activity, const ErrorRecord* err) {
  if (activity != nullptr && *activity == 0) return;
  if (err != nullptr && err->flag != 0) return;  // a refused entry fails the whole copy: write nothing
  for (unsigned t = blockIdx.x; t < tokens; t += gridDim.x) {
    unsigned logical = start + t;
    unsigned page = table[2 * (logical / page_tokens)];
    size_t pool_row = (static_cast<size_t>(page) * page_tokens + logical % page_tokens) * elements;
    size_t ord_row = static_cast<size_t>(t) * o_row_stride;
    for (unsigned i = threadIdx.x; i < elements; i += blockDim.x) {
      if (into_pages) store_from_f32(pool, p_dt, pool_row + i, load_as_f32(ordinary, o_dt, ord_row + i));
      else store_from_f32(ordinary, o_dt, ord_row + i, load_as_f32(pool, p_dt, pool_row + i));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// decode attention on tensor cores (mma.sync m16n8k16, 16-bit inputs, f32 accumulation)
// ---------------------------------------------------------------------------------------------

constexpr int kWarps = 4;
constexpr int kStages = 3;
constexpr int kPageTokens = 16;
constexpr int kHeadDim = 128;
constexpr int kRowBytes = kHeadDim * 2;                 // 256 B per token and KV head
constexpr int kTileBytes = kPageTokens * kRowBytes;     // 4 KB: one page of K (or V) for one KV head
constexpr int kStageBytes = 2 * kTileBytes;             // K then V
constexpr int kDecodeSmem = kWarps * kStages * kStageBytes;  // 96 KB

struct DecodeParams {
  const AttnSeq* seqs;
  const AttnWork* work;
  unsigned n_work;
  const char* kpool;
  const char* vpool;
  const unsigned* generations;
  unsigned physical_pages, q_heads, kv_heads, group;
  float scale;
  int out_dtype;
  float* part_o;
  float* part_ml;
  unsigned* counters;
  ErrorRecord* err;
  const unsigned* n_work_dev;  // when set: the live item count on the device; the grid may be larger (a replayed graph)
};

__device__ inline void cp_async_16(unsigned smem_addr, const void* gmem, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ inline void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ inline void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ inline void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
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
template <bool kBF16> __device__ inline unsigned pack2(float lo, float hi) {
  if (kBF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Writes the final rows of one (sequence, kv head): thread t owns column t of every row.
__device__ inline void store_rows(const AttnSeq& seq, const DecodeParams& p, unsigned kv_head, unsigned column, const float* values /*[16]*/,
                                  const float* denominators /*[16]*/, bool zero) {
  const unsigned rows = seq.q_len * p.group;
  for (unsigned r = 0; r < rows; ++r) {
    unsigned tok = r / p.group, head = kv_head * p.group + r % p.group;
    float v = (zero || denominators[r] <= 0.0f) ? 0.0f : values[r] / denominators[r];
    size_t off = static_cast<size_t>(tok) * seq.o_tok_stride + static_cast<size_t>(head) * seq.o_head_stride + column;
    store_from_f32(seq.out, p.out_dtype, off, v);
  }
}

template <bool kBF16>
__global__ void __launch_bounds__(kWarps * 32, 2) attn_decode_mma_kernel(DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ unsigned s_ticket;
  pdl_sync();
  const unsigned item = blockIdx.x;
  if (item >= p.n_work || (p.n_work_dev != nullptr && item >= *p.n_work_dev)) return;
  const AttnWork work = p.work[item];
  const AttnSeq seq = p.seqs[work.seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned kv_head = work.kv_head;

  if (seq.activity != nullptr && *seq.activity == 0) {  // inactive lane: zeros, no reads (lib.rs:319-328)
    if (work.split == 0) {
      float zeros[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) zeros[r] = 0.0f;
      store_rows(seq, p, kv_head, threadIdx.x, zeros, zeros, true);
    }
    return;
  }

  // rows of the 16-row MMA tile: row r -> query token r / group, head-in-group r % group
  const unsigned r0 = lane >> 2, r1 = r0 + 8;
  const unsigned n_rows = seq.q_len * p.group;
  unsigned limit[2];
  {
    unsigned t0 = r0 / p.group, t1 = r1 / p.group;
    unsigned l0 = seq.causal ? min(seq.key_length, seq.q_start + t0 + 1) : seq.key_length;
    unsigned l1 = seq.causal ? min(seq.key_length, seq.q_start + t1 + 1) : seq.key_length;
    limit[0] = r0 < n_rows ? l0 : 0;
    limit[1] = r1 < n_rows ? l1 : 0;
  }

  // Q fragments (A operand), loaded once from global memory
  unsigned qf[8][4];
  {
    const unsigned short* qbase = static_cast<const unsigned short*>(seq.q);
    const unsigned c0 = (lane & 3) * 2;
    size_t off0 = static_cast<size_t>(r0 / p.group) * seq.q_tok_stride + static_cast<size_t>(kv_head * p.group + r0 % p.group) * seq.q_head_stride;
    size_t off1 = static_cast<size_t>(r1 / p.group) * seq.q_tok_stride + static_cast<size_t>(kv_head * p.group + r1 % p.group) * seq.q_head_stride;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      unsigned col = ks * 16 + c0;
      qf[ks][0] = r0 < n_rows ? *reinterpret_cast<const unsigned*>(qbase + off0 + col) : 0u;
      qf[ks][1] = r1 < n_rows ? *reinterpret_cast<const unsigned*>(qbase + off1 + col) : 0u;
      qf[ks][2] = r0 < n_rows ? *reinterpret_cast<const unsigned*>(qbase + off0 + col + 8) : 0u;
      qf[ks][3] = r1 < n_rows ? *reinterpret_cast<const unsigned*>(qbase + off1 + col + 8) : 0u;
    }
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  int bad = 0;

  const unsigned first_page = work.t_begin / kPageTokens;
  const unsigned end_page = (work.t_end + kPageTokens - 1) / kPageTokens;
  const unsigned my_first = first_page + warp;
  const unsigned n_mine = my_first < end_page ? (end_page - my_first + kWarps - 1) / kWarps : 0;
  const unsigned smem_base = static_cast<unsigned>(__cvta_generic_to_shared(smem)) + warp * kStages * kStageBytes;
  const size_t plane_row_bytes = static_cast<size_t>(p.kv_heads) * kRowBytes;

  // Page-table entries are authenticated 32 pages at a time (lane l owns the warp's page base + l)
  // so the dependent table -> generation loads stay out of the steady-state loop.
  unsigned ent_page = 0;
  int ent_ok = 0;
  auto fetch_entries = [&](unsigned base_j) {
    const unsigned j = base_j + lane;
    ent_page = 0;
    ent_ok = 0;
    if (j < n_mine) {
      const unsigned lp = my_first + j * kWarps;
      bool ok = lp < seq.table_pages;
      unsigned page = 0;
      if (ok) {
        page = seq.table[2 * lp];
        ok = authenticate(page, seq.table[2 * lp + 1], p.generations, p.physical_pages);
      }
      if (!ok) {
        bad = 1;
        report_error(p.err != nullptr ? p.err + seq.err_index : nullptr, ERR_PAGE, lp);
        page = 0;
      }
      ent_page = page;
      ent_ok = ok ? 1 : 0;
    }
  };
  fetch_entries(0);

  auto issue = [&](unsigned j) {
    if (j < n_mine) {
      if (j != 0 && (j & 31) == 0) fetch_entries(j);
      const unsigned lp = my_first + j * kWarps;
      const unsigned page = __shfl_sync(0xffffffffu, ent_page, j & 31);
      const bool ok = __shfl_sync(0xffffffffu, ent_ok, j & 31) != 0;
      const unsigned stage = smem_base + (j % kStages) * kStageBytes;
      const size_t page_off = (static_cast<size_t>(page) * kPageTokens * p.kv_heads + kv_head) * kRowBytes;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const unsigned chunk = lane + 32 * i;       // 256 chunks of 16 B per tile
        const unsigned row = chunk >> 4, c16 = chunk & 15;
        const unsigned bytes = (ok && lp * kPageTokens + row < work.t_end) ? 16u : 0u;
        const size_t src = page_off + row * plane_row_bytes + c16 * 16;
        const unsigned dst = row * kRowBytes + ((c16 ^ (row & 7)) << 4);
        cp_async_16(stage + dst, p.kpool + src, bytes);
        cp_async_16(stage + kTileBytes + dst, p.vpool + src, bytes);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s);

  for (unsigned j = 0; j < n_mine; ++j) {
    issue(j + kStages - 1);
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const unsigned stage = smem_base + (j % kStages) * kStageBytes;
    const unsigned tok_base = (my_first + j * kWarps) * kPageTokens;

    // S = Q K^T for the 16 tokens of this page: two n-tiles of 8 tokens
    float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
    {
      const unsigned mi = lane >> 3, rr = lane & 7;
      const unsigned token = (mi >> 1) * 8 + rr;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const unsigned chunk = ks * 2 + (mi & 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, stage + token * kRowBytes + ((chunk ^ (token & 7)) << 4));
        mma_16816<kBF16>(s[0], qf[ks], b0, b1);
        mma_16816<kBF16>(s[1], qf[ks], b2, b3);
      }
    }
    // scale, mask, online softmax (rows r0: regs 0,1; r1: regs 2,3)
    float row_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const unsigned tok = tok_base + nt * 8 + (lane & 3) * 2 + (e & 1);
        const int r = e >> 1;
        float v = s[nt][e] * p.scale;
        v = tok < limit[r] ? v : -INFINITY;
        s[nt][e] = v;
        row_max[r] = fmaxf(row_max[r], v);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      row_max[r] = fmaxf(row_max[r], __shfl_xor_sync(0xffffffffu, row_max[r], 1));
      row_max[r] = fmaxf(row_max[r], __shfl_xor_sync(0xffffffffu, row_max[r], 2));
      const float m_new = fmaxf(m[r], row_max[r]);
      const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
      alpha[r] = m[r] == -INFINITY ? 0.0f : expf(m[r] - m_safe);
      m[r] = m_new;
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float p0 = expf(s[nt][2 * r] - m_safe), p1 = expf(s[nt][2 * r + 1] - m_safe);
        s[nt][2 * r] = p0;
        s[nt][2 * r + 1] = p1;
        sum += p0 + p1;
      }
      l[r] = l[r] * alpha[r] + sum;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    // O += P V
    unsigned pf[4];
    pf[0] = pack2<kBF16>(s[0][0], s[0][1]);
    pf[1] = pack2<kBF16>(s[0][2], s[0][3]);
    pf[2] = pack2<kBF16>(s[1][0], s[1][1]);
    pf[3] = pack2<kBF16>(s[1][2], s[1][3]);
    {
      const unsigned mi = lane >> 3, rr = lane & 7;
      const unsigned token = (mi & 1) * 8 + rr;
#pragma unroll
      for (int jn = 0; jn < 8; ++jn) {
        const unsigned chunk = jn * 2 + (mi >> 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, stage + kTileBytes + token * kRowBytes + ((chunk ^ (token & 7)) << 4));
        mma_16816<kBF16>(o[2 * jn], pf, b0, b1);
        mma_16816<kBF16>(o[2 * jn + 1], pf, b2, b3);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const int any_bad = __syncthreads_or(bad);  // also: every warp is done with the pipeline buffers

  // combine the four warps through shared memory; only the n_rows valid rows of the tile matter
  float* o_buf = reinterpret_cast<float*>(smem);                       // [4][16][128]
  float* ml_buf = o_buf + kWarps * 16 * kHeadDim;                      // [4][2][16] running max, denominator
  float* f_buf = ml_buf + kWarps * 2 * 16;                             // [4][16] warp factors, [16] row max, [16] row denominator
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const unsigned c = nt * 8 + (lane & 3) * 2;
    float* base = o_buf + (warp * 16) * kHeadDim + c;
    if (r0 < n_rows) *reinterpret_cast<float2*>(base + r0 * kHeadDim) = make_float2(o[nt][0], o[nt][1]);
    if (r1 < n_rows) *reinterpret_cast<float2*>(base + r1 * kHeadDim) = make_float2(o[nt][2], o[nt][3]);
  }
  if ((lane & 3) == 0) {
    ml_buf[(warp * 2 + 0) * 16 + r0] = m[0];
    ml_buf[(warp * 2 + 1) * 16 + r0] = l[0];
    ml_buf[(warp * 2 + 0) * 16 + r1] = m[1];
    ml_buf[(warp * 2 + 1) * 16 + r1] = l[1];
  }
  __syncthreads();
  if (threadIdx.x < 16) {
    const int r = threadIdx.x;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) big = fmaxf(big, ml_buf[(w * 2) * 16 + r]);
    float d = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = ml_buf[(w * 2) * 16 + r];
      const float f = mw == -INFINITY ? 0.0f : expf(mw - big);
      f_buf[w * 16 + r] = f;
      d += f * ml_buf[(w * 2 + 1) * 16 + r];
    }
    f_buf[kWarps * 16 + r] = big;
    f_buf[kWarps * 16 + 16 + r] = d;
  }
  __syncthreads();

  const unsigned col = threadIdx.x;  // 128 threads = 128 columns
  const bool single = work.n_splits == 1;
  float* po = p.part_o + static_cast<size_t>(work.slot) * 16 * kHeadDim;
  float* pml = p.part_ml + static_cast<size_t>(work.slot) * 32;
  for (unsigned r = 0; r < n_rows; ++r) {
    float a = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) a += f_buf[w * 16 + r] * o_buf[(w * 16 + r) * kHeadDim + col];
    if (single) {
      const float d = f_buf[kWarps * 16 + 16 + r];
      const unsigned tok = r / p.group, head = kv_head * p.group + r % p.group;
      const float v = (any_bad || d <= 0.0f) ? 0.0f : a / d;
      store_from_f32(seq.out, p.out_dtype, static_cast<size_t>(tok) * seq.o_tok_stride + static_cast<size_t>(head) * seq.o_head_stride + col, v);
    } else {
      po[r * kHeadDim + col] = a;
    }
  }
  if (single) return;

  // split-K: publish this CTA's partial, the last CTA of the (sequence, kv head) group merges
  if (col < 16) { pml[col] = f_buf[kWarps * 16 + col]; pml[16 + col] = f_buf[kWarps * 16 + 16 + col]; }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_ticket = atomicAdd(&p.counters[work.group_index], 1u + (any_bad ? 0x10000u : 0u)) + 1u + (any_bad ? 0x10000u : 0u);
  __syncthreads();
  const unsigned ticket = s_ticket;
  if ((ticket & 0xFFFFu) != work.n_splits) return;
  __threadfence();
  const unsigned slot_base = work.slot - work.split;
  const bool zero = (ticket >> 16) != 0;
  for (unsigned r = 0; r < n_rows; ++r) {
    float big = -INFINITY;
    for (unsigned sp = 0; sp < work.n_splits; ++sp) big = fmaxf(big, __ldcg(p.part_ml + static_cast<size_t>(slot_base + sp) * 32 + r));
    float a = 0.0f, d = 0.0f;
    for (unsigned sp = 0; sp < work.n_splits; ++sp) {
      const float ms = __ldcg(p.part_ml + static_cast<size_t>(slot_base + sp) * 32 + r);
      const float f = ms == -INFINITY ? 0.0f : expf(ms - big);
      a += f * __ldcg(p.part_o + (static_cast<size_t>(slot_base + sp) * 16 + r) * kHeadDim + col);
      d += f * __ldcg(p.part_ml + static_cast<size_t>(slot_base + sp) * 32 + 16 + r);
    }
    const unsigned tok = r / p.group, head = kv_head * p.group + r % p.group;
    const float v = (zero || d <= 0.0f) ? 0.0f : a / d;
    store_from_f32(seq.out, p.out_dtype, static_cast<size_t>(tok) * seq.o_tok_stride + static_cast<size_t>(head) * seq.o_head_stride + col, v);
  }
  if (threadIdx.x == 0) p.counters[work.group_index] = 0;  // leave the counter ready for the next launch
}

// Chunked-prefill attention on tensor cores lives in fj_attn_tc5.cu (tcgen05, 128 query rows per CTA).

// ---------------------------------------------------------------------------------------------
// generic attention: one CTA per (sequence, head, query row), f32 math, any float dtypes
// ---------------------------------------------------------------------------------------------

constexpr int kGenThreads = 256;
constexpr int kGenTile = 256;

struct GenericParams {
  const AttnSeq* seqs;
  unsigned n_seqs, max_q_len;
  const void* kpool;
  const void* vpool;
  const unsigned* generations;
  unsigned physical_pages, q_heads, kv_heads, head_dim, value_dim, page_tokens;
  int q_dtype, kv_dtype, out_dtype;
  float scale;
  ErrorRecord* err;
};

__global__ void __launch_bounds__(kGenThreads) attn_generic_kernel(GenericParams p) {
  __shared__ float q_s[256];
  __shared__ float scores[kGenTile];
  __shared__ unsigned long long row_base[kGenTile];  // plane row index (page * page_tokens + offset), ~0 = refused
  __shared__ float red[32];
  __shared__ int s_bad;
  const unsigned qrow = blockIdx.x % p.max_q_len;
  const unsigned head = (blockIdx.x / p.max_q_len) % p.q_heads;
  const unsigned si = blockIdx.x / (p.max_q_len * p.q_heads);
  if (si >= p.n_seqs) return;
  const AttnSeq seq = p.seqs[si];
  if (qrow >= seq.q_len) return;
  const unsigned tid = threadIdx.x;
  const size_t out_off = static_cast<size_t>(qrow) * seq.o_tok_stride + static_cast<size_t>(head) * seq.o_head_stride;
  if (seq.activity != nullptr && *seq.activity == 0) {
    for (unsigned c = tid; c < p.value_dim; c += kGenThreads) store_from_f32(seq.out, p.out_dtype, out_off + c, 0.0f);
    return;
  }
  const unsigned kv_head = head / (p.q_heads / p.kv_heads);
  const unsigned attended = seq.causal ? min(seq.key_length, seq.q_start + qrow + 1) : seq.key_length;
  for (unsigned c = tid; c < p.head_dim; c += kGenThreads)
    q_s[c] = load_as_f32(seq.q, p.q_dtype, static_cast<size_t>(qrow) * seq.q_tok_stride + static_cast<size_t>(head) * seq.q_head_stride + c);
  if (tid == 0) s_bad = 0;
  __syncthreads();
  float m = -INFINITY, l = 0.0f, acc = 0.0f;  // acc: output column tid (tid < value_dim)
  for (unsigned tile = 0; tile < attended; tile += kGenTile) {
    const unsigned n = min(static_cast<unsigned>(kGenTile), attended - tile);
    float local_max = -INFINITY;
    for (unsigned i = tid; i < n; i += kGenThreads) {
      const unsigned tok = tile + i, lp = tok / p.page_tokens;
      bool ok = lp < seq.table_pages;
      unsigned page = 0;
      if (ok) { page = seq.table[2 * lp]; ok = authenticate(page, seq.table[2 * lp + 1], p.generations, p.physical_pages); }
      float sc = -INFINITY;
      if (!ok) {
        report_error(p.err != nullptr ? p.err + seq.err_index : nullptr, ERR_PAGE, lp);
        s_bad = 1;
        row_base[i] = ~0ull;
      } else {
        const unsigned long long row = static_cast<unsigned long long>(page) * p.page_tokens + tok % p.page_tokens;
        row_base[i] = row;
        const size_t base = (row * p.kv_heads + kv_head) * p.head_dim;
        float dot = 0.0f;
        for (unsigned c = 0; c < p.head_dim; ++c) dot += q_s[c] * load_as_f32(p.kpool, p.kv_dtype, base + c);
        sc = dot * p.scale;
      }
      scores[i] = sc;
      local_max = fmaxf(local_max, sc);
    }
    local_max = warp_max(local_max);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = local_max;
    __syncthreads();
    float tile_max = -INFINITY;
    for (int w = 0; w < kGenThreads / 32; ++w) tile_max = fmaxf(tile_max, red[w]);
    const float m_new = fmaxf(m, tile_max);
    const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
    const float alpha = m == -INFINITY ? 0.0f : expf(m - m_safe);
    float local_sum = 0.0f;
    for (unsigned i = tid; i < n; i += kGenThreads) {
      float pr = expf(scores[i] - m_safe);
      scores[i] = pr;
      local_sum += pr;
    }
    const float tile_sum = block_sum(local_sum, red);  // includes the barriers that publish scores[]
    l = l * alpha + tile_sum;
    m = m_new;
    if (tid < p.value_dim) {
      acc *= alpha;
      for (unsigned i = 0; i < n; ++i) {
        const unsigned long long row = row_base[i];
        if (row == ~0ull) continue;
        acc += scores[i] * load_as_f32(p.vpool, p.kv_dtype, (row * p.kv_heads + kv_head) * p.value_dim + tid);
      }
    }
    __syncthreads();
  }
  if (tid < p.value_dim) store_from_f32(seq.out, p.out_dtype, out_off + tid, (s_bad || l <= 0.0f) ? 0.0f : acc / l);
}

}  // namespace

size_t attn_part_o_bytes(unsigned slots, unsigned head_dim) { return static_cast<size_t>(slots) * 16 * head_dim * sizeof(float); }
size_t attn_part_ml_bytes(unsigned slots) { return static_cast<size_t>(slots) * 32 * sizeof(float); }

bool attn_decode_mma_supported(const AttnGeometry& g, unsigned max_q_len) {
  if (g.head_dim != kHeadDim || g.value_dim != kHeadDim || g.page_tokens != kPageTokens) return false;
  if (g.q_dtype != g.kv_dtype || (g.kv_dtype != BF16 && g.kv_dtype != F16)) return false;
  if (g.kv_heads == 0 || g.q_heads % g.kv_heads != 0) return false;
  const unsigned group = g.q_heads / g.kv_heads;
  return max_q_len >= 1 && group * max_q_len <= 16;
}

void launch_attn_decode_mma(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, const AttnWork* work, unsigned n_work,
                            const void* kpool, const void* vpool, const unsigned* generations, const AttnScratch& scratch,
                            ErrorRecord* err, const unsigned* n_work_dev) {
  if (n_work == 0) return;
  DecodeParams p;
  p.n_work_dev = n_work_dev;
  p.seqs = seqs; p.work = work; p.n_work = n_work;
  p.kpool = static_cast<const char*>(kpool); p.vpool = static_cast<const char*>(vpool);
  p.generations = generations; p.physical_pages = g.physical_pages;
  p.q_heads = g.q_heads; p.kv_heads = g.kv_heads; p.group = g.q_heads / g.kv_heads;
  p.scale = g.scale; p.out_dtype = g.out_dtype;
  p.part_o = scratch.part_o; p.part_ml = scratch.part_ml; p.counters = scratch.counters; p.err = err;
  static SmemOptIn opted_bf16, opted_f16;
  if (g.kv_dtype == BF16) opt_in_smem(opted_bf16, attn_decode_mma_kernel<true>, kDecodeSmem);
  else opt_in_smem(opted_f16, attn_decode_mma_kernel<false>, kDecodeSmem);
  if (g.kv_dtype == BF16) launch_pdl(attn_decode_mma_kernel<true>, dim3(n_work), dim3(kWarps * 32), kDecodeSmem, ctx.stream, p);
  else launch_pdl(attn_decode_mma_kernel<false>, dim3(n_work), dim3(kWarps * 32), kDecodeSmem, ctx.stream, p);
  ctx.launches++;
}

bool attn_prefill_mma_supported(const AttnGeometry& g) { return attn_prefill_tc5_supported(g); }

unsigned attn_prefill_tokens_per_block(const AttnGeometry& g) { return attn_prefill_tc5_tokens_per_block(g); }

void launch_attn_prefill_mma(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, const uint2* items, unsigned n_items, const void* kpool, const void* vpool,
                             const unsigned* generations, ErrorRecord* err) {
  launch_attn_prefill_tc5(ctx, g, seqs, items, n_items, kpool, vpool, generations, err);
}

void launch_attn_generic(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, unsigned n_seqs, unsigned max_q_len,
                         const void* kpool, const void* vpool, const unsigned* generations, ErrorRecord* err) {
  if (n_seqs == 0 || max_q_len == 0) return;
  GenericParams p;
  p.seqs = seqs; p.n_seqs = n_seqs; p.max_q_len = max_q_len; p.kpool = kpool; p.vpool = vpool; p.generations = generations;
  p.physical_pages = g.physical_pages; p.q_heads = g.q_heads; p.kv_heads = g.kv_heads; p.head_dim = g.head_dim;
  p.value_dim = g.value_dim; p.page_tokens = g.page_tokens; p.q_dtype = g.q_dtype; p.kv_dtype = g.kv_dtype;
  p.out_dtype = g.out_dtype; p.scale = g.scale; p.err = err;
  size_t blocks = static_cast<size_t>(n_seqs) * g.q_heads * max_q_len;
  attn_generic_kernel<<<static_cast<unsigned>(blocks), kGenThreads, 0, ctx.stream>>>(p);
  ctx.launches++;
}

namespace {

__global__ void __launch_bounds__(128) paged_append_batch_kernel(const AppendLane* __restrict__ lanes, unsigned count, void* kpool, void* vpool, int pool_dt,
                                                                 const unsigned* __restrict__ generations, unsigned physical_pages, unsigned page_tokens,
                                                                 unsigned k_elements, unsigned v_elements, ErrorRecord* err) {
  pdl_sync();
  const unsigned i = blockIdx.x;
  if (i >= count) return;
  const AppendLane lane = lanes[i];
  if (lane.activity != nullptr && *lane.activity == 0) return;  // inactive lane: nothing is copied, its table is not read
  const unsigned lp = lane.q_start / page_tokens;
  bool ok = lp < lane.table_pages;
  unsigned page = 0;
  if (ok) { page = lane.table[2 * lp]; ok = authenticate(page, lane.table[2 * lp + 1], generations, physical_pages); }
  if (!ok) {
    if (threadIdx.x == 0) report_error(err != nullptr ? err + lane.err_index : nullptr, ERR_PAGE, lp);
    return;
  }
  const size_t row = static_cast<size_t>(page) * page_tokens + lane.q_start % page_tokens;
  for (unsigned e = threadIdx.x; e < k_elements; e += blockDim.x) store_from_f32(kpool, pool_dt, row * k_elements + e, load_as_f32(lane.k_new, lane.k_dtype, e));
  for (unsigned e = threadIdx.x; e < v_elements; e += blockDim.x) store_from_f32(vpool, pool_dt, row * v_elements + e, load_as_f32(lane.v_new, lane.v_dtype, e));
}

// One CTA: exclusive scan of the lanes' item counts, then every lane writes its items.
__global__ void __launch_bounds__(256) build_work_from_seqs_kernel(const AttnSeq* __restrict__ seqs, unsigned count, unsigned kv_heads, unsigned chunk, AttnWork* work,
                                                                   unsigned work_cap) {
  __shared__ unsigned warp_totals[8];
  __shared__ unsigned s_base;
  pdl_sync();
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  for (unsigned l0 = 0; l0 < count; l0 += blockDim.x) {
    const unsigned lane = l0 + threadIdx.x;
    unsigned len = 0, splits = 0;
    if (lane < count) { len = seqs[lane].key_length; splits = len == 0 ? 1u : (len + chunk - 1) / chunk; }
    const unsigned items = splits * kv_heads;
    // block-wide exclusive scan of `items`
    unsigned inclusive = items;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const unsigned t = __shfl_up_sync(0xffffffffu, inclusive, o); if ((threadIdx.x & 31) >= static_cast<unsigned>(o)) inclusive += t; }
    if ((threadIdx.x & 31) == 31) warp_totals[threadIdx.x >> 5] = inclusive;
    __syncthreads();
    unsigned before = s_base, total = 0;
    for (unsigned w = 0; w < blockDim.x / 32; ++w) { if (w < (threadIdx.x >> 5)) before += warp_totals[w]; total += warp_totals[w]; }
    const unsigned first = before + inclusive - items;
    if (lane < count) {
      for (unsigned h = 0; h < kv_heads; ++h) {
        for (unsigned sp = 0; sp < splits; ++sp) {
          const unsigned idx = first + h * splits + sp;
          if (idx >= work_cap) continue;
          AttnWork w;
          w.seq = lane; w.kv_head = h; w.t_begin = sp * chunk; w.t_end = min(len, (sp + 1) * chunk);
          w.split = sp; w.n_splits = splits; w.slot = idx; w.group_index = lane * kv_heads + h;
          work[idx] = w;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) s_base += total;
    __syncthreads();
  }
}

}  // namespace

void launch_paged_append_batch(Ctx& ctx, const AppendLane* lanes, unsigned count, void* kpool, void* vpool, int pool_dt, const unsigned* generations,
                               unsigned physical_pages, unsigned page_tokens, unsigned k_elements, unsigned v_elements, ErrorRecord* err) {
  if (count == 0) return;
  launch_pdl(paged_append_batch_kernel, dim3(count), dim3(128), 0, ctx.stream, lanes, count, kpool, vpool, pool_dt, generations, physical_pages, page_tokens, k_elements, v_elements, err);
  ctx.launches++;
}

void launch_build_work_from_seqs(Ctx& ctx, const AttnSeq* seqs, unsigned count, unsigned kv_heads, unsigned chunk, AttnWork* work, unsigned work_cap) {
  if (count == 0) return;
  launch_pdl(build_work_from_seqs_kernel, dim3(1), dim3(256), 0, ctx.stream, seqs, count, kv_heads, chunk, work, work_cap);
  ctx.launches++;
}

void launch_paged_copy(Ctx& ctx, bool into_pages, void* ordinary, int o_dt, size_t o_row_stride, void* pool, int p_dt,
                       const unsigned* table, unsigned table_pages, const unsigned* generations, unsigned physical_pages,
                       unsigned start, unsigned tokens, unsigned page_tokens, unsigned elements, const unsigned* activity,
                       ErrorRecord* err) {
  if (tokens == 0) return;
  unsigned first = start / page_tokens, last = (start + tokens - 1) / page_tokens;
  paged_validate_kernel<<<1, 256, 0, ctx.stream>>>(table, table_pages, generations, physical_pages, first, last, activity, err);
  paged_copy_kernel<<<min(tokens, 4096u), 128, 0, ctx.stream>>>(into_pages ? 1 : 0, ordinary, o_dt, o_row_stride, pool, p_dt, table, start, tokens, page_tokens, elements, activity, err);
  ctx.launches += 2;
}

}  // namespace fj

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate
// ---------------------------------------------------------------------------------------------
// Some hosts of this library hand every byte of device memory to the KV page planes up front and
// run the serving loop under a fixed quota, and some call from a latency-critical step where a
// trip into the driver's allocator (which may synchronise the whole device) is not acceptable.
// For them the split-K decode attention is offered once more with all of its scratch - lane
// descriptors, work list, split partials, completion counters - carved out of one fixed array
// that lives in the library image. Nothing is allocated, now or on first use; the price is a hard
// ceiling on the batch (see the FJ_STATIC_ATTENTION_* limits) and that calls share the array.

#include "fj_backend.h"

namespace fj {
namespace {

constexpr unsigned kStaticMaxLanes = FJ_STATIC_ATTENTION_MAX_LANES;
constexpr unsigned kStaticMaxGroups = FJ_STATIC_ATTENTION_MAX_GROUPS;
constexpr unsigned kStaticMaxItems = FJ_STATIC_ATTENTION_MAX_ITEMS;

// layout of the static scratch (byte offsets, each a multiple of 256)
constexpr size_t kOffCounters = 0;                                                     // [groups] u32
constexpr size_t kOffSeqs = kOffCounters + ((kStaticMaxGroups * 4 + 255) / 256) * 256;  // [lanes] AttnSeq
constexpr size_t kOffWork = kOffSeqs + ((kStaticMaxLanes * sizeof(AttnSeq) + 255) / 256) * 256;
constexpr size_t kOffPartMl = kOffWork + ((kStaticMaxItems * sizeof(AttnWork) + 255) / 256) * 256;
constexpr size_t kOffPartO = kOffPartMl + static_cast<size_t>(kStaticMaxItems) * 32 * sizeof(float);
constexpr size_t kStaticBytes = kOffPartO + static_cast<size_t>(kStaticMaxItems) * 16 * kHeadDim * sizeof(float);

// Held by every GPU that loads the library, from load until exit (about 8.6 MB).
static __device__ __align__(256) unsigned char g_static_attention_scratch[kStaticBytes];

struct StaticPlan {
  unsigned key_length[kStaticMaxLanes];
  unsigned lanes, kv_heads, q_heads, table_pages, chunk, elem_bytes;
  const char* q;
  char* out;
  const unsigned* tables;
  unsigned* status;  // caller's two status words or nullptr
};

// Fills the lane descriptors and the work list inside the static array, zeroes the completion
// counters (a previous call that ended early may have left them nonzero) and resets the caller's
// status words. One CTA; the lists are a few thousand words.
__global__ void static_attention_plan_kernel(StaticPlan plan, unsigned char* scratch) {
  unsigned* counters = reinterpret_cast<unsigned*>(scratch + kOffCounters);
  AttnSeq* seqs = reinterpret_cast<AttnSeq*>(scratch + kOffSeqs);
  AttnWork* work = reinterpret_cast<AttnWork*>(scratch + kOffWork);
  for (unsigned g = threadIdx.x; g < plan.lanes * plan.kv_heads; g += blockDim.x) counters[g] = 0;
  if (plan.status != nullptr && threadIdx.x == 0) { plan.status[0] = 0; plan.status[1] = 0xFFFFFFFFu; }
  const size_t row_elems = static_cast<size_t>(plan.q_heads) * kHeadDim;
  for (unsigned lane = threadIdx.x; lane < plan.lanes; lane += blockDim.x) {
    const unsigned len = plan.key_length[lane];
    AttnSeq s;
    s.q = plan.q + lane * row_elems * plan.elem_bytes;
    s.out = plan.out + lane * row_elems * plan.elem_bytes;
    s.table = plan.tables + static_cast<size_t>(lane) * plan.table_pages * 2;
    s.activity = nullptr;
    s.q_len = 1; s.q_start = len ? len - 1 : 0; s.key_length = len; s.table_pages = plan.table_pages;
    s.q_tok_stride = row_elems; s.q_head_stride = kHeadDim; s.o_tok_stride = row_elems; s.o_head_stride = kHeadDim;
    s.causal = 1; s.err_index = 0;
    seqs[lane] = s;
    // items of this lane start after those of the lanes before it
    unsigned first = 0;
    for (unsigned other = 0; other < lane; ++other) {
      const unsigned n = plan.key_length[other];
      first += (n == 0 ? 1 : (n + plan.chunk - 1) / plan.chunk) * plan.kv_heads;
    }
    const unsigned splits = len == 0 ? 1 : (len + plan.chunk - 1) / plan.chunk;
    for (unsigned h = 0; h < plan.kv_heads; ++h) {
      for (unsigned sp = 0; sp < splits; ++sp) {
        AttnWork w;
        w.seq = lane; w.kv_head = h; w.t_begin = sp * plan.chunk; w.t_end = min(len, (sp + 1) * plan.chunk);
        w.split = sp; w.n_splits = splits; w.slot = first + h * splits + sp; w.group_index = lane * plan.kv_heads + h;
        work[w.slot] = w;
      }
    }
  }
}

void* g_static_ptr[16] = {nullptr};  // device address of the array, one per CUDA device
std::mutex g_static_mutex;

}  // namespace
}  // namespace fj

extern "C" int32_t fj_paged_decode_attention_static(fj_backend* be, const void* q, void* out, const void* kpool, const void* vpool, const uint32_t* tables,
                                                    const uint32_t* generations, const uint32_t* key_lengths, uint32_t lanes, uint32_t table_pages,
                                                    uint32_t physical_pages, uint32_t q_heads, uint32_t kv_heads, uint32_t dtype, float scale, uint32_t* status) {
  using namespace fj;
  if (!be || !q || !out || !kpool || !vpool || !tables || !generations || !key_lengths || lanes == 0) return FJ_INVALID_INPUT;
  if ((dtype != FJ_BF16 && dtype != FJ_F16) || kv_heads == 0 || q_heads % kv_heads != 0 || q_heads / kv_heads > 16 || !isfinite(scale)) return FJ_INVALID_INPUT;
  if ((reinterpret_cast<size_t>(q) | reinterpret_cast<size_t>(out)) & 3) return FJ_INVALID_INPUT;
  // ceilings of the fixed array: refuse, never spill into an allocation
  if (lanes > kStaticMaxLanes || static_cast<uint64_t>(lanes) * kv_heads > kStaticMaxGroups) return FJ_QUOTA_EXCEEDED;
  StaticPlan plan;
  uint64_t chunk = 256;
  for (;;) {
    uint64_t items = 0;
    for (uint32_t i = 0; i < lanes; ++i) {
      if (static_cast<uint64_t>(key_lengths[i]) > static_cast<uint64_t>(table_pages) * kPageTokens) return FJ_INVALID_INPUT;
      items += (key_lengths[i] == 0 ? 1 : (key_lengths[i] + chunk - 1) / chunk) * kv_heads;
    }
    if (items <= kStaticMaxItems) { plan.chunk = static_cast<unsigned>(chunk); break; }
    chunk *= 2;
    if (chunk > (1u << 20)) return FJ_QUOTA_EXCEEDED;
  }
  uint32_t n_work = 0;
  for (uint32_t i = 0; i < lanes; ++i) {
    plan.key_length[i] = key_lengths[i];
    n_work += (key_lengths[i] == 0 ? 1 : (key_lengths[i] + plan.chunk - 1) / plan.chunk) * kv_heads;
  }
  std::lock_guard<std::mutex> lock(be->mutex);
  if (be->device < 0 || be->device >= 16) return FJ_INVALID_INPUT;
  if (cudaSetDevice(be->device) != cudaSuccess) return FJ_DEVICE_EXECUTION_FAILED;
  void* scratch = nullptr;
  {
    // first call on this device: resolve the device address of the array (the host-side symbol
    // is only a stand-in) and raise the kernels' shared-memory limit. Neither allocates.
    std::lock_guard<std::mutex> setup(g_static_mutex);
    if (g_static_ptr[be->device] == nullptr) {
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_static_attention_scratch) != cudaSuccess || ptr == nullptr) { cudaGetLastError(); return FJ_DEVICE_EXECUTION_FAILED; }
      if (cudaFuncSetAttribute(attn_decode_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem) != cudaSuccess ||
          cudaFuncSetAttribute(attn_decode_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem) != cudaSuccess) {
        cudaGetLastError();
        return FJ_DEVICE_EXECUTION_FAILED;
      }
      g_static_ptr[be->device] = ptr;
    }
    scratch = g_static_ptr[be->device];
  }
  unsigned char* base = static_cast<unsigned char*>(scratch);
  plan.lanes = lanes; plan.kv_heads = kv_heads; plan.q_heads = q_heads; plan.table_pages = table_pages; plan.elem_bytes = 2;
  plan.q = static_cast<const char*>(q); plan.out = static_cast<char*>(out); plan.tables = tables; plan.status = status;
  static_attention_plan_kernel<<<1, 256, 0, be->stream>>>(plan, base);
  DecodeParams p;
  p.seqs = reinterpret_cast<const AttnSeq*>(base + kOffSeqs);
  p.work = reinterpret_cast<const AttnWork*>(base + kOffWork);
  p.n_work = n_work;
  p.kpool = static_cast<const char*>(kpool); p.vpool = static_cast<const char*>(vpool);
  p.generations = generations; p.physical_pages = physical_pages;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = q_heads / kv_heads;
  p.scale = scale; p.out_dtype = static_cast<int>(dtype);
  p.part_o = reinterpret_cast<float*>(base + kOffPartO);
  p.part_ml = reinterpret_cast<float*>(base + kOffPartMl);
  p.counters = reinterpret_cast<unsigned*>(base + kOffCounters);
  p.err = reinterpret_cast<ErrorRecord*>(status);
  if (dtype == FJ_BF16) attn_decode_mma_kernel<true><<<n_work, kWarps * 32, kDecodeSmem, be->stream>>>(p);
  else attn_decode_mma_kernel<false><<<n_work, kWarps * 32, kDecodeSmem, be->stream>>>(p);
  be->ctx.launches += 2;
  return cudaGetLastError() == cudaSuccess ? FJ_OK : FJ_DEVICE_EXECUTION_FAILED;
}
