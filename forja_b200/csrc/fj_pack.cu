// Device-resident bookkeeping of the continuous-batching step: the paged-KV page allocator and the
// ragged-batch packer. All of it is integer work that must equal the host reference bit for bit:
//  * allocator: LIFO free stack with page 0 on top after initialisation, generation + 1 on every
//    allocation and never 0xFFFFFFFF, refusals change nothing (PagePool::reserve / release /
//    add_slab / allocate_pages, crates/forja-core/src/paged_pool.rs:204-232, 308-327, 1229-1326);
//    prefix sharing: a page carries a reference count, a fork retains the shared prefix pages and
//    marks them immutable for both owners, a shared tail page is replaced by a private copy before it
//    is written (fork_reserved :949-1018, cow_tail :1025-1054), a page returns to the free stack
//    when its last reference goes;
//  * packer: per-lane logical_length / query_start / absolute_position / activity
//    (write_paged_lane_metadata, crates/forja-host/src/lib.rs:4977-5065) plus cu_seqlens, per-row
//    positions, slot_mapping (= physical page * page_tokens + offset) and row_lane.
// One CTA per call keeps request order deterministic; these kernels are latency-bound (a few
// microseconds) and replace host loops plus several small host-to-device copies per step.
#include "fj_kernels.h"

namespace fj {

namespace {

constexpr unsigned POISON = 0xFFFFFFFFu;
constexpr int kPackThreads = 256;

__global__ void kvpool_init_kernel(KvPoolDevice pool) {
  for (unsigned i = threadIdx.x; i < pool.physical_pages; i += blockDim.x) {
    pool.free_stack[i] = pool.physical_pages - 1 - i;  // (start..end).rev(): page 0 pops first
    pool.generations[i] = 0;
    pool.refcounts[i] = 0;
  }
  for (size_t i = threadIdx.x; i < static_cast<size_t>(pool.lanes) * pool.table_pages; i += blockDim.x) {
    pool.tables[2 * i] = 0;
    pool.tables[2 * i + 1] = POISON;
    pool.immutable[i] = 0;
  }
  for (unsigned i = threadIdx.x; i < pool.lanes; i += blockDim.x) pool.lane_pages[i] = 0;
  if (threadIdx.x == 0) *pool.free_count = pool.physical_pages;
}

__global__ void kvpool_reserve_kernel(KvPoolDevice pool, const unsigned* __restrict__ lanes, const unsigned* __restrict__ tokens,
                                      unsigned count, int* status) {
  __shared__ int s_status;
  __shared__ unsigned s_free;
  for (unsigned i = 0; i < count; ++i) {
    const unsigned lane = lanes[i];
    const unsigned need = tokens[i] == 0 ? 0 : (tokens[i] + pool.page_tokens - 1) / pool.page_tokens;
    if (threadIdx.x == 0) {
      s_free = *pool.free_count;
      int st = 0;  // FJ_OK
      if (lane >= pool.lanes || need > pool.table_pages || pool.lane_pages[lane] != 0) st = 7;  // FJ_INVALID_INPUT
      else if (need > s_free) st = 1;                                                         // FJ_QUOTA_EXCEEDED
      s_status = st;
    }
    __syncthreads();
    if (s_status == 0) {
      // preflight: no page of the request may step onto the poison generation
      int overflow = 0;
      for (unsigned j = threadIdx.x; j < need; j += blockDim.x) {
        unsigned g = pool.generations[pool.free_stack[s_free - 1 - j]];
        if (g >= POISON - 1) overflow = 1;
      }
      overflow = __syncthreads_or(overflow);
      if (overflow) {
        if (threadIdx.x == 0) s_status = 3;  // FJ_EXECUTION_FAILED (arithmetic overflow in the reference)
      } else {
        for (unsigned j = threadIdx.x; j < need; j += blockDim.x) {
          const unsigned page = pool.free_stack[s_free - 1 - j];
          const unsigned g = pool.generations[page] + 1;
          pool.generations[page] = g;
          pool.refcounts[page] = 1;
          pool.immutable[static_cast<size_t>(lane) * pool.table_pages + j] = 0;
          pool.tables[(static_cast<size_t>(lane) * pool.table_pages + j) * 2] = page;
          pool.tables[(static_cast<size_t>(lane) * pool.table_pages + j) * 2 + 1] = g;
        }
        if (threadIdx.x == 0) { *pool.free_count = s_free - need; pool.lane_pages[lane] = need; }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && status != nullptr) status[i] = s_status;
    __syncthreads();
  }
}

// Exclusive scan of per-lane values over one CTA (lanes processed in chunks of blockDim.x).
__device__ inline unsigned block_exclusive_scan(unsigned value, unsigned* total, unsigned* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned inclusive = value;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned n = __shfl_up_sync(0xffffffffu, inclusive, o);
    if (lane >= o) inclusive += n;
  }
  __syncthreads();
  if (lane == 31) warp_sums[warp] = inclusive;
  __syncthreads();
  unsigned offset = 0;
  const int warps = blockDim.x >> 5;
  for (int w = 0; w < warps; ++w) {
    if (w < warp) offset += warp_sums[w];
  }
  unsigned sum_all = 0;
  for (int w = 0; w < warps; ++w) sum_all += warp_sums[w];
  *total = sum_all;
  return offset + inclusive - value;
}

// Drops one reference of `page`; true when that was the last one.
__device__ inline bool drop_page_reference(const KvPoolDevice& pool, unsigned page) { return atomicSub(&pool.refcounts[page], 1u) == 1u; }

__global__ void kvpool_release_kernel(KvPoolDevice pool, const unsigned* __restrict__ lanes, unsigned count) {
  __shared__ unsigned s_free, s_pages, s_total;
  __shared__ unsigned warp_sums[32];
  for (unsigned i = 0; i < count; ++i) {
    const unsigned lane = lanes[i];
    if (lane >= pool.lanes) continue;
    if (threadIdx.x == 0) { s_free = *pool.free_count; s_pages = pool.lane_pages[lane]; }
    __syncthreads();
    const unsigned pages = s_pages;
    // sequence order: the pages whose last reference goes are appended in table order (the last one ends on top)
    for (unsigned j0 = 0; j0 < pages; j0 += blockDim.x) {
      const unsigned j = j0 + threadIdx.x;
      unsigned page = 0, freed = 0;
      if (j < pages) {
        const size_t e = static_cast<size_t>(lane) * pool.table_pages + j;
        page = pool.tables[2 * e];
        freed = drop_page_reference(pool, page) ? 1u : 0u;
        pool.tables[2 * e] = 0;
        pool.tables[2 * e + 1] = POISON;
        pool.immutable[e] = 0;
      }
      const unsigned at = block_exclusive_scan(freed, &s_total, warp_sums);
      if (freed) pool.free_stack[s_free + at] = page;
      __syncthreads();
      if (threadIdx.x == 0) s_free += s_total;
      __syncthreads();
    }
    if (threadIdx.x == 0) { *pool.free_count = s_free; pool.lane_pages[lane] = 0; }
    __syncthreads();
  }
}

// fork_reserved: lane `dst` (unbound) shares the first ceil(prefix / page_tokens) pages of lane `src` and gets private pages
// up to `reserved` tokens. Refusals change nothing. args = {src, dst, prefix_tokens, reserved_tokens}.
__global__ void kvpool_fork_kernel(KvPoolDevice pool, const unsigned* __restrict__ args, int* status) {
  __shared__ int s_status;
  __shared__ unsigned s_free;
  const unsigned src = args[0], dst = args[1], prefix = args[2], reserved = args[3];
  const unsigned shared = prefix == 0 ? 0 : (prefix + pool.page_tokens - 1) / pool.page_tokens;
  const unsigned total = reserved == 0 ? 0 : (reserved + pool.page_tokens - 1) / pool.page_tokens;
  if (threadIdx.x == 0) {
    s_free = *pool.free_count;
    int st = 0;
    if (src >= pool.lanes || dst >= pool.lanes || src == dst || reserved < prefix || total > pool.table_pages || pool.lane_pages[dst] != 0 || shared > pool.lane_pages[src]) st = 7;
    else if (total - shared > s_free) st = 1;
    s_status = st;
  }
  __syncthreads();
  if (s_status == 0) {
    const unsigned fresh = total - shared;
    int overflow = 0;
    for (unsigned j = threadIdx.x; j < fresh; j += blockDim.x)
      if (pool.generations[pool.free_stack[s_free - 1 - j]] >= POISON - 1) overflow = 1;
    for (unsigned j = threadIdx.x; j < shared; j += blockDim.x)
      if (pool.refcounts[pool.tables[(static_cast<size_t>(src) * pool.table_pages + j) * 2]] == 0xFFFFFFFFu) overflow = 1;
    overflow = __syncthreads_or(overflow);
    if (overflow) {
      if (threadIdx.x == 0) s_status = 3;
    } else {
      for (unsigned j = threadIdx.x; j < total; j += blockDim.x) {
        const size_t d = static_cast<size_t>(dst) * pool.table_pages + j;
        if (j < shared) {
          const size_t e = static_cast<size_t>(src) * pool.table_pages + j;
          atomicAdd(&pool.refcounts[pool.tables[2 * e]], 1u);
          pool.tables[2 * d] = pool.tables[2 * e];
          pool.tables[2 * d + 1] = pool.tables[2 * e + 1];
          pool.immutable[e] = 1;
          pool.immutable[d] = 1;
        } else {
          const unsigned page = pool.free_stack[s_free - 1 - (j - shared)];
          const unsigned g = pool.generations[page] + 1;
          pool.generations[page] = g;
          pool.refcounts[page] = 1;
          pool.tables[2 * d] = page;
          pool.tables[2 * d + 1] = g;
          pool.immutable[d] = 0;
        }
      }
      if (threadIdx.x == 0) { *pool.free_count = s_free - fresh; pool.lane_pages[dst] = total; }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *status = s_status;
}

// cow_tail: when the page that holds token logical_len - 1 of `lane` is shared (immutable for this lane or referenced by
// another), a fresh page takes its place in the lane's table and the old reference is dropped; the caller then copies
// `tokens` rows from page `src` to page `dst`. result = {status, copied, src, dst, tokens}. args = {lane, logical_len}.
__global__ void kvpool_cow_tail_kernel(KvPoolDevice pool, const unsigned* __restrict__ args, int* result) {
  if (threadIdx.x != 0) return;
  const unsigned lane = args[0], length = args[1];
  result[0] = 0; result[1] = 0; result[2] = 0; result[3] = 0; result[4] = 0;
  if (lane >= pool.lanes) { result[0] = 7; return; }
  if (length == 0 || length % pool.page_tokens == 0) return;
  const unsigned tail = (length - 1) / pool.page_tokens;
  if (tail >= pool.lane_pages[lane]) { result[0] = 7; return; }
  const size_t e = static_cast<size_t>(lane) * pool.table_pages + tail;
  const unsigned old = pool.tables[2 * e];
  if (pool.immutable[e] == 0 && pool.refcounts[old] == 1) return;
  unsigned free_count = *pool.free_count;
  if (free_count == 0) { result[0] = 1; return; }
  const unsigned fresh = pool.free_stack[free_count - 1];
  if (pool.generations[fresh] >= POISON - 1) { result[0] = 3; return; }
  --free_count;
  const unsigned g = pool.generations[fresh] + 1;
  pool.generations[fresh] = g;
  pool.refcounts[fresh] = 1;
  pool.tables[2 * e] = fresh;
  pool.tables[2 * e + 1] = g;
  pool.immutable[e] = 0;
  if (--pool.refcounts[old] == 0) pool.free_stack[free_count++] = old;
  *pool.free_count = free_count;
  result[1] = 1; result[2] = static_cast<int>(old); result[3] = static_cast<int>(fresh); result[4] = static_cast<int>(length % pool.page_tokens);
}

// Drops one reference of `page` and returns it to the free stack when that was the last one; false when the page holds
// no reference to drop (PagePool::release answers CorruptState there, crates/forja-core/src/paged_pool.rs:308-327).
__device__ inline bool release_page(const KvPoolDevice& pool, unsigned page) {
  if (page >= pool.physical_pages || pool.refcounts[page] == 0) return false;
  if (--pool.refcounts[page] == 0) pool.free_stack[(*pool.free_count)++] = page;
  return true;
}

// Sequence boundaries on the device pool (PagedSequence::rewind_private / checkpoint / rollback and the checkpoint's Drop,
// crates/forja-core/src/paged_pool.rs:864-883, 1061-1123, 1167-1175). One thread; args[0] selects the operation:
//   0 rewind check  {0, lane, current_len, new_len}                       -> {status}
//   1 checkpoint    {1, lane, logical_len}                                -> {status, has_tail, index, page, immutable, retained}
//   2 rollback      {2, lane, has_tail, index, page, immutable, retained} -> {status}
//   3 drop          {3, page, retained}                                   -> {status}
// Status: 0 ok, 7 invalid input, 30 shared tail, 31 invalid checkpoint, 32 corrupt state, 3 reference count would overflow.
// Rollback follows the reference as written: when the tail page is unchanged and the checkpoint had retained it, the
// reference taken at the checkpoint is released by rollback and once more when the consumed checkpoint is dropped.
__global__ void kvpool_boundary_kernel(KvPoolDevice pool, const unsigned* __restrict__ args, int* result) {
  if (threadIdx.x != 0) return;
  for (int i = 0; i < 6; ++i) result[i] = 0;
  const unsigned op = args[0];
  if (op == 3) {
    if (args[2] && !release_page(pool, args[1])) result[0] = 32;
    return;
  }
  const unsigned lane = args[1];
  if (lane >= pool.lanes) { result[0] = 7; return; }
  const unsigned bound = pool.lane_pages[lane];
  if (op == 0) {
    const unsigned current = args[2], target = args[3];
    if (target >= current) { result[0] = 31; return; }
    const unsigned first = target / pool.page_tokens, last = (current + pool.page_tokens - 1) / pool.page_tokens;
    if (last > bound) { result[0] = 32; return; }
    for (unsigned j = first; j < last; ++j) {
      const size_t e = static_cast<size_t>(lane) * pool.table_pages + j;
      if (pool.immutable[e] != 0 || pool.refcounts[pool.tables[2 * e]] != 1) { result[0] = 30; return; }
    }
    return;
  }
  if (op == 1) {
    const unsigned length = args[2];
    if (length == 0) return;
    const unsigned tail = (length - 1) / pool.page_tokens;
    if (tail >= bound) { result[0] = 32; return; }
    const size_t e = static_cast<size_t>(lane) * pool.table_pages + tail;
    const unsigned page = pool.tables[2 * e], immutable = pool.immutable[e] != 0 ? 1u : 0u;
    const unsigned retained = (immutable || pool.refcounts[page] > 1) ? 1u : 0u;
    if (retained) {
      if (pool.refcounts[page] == 0xFFFFFFFFu) { result[0] = 3; return; }
      pool.refcounts[page] += 1;
    }
    result[1] = 1; result[2] = static_cast<int>(tail); result[3] = static_cast<int>(page); result[4] = static_cast<int>(immutable); result[5] = static_cast<int>(retained);
    return;
  }
  if (op == 2) {
    if (args[2] == 0) return;  // checkpoint of an empty sequence: only the length goes back
    const unsigned index = args[3], page = args[4], immutable = args[5];
    unsigned retained = args[6];
    if (index >= bound) { if (retained) release_page(pool, page); result[0] = 32; return; }
    const size_t e = static_cast<size_t>(lane) * pool.table_pages + index;
    const unsigned current = pool.tables[2 * e];
    if (current == page) {
      if (retained && !release_page(pool, page)) { result[0] = 32; return; }
    } else {
      if (!release_page(pool, current)) { if (retained) release_page(pool, page); result[0] = 32; return; }
      pool.tables[2 * e] = page;
      pool.tables[2 * e + 1] = pool.generations[page];
      retained = 0;
    }
    pool.immutable[e] = immutable;
    if (retained && !release_page(pool, page)) result[0] = 32;  // the consumed checkpoint is dropped
    return;
  }
  result[0] = 7;
}

__global__ void pack_step_kernel(KvPoolDevice pool, const unsigned* __restrict__ starts, const unsigned* __restrict__ tokens,
                                 unsigned lanes, PackOutputs out, unsigned rows_cap) {
  __shared__ unsigned warp_sums[kPackThreads / 32];
  __shared__ unsigned s_base;
  if (threadIdx.x == 0) { s_base = 0; out.cu_seqlens[0] = 0; }
  __syncthreads();
  for (unsigned l0 = 0; l0 < lanes; l0 += blockDim.x) {
    const unsigned lane = l0 + threadIdx.x;
    const unsigned t = lane < lanes ? tokens[lane] : 0;
    unsigned total;
    const unsigned offset = block_exclusive_scan(t, &total, warp_sums) + s_base;
    if (lane < lanes) {
      const unsigned start = starts[lane];
      out.cu_seqlens[lane + 1] = offset + t;
      out.logical_lengths[lane] = t ? start : 0;
      out.query_starts[lane] = t ? start : 0;
      out.absolute_positions[lane] = t ? start + t - 1 : 0;
      out.activity[lane] = t ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) s_base += total;
    __syncthreads();
  }
  // per-row outputs: all threads share the rows; the lane of a row is found by bisection over cu_seqlens
  const unsigned rows = min(s_base, rows_cap);
  for (unsigned row = threadIdx.x; row < rows; row += blockDim.x) {
    unsigned lo = 0, hi = lanes;  // cu_seqlens[lo] <= row < cu_seqlens[hi]
    while (hi - lo > 1) {
      const unsigned mid = (lo + hi) / 2;
      if (out.cu_seqlens[mid] <= row) lo = mid; else hi = mid;
    }
    const unsigned lane = lo;
    const unsigned position = starts[lane] + (row - out.cu_seqlens[lane]), lp = position / pool.page_tokens;
    unsigned slot = POISON;
    if (lp < pool.table_pages) {
      const size_t e = (static_cast<size_t>(lane) * pool.table_pages + lp) * 2;
      if (pool.tables[e + 1] != POISON) slot = pool.tables[e] * pool.page_tokens + position % pool.page_tokens;
    }
    out.positions[row] = position;
    out.slot_mapping[row] = slot;
    out.row_lane[row] = lane;
  }
  // Rows between the packed count and the lane count are padding for callers that always run `lanes` rows (a
  // recorded launch sequence replayed with fixed grids): position 0 and a refused slot, so nothing is appended for them.
  for (unsigned row = rows + threadIdx.x; row < min(lanes, rows_cap); row += blockDim.x) {
    out.positions[row] = 0;
    out.slot_mapping[row] = POISON;
    out.row_lane[row] = 0;
  }
}

__global__ void build_attn_lists_kernel(KvPoolDevice pool, PackOutputs pack, unsigned lanes, unsigned kv_heads, unsigned chunk_tokens,
                                        const char* q_base, char* out_base, unsigned q_heads, unsigned head_dim, int elem_bytes,
                                        AttnSeq* seqs, AttnWork* work, unsigned* n_work, unsigned work_cap) {
  __shared__ unsigned warp_sums[kPackThreads / 32];
  __shared__ unsigned s_item_base, s_group_base;
  if (threadIdx.x == 0) { s_item_base = 0; s_group_base = 0; }
  __syncthreads();
  const size_t row_elems = static_cast<size_t>(q_heads) * head_dim;
  for (unsigned l0 = 0; l0 < lanes; l0 += blockDim.x) {
    const unsigned lane = l0 + threadIdx.x;
    unsigned q_len = 0, start = 0, key_length = 0, splits = 0;
    if (lane < lanes) {
      q_len = pack.cu_seqlens[lane + 1] - pack.cu_seqlens[lane];
      start = pack.query_starts[lane];
      key_length = q_len ? start + q_len : 0;
      splits = key_length ? (key_length + chunk_tokens - 1) / chunk_tokens : 0;
      AttnSeq s;
      s.q = q_base + static_cast<size_t>(pack.cu_seqlens[lane]) * row_elems * elem_bytes;
      s.out = out_base + static_cast<size_t>(pack.cu_seqlens[lane]) * row_elems * elem_bytes;
      s.table = pool.tables + static_cast<size_t>(lane) * pool.table_pages * 2;
      s.activity = nullptr;
      s.q_len = q_len; s.q_start = start; s.key_length = key_length; s.table_pages = pool.table_pages;
      s.q_tok_stride = row_elems; s.q_head_stride = head_dim; s.o_tok_stride = row_elems; s.o_head_stride = head_dim;
      s.causal = 1; s.err_index = 0;
      seqs[lane] = s;
    }
    unsigned total_items, total_groups;
    const unsigned item_off = block_exclusive_scan(splits * kv_heads, &total_items, warp_sums) + s_item_base;
    const unsigned group_off = block_exclusive_scan(splits ? kv_heads : 0, &total_groups, warp_sums) + s_group_base;
    if (lane < lanes && splits) {
      for (unsigned h = 0; h < kv_heads; ++h) {
        for (unsigned sp = 0; sp < splits; ++sp) {
          const unsigned idx = item_off + h * splits + sp;
          if (idx >= work_cap) continue;
          AttnWork w;
          w.seq = lane; w.kv_head = h;
          w.t_begin = sp * chunk_tokens;
          w.t_end = min(key_length, (sp + 1) * chunk_tokens);
          w.split = sp; w.n_splits = splits; w.slot = idx; w.group_index = group_off + h;
          work[idx] = w;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) { s_item_base += total_items; s_group_base += total_groups; }
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_work = min(s_item_base, work_cap);
}

}  // namespace

void launch_kvpool_init(Ctx& ctx, const KvPoolDevice& pool) {
  kvpool_init_kernel<<<1, 1024, 0, ctx.stream>>>(pool);
  ctx.launches++;
}
void launch_kvpool_reserve(Ctx& ctx, const KvPoolDevice& pool, const unsigned* lanes, const unsigned* tokens, unsigned count,
                           int* status) {
  if (count == 0) return;
  kvpool_reserve_kernel<<<1, 256, 0, ctx.stream>>>(pool, lanes, tokens, count, status);
  ctx.launches++;
}
void launch_kvpool_release(Ctx& ctx, const KvPoolDevice& pool, const unsigned* lanes, unsigned count) {
  if (count == 0) return;
  kvpool_release_kernel<<<1, 256, 0, ctx.stream>>>(pool, lanes, count);
  ctx.launches++;
}
void launch_kvpool_fork(Ctx& ctx, const KvPoolDevice& pool, const unsigned* args, int* status) {
  kvpool_fork_kernel<<<1, 256, 0, ctx.stream>>>(pool, args, status);
  ctx.launches++;
}
void launch_kvpool_cow_tail(Ctx& ctx, const KvPoolDevice& pool, const unsigned* args, int* result) {
  kvpool_cow_tail_kernel<<<1, 32, 0, ctx.stream>>>(pool, args, result);
  ctx.launches++;
}
void launch_kvpool_boundary(Ctx& ctx, const KvPoolDevice& pool, const unsigned* args, int* result) {
  kvpool_boundary_kernel<<<1, 32, 0, ctx.stream>>>(pool, args, result);
  ctx.launches++;
}
void launch_pack_step(Ctx& ctx, const KvPoolDevice& pool, const unsigned* starts, const unsigned* tokens, unsigned lanes,
                      const PackOutputs& out, unsigned rows_cap) {
  pack_step_kernel<<<1, kPackThreads, 0, ctx.stream>>>(pool, starts, tokens, lanes, out, rows_cap);
  ctx.launches++;
}
void launch_build_attn_lists(Ctx& ctx, const KvPoolDevice& pool, const PackOutputs& pack, unsigned lanes, unsigned kv_heads,
                             unsigned chunk_tokens, const void* q_base, void* out_base, unsigned q_heads, unsigned head_dim,
                             int elem_bytes, AttnSeq* seqs, AttnWork* work, unsigned* n_work, unsigned work_cap) {
  build_attn_lists_kernel<<<1, kPackThreads, 0, ctx.stream>>>(pool, pack, lanes, kv_heads, chunk_tokens, static_cast<const char*>(q_base),
                                                             static_cast<char*>(out_base), q_heads, head_dim, elem_bytes, seqs, work, n_work, work_cap);
  ctx.launches++;
}

}  // namespace fj
