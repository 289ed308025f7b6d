// Device-resident fast path of the continuous-batching forward step: the paged-KV pool with its
// on-device allocator and packer, and the dense decoder step that strings the kernels together
// without returning to the host between operators.
//
// Reference op order: Qwen3 dense, engines/qwen3/src/lib.rs:391-452 (layer) and :734-811 (sequence);
// SmolLM2, engines/smollm2/src/optimized.rs:97-245. Every intermediate the reference materialises
// is materialised here in the same dtype, so rounding points coincide.
#include "fj_backend.h"

#include <functional>

#include <string.h>

#include <algorithm>
#include <vector>

using namespace fjb;

namespace {

void* buf_ptr(fj_backend* be, uint64_t id) {
  fj_buffer_rec* r = find_buffer(be, id);
  return r ? r->ptr : nullptr;
}

bool ensure_row_buffers(fj_kvpool* pool, uint32_t rows) {
  if (rows <= pool->rows_cap) return true;
  fj_backend* be = pool->be;
  cudaStreamSynchronize(be->stream);
  uint32_t cap = std::max<uint32_t>(rows, std::max<uint32_t>(pool->rows_cap * 2, 256));
  for (int i = 0; i < 3; ++i) {
    if (pool->buf_rows[i]) {
      fj_buffer_rec* r = find_buffer(be, pool->buf_rows[i]);
      cudaFree(r->ptr);
      be->used_bytes -= r->bytes;
      be->buffers.erase(pool->buf_rows[i]);
      pool->buf_rows[i] = 0;
    }
    if (alloc_buffer(be, static_cast<uint64_t>(cap) * 4, &pool->buf_rows[i]) != FJ_OK) return false;
  }
  pool->rows_cap = cap;
  pool->pack.positions = static_cast<unsigned*>(buf_ptr(be, pool->buf_rows[0]));
  pool->pack.slot_mapping = static_cast<unsigned*>(buf_ptr(be, pool->buf_rows[1]));
  pool->pack.row_lane = static_cast<unsigned*>(buf_ptr(be, pool->buf_rows[2]));
  return true;
}

}  // namespace

extern "C" {

int32_t fj_kvpool_create(fj_backend* be, uint32_t page_tokens, uint32_t physical_pages, uint32_t lanes, uint32_t table_pages, fj_kvpool** out) {
  if (!be || !out || page_tokens == 0 || page_tokens > 4096 || physical_pages == 0 || lanes == 0 || table_pages == 0) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  auto* pool = new fj_kvpool();
  pool->be = be;
  int32_t st = FJ_OK;
  auto need = [&](uint64_t bytes, uint64_t* id) { if (st == FJ_OK) st = alloc_buffer(be, bytes, id); };
  need(static_cast<uint64_t>(physical_pages) * 4, &pool->buf_free);
  need(16, &pool->buf_count);
  need(static_cast<uint64_t>(physical_pages) * 4, &pool->buf_gens);
  need(static_cast<uint64_t>(lanes) * table_pages * 8, &pool->buf_tables);
  need(static_cast<uint64_t>(lanes) * 4, &pool->buf_lane_pages);
  need(static_cast<uint64_t>(physical_pages) * 4, &pool->buf_refcounts);
  need(static_cast<uint64_t>(lanes) * table_pages * 4, &pool->buf_immutable);
  for (int i = 0; i < 4; ++i) need(static_cast<uint64_t>(lanes) * 4, &pool->buf_lane_meta[i]);
  need(static_cast<uint64_t>(lanes + 1) * 4, &pool->buf_lane_meta[4]);
  need(static_cast<uint64_t>(lanes) * 8, &pool->buf_stage);
  if (st != FJ_OK) { delete pool; return st; }
  pool->dev.free_stack = static_cast<unsigned*>(buf_ptr(be, pool->buf_free));
  pool->dev.free_count = static_cast<unsigned*>(buf_ptr(be, pool->buf_count));
  pool->dev.generations = static_cast<unsigned*>(buf_ptr(be, pool->buf_gens));
  pool->dev.tables = static_cast<unsigned*>(buf_ptr(be, pool->buf_tables));
  pool->dev.lane_pages = static_cast<unsigned*>(buf_ptr(be, pool->buf_lane_pages));
  pool->dev.refcounts = static_cast<unsigned*>(buf_ptr(be, pool->buf_refcounts));
  pool->dev.immutable = static_cast<unsigned*>(buf_ptr(be, pool->buf_immutable));
  pool->dev.physical_pages = physical_pages; pool->dev.lanes = lanes; pool->dev.table_pages = table_pages; pool->dev.page_tokens = page_tokens;
  pool->pack.logical_lengths = static_cast<unsigned*>(buf_ptr(be, pool->buf_lane_meta[0]));
  pool->pack.query_starts = static_cast<unsigned*>(buf_ptr(be, pool->buf_lane_meta[1]));
  pool->pack.absolute_positions = static_cast<unsigned*>(buf_ptr(be, pool->buf_lane_meta[2]));
  pool->pack.activity = static_cast<unsigned*>(buf_ptr(be, pool->buf_lane_meta[3]));
  pool->pack.cu_seqlens = static_cast<unsigned*>(buf_ptr(be, pool->buf_lane_meta[4]));
  if (!ensure_row_buffers(pool, 256)) { delete pool; return FJ_ALLOCATION_FAILED; }
  fj::launch_kvpool_init(be->ctx, pool->dev);
  *out = pool;
  return cuda_status(cudaStreamSynchronize(be->stream));
}

void fj_kvpool_destroy(fj_kvpool* pool) {
  if (!pool) return;
  fj_backend* be = pool->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  cudaStreamSynchronize(be->stream);
  uint64_t ids[] = {pool->buf_free, pool->buf_count, pool->buf_gens, pool->buf_tables, pool->buf_lane_pages, pool->buf_refcounts, pool->buf_immutable, pool->buf_lane_meta[0], pool->buf_lane_meta[1],
                    pool->buf_lane_meta[2], pool->buf_lane_meta[3], pool->buf_lane_meta[4], pool->buf_rows[0], pool->buf_rows[1], pool->buf_rows[2], pool->buf_stage};
  for (uint64_t id : ids) {
    fj_buffer_rec* r = id ? find_buffer(be, id) : nullptr;
    if (r) { cudaFree(r->ptr); be->used_bytes -= r->bytes; be->buffers.erase(id); }
  }
  delete pool;
}

int32_t fj_kvpool_reserve(fj_kvpool* pool, const uint32_t* lanes, const uint32_t* tokens, uint32_t count, int32_t* status) {
  if (!pool || (count && (!lanes || !tokens))) return FJ_INVALID_INPUT;
  if (count == 0) return FJ_OK;
  fj_backend* be = pool->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  unsigned* staged = nullptr;
  if (cudaMallocAsync(reinterpret_cast<void**>(&staged), static_cast<size_t>(count) * 12, be->stream) != cudaSuccess) { cudaGetLastError(); return FJ_ALLOCATION_FAILED; }
  cudaMemcpyAsync(staged, lanes, count * 4, cudaMemcpyHostToDevice, be->stream);
  cudaMemcpyAsync(staged + count, tokens, count * 4, cudaMemcpyHostToDevice, be->stream);
  int* dev_status = reinterpret_cast<int*>(staged + 2 * count);
  fj::launch_kvpool_reserve(be->ctx, pool->dev, staged, staged + count, count, dev_status);
  int32_t result = FJ_OK;
  if (status) {
    cudaMemcpyAsync(status, dev_status, count * 4, cudaMemcpyDeviceToHost, be->stream);
    result = cuda_status(cudaStreamSynchronize(be->stream));
  }
  cudaFreeAsync(staged, be->stream);
  return result;
}

int32_t fj_kvpool_release(fj_kvpool* pool, const uint32_t* lanes, uint32_t count) {
  if (!pool || (count && !lanes)) return FJ_INVALID_INPUT;
  if (count == 0) return FJ_OK;
  fj_backend* be = pool->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  unsigned* staged = nullptr;
  if (cudaMallocAsync(reinterpret_cast<void**>(&staged), static_cast<size_t>(count) * 4, be->stream) != cudaSuccess) { cudaGetLastError(); return FJ_ALLOCATION_FAILED; }
  cudaMemcpyAsync(staged, lanes, count * 4, cudaMemcpyHostToDevice, be->stream);
  fj::launch_kvpool_release(be->ctx, pool->dev, staged, count);
  if (pool->lane_epoch.size() < pool->dev.lanes) pool->lane_epoch.resize(pool->dev.lanes, 0);
  for (uint32_t i = 0; i < count; ++i)
    if (lanes[i] < pool->dev.lanes) ++pool->lane_epoch[lanes[i]];  // whatever binds this lane next is another sequence
  cudaFreeAsync(staged, be->stream);
  return FJ_OK;
}

int32_t fj_kvpool_read_table(fj_kvpool* pool, uint32_t lane, uint32_t* entries) {
  if (!pool || !entries || lane >= pool->dev.lanes) return FJ_INVALID_INPUT;
  return fj_read(pool->be, pool->buf_tables, static_cast<uint64_t>(lane) * pool->dev.table_pages * 8, entries, static_cast<uint64_t>(pool->dev.table_pages) * 8);
}
int32_t fj_kvpool_read_generations(fj_kvpool* pool, uint32_t* generations) {
  if (!pool || !generations) return FJ_INVALID_INPUT;
  return fj_read(pool->be, pool->buf_gens, 0, generations, static_cast<uint64_t>(pool->dev.physical_pages) * 4);
}
int32_t fj_kvpool_read_free(fj_kvpool* pool, uint32_t* pages, uint32_t cap, uint32_t* count) {
  if (!pool || !count) return FJ_INVALID_INPUT;
  uint32_t n = 0;
  int32_t st = fj_read(pool->be, pool->buf_count, 0, &n, 4);
  if (st != FJ_OK) return st;
  *count = n;
  if (pages && n) return fj_read(pool->be, pool->buf_free, 0, pages, static_cast<uint64_t>(std::min(n, cap)) * 4);
  return FJ_OK;
}
int32_t fj_kvpool_read_refcounts(fj_kvpool* pool, uint32_t* refcounts) {
  if (!pool || !refcounts) return FJ_INVALID_INPUT;
  return fj_read(pool->be, pool->buf_refcounts, 0, refcounts, static_cast<uint64_t>(pool->dev.physical_pages) * 4);
}

// Runs one single-CTA pool kernel on `words_in` staged argument words and reads `words_out` result words back.
static int32_t pool_control_call(fj_kvpool* pool, const uint32_t* args, unsigned words_in, int32_t* result, unsigned words_out,
                                 const std::function<void(fj::Ctx&, const unsigned*, int*)>& launch) {
  fj_backend* be = pool->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  unsigned* staged = nullptr;
  if (cudaMallocAsync(reinterpret_cast<void**>(&staged), (words_in + words_out) * 4, be->stream) != cudaSuccess) { cudaGetLastError(); return FJ_ALLOCATION_FAILED; }
  cudaMemcpyAsync(staged, args, words_in * 4, cudaMemcpyHostToDevice, be->stream);
  launch(be->ctx, staged, reinterpret_cast<int*>(staged + words_in));
  cudaMemcpyAsync(result, staged + words_in, words_out * 4, cudaMemcpyDeviceToHost, be->stream);
  cudaFreeAsync(staged, be->stream);
  return cuda_status(cudaStreamSynchronize(be->stream));
}

int32_t fj_kvpool_fork(fj_kvpool* pool, uint32_t src_lane, uint64_t src_logical_len, uint32_t dst_lane, uint64_t prefix_tokens, uint64_t reserved_tokens) {
  if (!pool) return FJ_INVALID_INPUT;
  // PagedSequence::fork_reserved refuses a prefix beyond what the source has committed and a reservation below the prefix
  if (prefix_tokens > src_logical_len || reserved_tokens < prefix_tokens || reserved_tokens > 0xFFFFFFFFull - pool->dev.page_tokens) return FJ_INVALID_INPUT;
  const uint32_t args[4] = {src_lane, dst_lane, static_cast<uint32_t>(prefix_tokens), static_cast<uint32_t>(reserved_tokens)};
  int32_t status = FJ_OK;
  const int32_t call = pool_control_call(pool, args, 4, &status, 1,
                                         [&](fj::Ctx& ctx, const unsigned* a, int* r) { fj::launch_kvpool_fork(ctx, pool->dev, a, r); });
  return call != FJ_OK ? call : status;
}

int32_t fj_kvpool_cow_tail(fj_kvpool* pool, uint32_t lane, uint64_t logical_len, uint32_t* out4) {
  if (!pool || !out4 || logical_len > 0xFFFFFFFFull) return FJ_INVALID_INPUT;
  const uint32_t args[2] = {lane, static_cast<uint32_t>(logical_len)};
  int32_t result[5] = {0, 0, 0, 0, 0};
  const int32_t call = pool_control_call(pool, args, 2, result, 5,
                                         [&](fj::Ctx& ctx, const unsigned* a, int* r) { fj::launch_kvpool_cow_tail(ctx, pool->dev, a, r); });
  if (call != FJ_OK) return call;
  for (int i = 0; i < 4; ++i) out4[i] = static_cast<uint32_t>(result[1 + i]);
  return result[0];
}

// ---- sequence boundaries: rewind_private / checkpoint / rollback, crates/forja-core/src/paged_pool.rs:864-883, 1061-1123 ----

int32_t fj_kvpool_rewind_private(fj_kvpool* pool, uint32_t lane, uint64_t current_len, uint64_t new_len) {
  if (!pool || current_len > 0xFFFFFFFFull || new_len > 0xFFFFFFFFull) return FJ_INVALID_INPUT;
  const uint32_t args[4] = {0, lane, static_cast<uint32_t>(current_len), static_cast<uint32_t>(new_len)};
  int32_t result[6] = {0, 0, 0, 0, 0, 0};
  const int32_t call = pool_control_call(pool, args, 4, result, 6, [&](fj::Ctx& ctx, const unsigned* a, int* r) { fj::launch_kvpool_boundary(ctx, pool->dev, a, r); });
  return call != FJ_OK ? call : result[0];
}

int32_t fj_kvpool_checkpoint(fj_kvpool* pool, uint32_t lane, uint64_t logical_len, fj_kv_checkpoint* out) {
  if (!pool || !out || logical_len > 0xFFFFFFFFull || lane >= pool->dev.lanes) return FJ_INVALID_INPUT;
  const uint32_t args[3] = {1, lane, static_cast<uint32_t>(logical_len)};
  int32_t result[6] = {0, 0, 0, 0, 0, 0};
  const int32_t call = pool_control_call(pool, args, 3, result, 6, [&](fj::Ctx& ctx, const unsigned* a, int* r) { fj::launch_kvpool_boundary(ctx, pool->dev, a, r); });
  if (call != FJ_OK) return call;
  if (result[0] != 0) return result[0];
  memset(out, 0, sizeof(*out));
  out->pool = reinterpret_cast<uint64_t>(pool);
  out->lane_epoch = pool->lane_epoch.size() > lane ? pool->lane_epoch[lane] : 0;
  out->logical_len = logical_len;
  out->lane = lane; out->active = 1;
  out->has_tail = static_cast<uint32_t>(result[1]); out->index = static_cast<uint32_t>(result[2]); out->page = static_cast<uint32_t>(result[3]);
  out->immutable = static_cast<uint32_t>(result[4]); out->retained = static_cast<uint32_t>(result[5]);
  return FJ_OK;
}

// SequenceCheckpoint::belongs_to: live, made by this pool, and the lane still holds the sequence it held then.
static bool checkpoint_belongs_to(fj_kvpool* pool, uint32_t lane, const fj_kv_checkpoint* cp) {
  return cp->active != 0 && cp->pool == reinterpret_cast<uint64_t>(pool) && cp->lane == lane && lane < pool->dev.lanes &&
         (pool->lane_epoch.size() > lane ? pool->lane_epoch[lane] : 0) == cp->lane_epoch;
}

int32_t fj_kvpool_checkpoint_drop(fj_kvpool* pool, fj_kv_checkpoint* cp) {
  if (!pool || !cp) return FJ_INVALID_INPUT;
  if (cp->active == 0 && cp->retained == 0) return FJ_OK;
  const bool owes = cp->has_tail && cp->retained && cp->pool == reinterpret_cast<uint64_t>(pool);
  cp->active = 0; cp->retained = 0;
  if (!owes) return FJ_OK;
  const uint32_t args[3] = {3, cp->page, 1};
  int32_t result[6] = {0, 0, 0, 0, 0, 0};
  const int32_t call = pool_control_call(pool, args, 3, result, 6, [&](fj::Ctx& ctx, const unsigned* a, int* r) { fj::launch_kvpool_boundary(ctx, pool->dev, a, r); });
  return call != FJ_OK ? call : result[0];
}

int32_t fj_kvpool_rollback(fj_kvpool* pool, uint32_t lane, fj_kv_checkpoint* cp, uint64_t* logical_len) {
  if (!pool || !cp) return FJ_INVALID_INPUT;
  if (!checkpoint_belongs_to(pool, lane, cp)) {  // a foreign or stale checkpoint is refused and dropped
    fj_kvpool_checkpoint_drop(pool, cp);
    return FJ_POOL_INVALID_CHECKPOINT;
  }
  const uint32_t args[7] = {2, lane, cp->has_tail, cp->index, cp->page, cp->immutable, cp->retained};
  int32_t result[6] = {0, 0, 0, 0, 0, 0};
  const int32_t call = pool_control_call(pool, args, 7, result, 6, [&](fj::Ctx& ctx, const unsigned* a, int* r) { fj::launch_kvpool_boundary(ctx, pool->dev, a, r); });
  cp->active = 0; cp->retained = 0;  // consumed: the kernel has settled every reference the checkpoint held
  if (call != FJ_OK) return call;
  if (result[0] != 0) return result[0];
  if (logical_len) *logical_len = cp->logical_len;
  return FJ_OK;
}

uint64_t fj_kvpool_tables_buffer(fj_kvpool* pool) { return pool ? pool->buf_tables : 0; }
uint64_t fj_kvpool_generations_buffer(fj_kvpool* pool) { return pool ? pool->buf_gens : 0; }

int32_t fj_pack_step(fj_kvpool* pool, const uint32_t* starts, const uint32_t* tokens, uint32_t lanes, fj_pack_view* out) {
  if (!pool || !starts || !tokens || lanes == 0 || lanes > pool->dev.lanes) return FJ_INVALID_INPUT;
  fj_backend* be = pool->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  uint64_t rows = 0;
  for (uint32_t i = 0; i < lanes; ++i) {
    if (tokens[i] && static_cast<uint64_t>(starts[i]) + tokens[i] - 1 > 0xFFFFFFFFull) return FJ_INVALID_INPUT;  // "batch absolute position overflowed"
    rows += tokens[i];
  }
  if (rows > 0x7FFFFFFFull || !ensure_row_buffers(pool, static_cast<uint32_t>(rows))) return FJ_ALLOCATION_FAILED;
  unsigned* staged = static_cast<unsigned*>(buf_ptr(be, pool->buf_stage));
  cudaMemcpyAsync(staged, starts, lanes * 4, cudaMemcpyHostToDevice, be->stream);
  cudaMemcpyAsync(staged + pool->dev.lanes, tokens, lanes * 4, cudaMemcpyHostToDevice, be->stream);
  fj::launch_pack_step(be->ctx, pool->dev, staged, staged + pool->dev.lanes, lanes, pool->pack, pool->rows_cap);
  pool->host_starts.assign(starts, starts + lanes);
  pool->host_tokens.assign(tokens, tokens + lanes);
  pool->rows = static_cast<uint32_t>(rows);
  pool->lanes_packed = lanes;
  if (out) {
    out->rows = pool->rows; out->lanes = lanes;
    out->logical_lengths = pool->buf_lane_meta[0]; out->query_starts = pool->buf_lane_meta[1]; out->absolute_positions = pool->buf_lane_meta[2];
    out->activity = pool->buf_lane_meta[3]; out->cu_seqlens = pool->buf_lane_meta[4];
    out->positions = pool->buf_rows[0]; out->slot_mapping = pool->buf_rows[1]; out->row_lane = pool->buf_rows[2];
  }
  return FJ_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// dense decoder
// ---------------------------------------------------------------------------------------------

struct fj_dense_model {
  fj_backend* be = nullptr;
  fj_kvpool* pool = nullptr;
  fj_dense_config cfg{};
  const void* embed = nullptr;
  const void* final_norm = nullptr;
  struct Layer { const void *input_norm, *q_norm, *k_norm, *wo, *post_norm, *w_down; void *wqkv, *w_gate_up, *k_plane, *v_plane; };
  std::vector<Layer> layers;
  std::vector<void*> owned;  // device allocations of the model
  // workspace
  void *hidden = nullptr, *hidden2 = nullptr, *normed = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *proj = nullptr, *gate_up = nullptr, *act = nullptr;
  void *last_hidden = nullptr, *last_normed = nullptr, *logits = nullptr, *argmax_scratch = nullptr;
  unsigned *tokens_in = nullptr, *tokens_out = nullptr;
  fj::AttnSeq* seqs = nullptr;
  fj::AttnWork* work = nullptr;
  unsigned* n_work_dev = nullptr;
  uint32_t work_cap = 0;
  uint2* prefill_items = nullptr;  // {lane, first token} blocks of the chunked-prefill attention
  uint32_t prefill_items_cap = 0;
  const float* inv_freq = nullptr;
  uint64_t last_kernels = 0, last_work_items = 0;
  // attention timing (CUDA event pairs on the backend's stream)
  bool profile_attention = false;
  std::vector<cudaEvent_t> event_pool;                         // reusable events
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;    // recorded, not yet measured
  uint64_t attention_ns = 0, attention_launches = 0;
  size_t plane_bytes = 0;
  // Recorded decode steps (CUDA graphs), one per bucket of the step's launch geometry; see fj_dense_graph_replay.
  struct StepGraph {
    uint64_t key[8];
    cudaGraphExec_t exec;
    uint64_t kernels;  // kernel launches one replay stands for
    uint64_t last_use;
  };
  bool graph_replay = false;
  std::vector<StepGraph> graphs;
  uint64_t graph_captures = 0, graph_replays = 0, graph_failures = 0, direct_decode_steps = 0, graph_clock = 0;
  cudaEvent_t take_event() {
    if (!event_pool.empty()) { cudaEvent_t e = event_pool.back(); event_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
};

namespace {

__global__ void feedback_tokens_kernel(const unsigned* __restrict__ cu_seqlens, const unsigned* __restrict__ previous, unsigned* tokens, unsigned lanes) {
  unsigned lane = blockIdx.x * blockDim.x + threadIdx.x;
  if (lane >= lanes) return;
  unsigned begin = cu_seqlens[lane], end = cu_seqlens[lane + 1];
  if (end > begin) tokens[end - 1] = previous[lane];
}

// last row of each lane -> [lanes, hidden]; inactive lanes get zeros
template <typename T>
__global__ void gather_last_rows_kernel(const T* __restrict__ hidden, const unsigned* __restrict__ cu_seqlens, T* out, unsigned lanes, unsigned width) {
  for (unsigned lane = blockIdx.x; lane < lanes; lane += gridDim.x) {
    unsigned begin = cu_seqlens[lane], end = cu_seqlens[lane + 1];
    for (unsigned i = threadIdx.x; i < width; i += blockDim.x)
      out[static_cast<size_t>(lane) * width + i] = end > begin ? hidden[static_cast<size_t>(end - 1) * width + i] : T{};
  }
}

// Seeded pseudo-random N(0, 1) fill (counter hash + Box-Muller), two values per thread iteration.
__device__ inline unsigned long long mix64(unsigned long long z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
__global__ void fill_words_kernel(unsigned* out, size_t elements, unsigned long long seed) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < elements; i += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[i] = static_cast<unsigned>(mix64(seed ^ (i * 0xD1342543DE82EF95ull)) >> 16);
}
__global__ void fill_normal_kernel(void* out, int dt, size_t elements, unsigned long long seed, float mean = 0.0f, float std = 1.0f) {
  const size_t pairs = (elements + 1) / 2;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < pairs; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const unsigned long long r = mix64(seed ^ (i * 0xD1342543DE82EF95ull));
    const float u1 = (static_cast<float>(static_cast<unsigned>(r >> 40)) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = (static_cast<float>(static_cast<unsigned>(r & 0xFFFFFFu)) + 0.5f) * (1.0f / 16777216.0f);
    const float radius = sqrtf(-2.0f * logf(u1));
    float s, c;
    sincospif(2.0f * u2, &s, &c);
    fj::store_from_f32(out, dt, 2 * i, mean + std * (radius * c));
    if (2 * i + 1 < elements) fj::store_from_f32(out, dt, 2 * i + 1, mean + std * (radius * s));
  }
}

}  // namespace

namespace fjb {
void launch_feedback_tokens(fj::Ctx& ctx, const unsigned* cu_seqlens, const unsigned* previous, unsigned* tokens, unsigned lanes) {
  feedback_tokens_kernel<<<(lanes + 127) / 128, 128, 0, ctx.stream>>>(cu_seqlens, previous, tokens, lanes);
  ctx.launches++;
}
void launch_gather_last_rows(fj::Ctx& ctx, const void* hidden, int dtype, const unsigned* cu_seqlens, void* out, unsigned lanes, unsigned width) {
  if (dtype == FJ_F32) gather_last_rows_kernel<float><<<std::min(lanes, 1024u), 256, 0, ctx.stream>>>(static_cast<const float*>(hidden), cu_seqlens, static_cast<float*>(out), lanes, width);
  else gather_last_rows_kernel<unsigned short><<<std::min(lanes, 1024u), 256, 0, ctx.stream>>>(static_cast<const unsigned short*>(hidden), cu_seqlens, static_cast<unsigned short*>(out), lanes, width);
  ctx.launches++;
}
}  // namespace fjb

extern "C" {

int32_t fj_dense_model_create(fj_backend* be, const fj_dense_config* config, uint64_t embed, uint64_t final_norm, const fj_dense_layer_weights* layers,
                              fj_kvpool* pool, fj_dense_model** out) {
  if (!be || !config || !layers || !pool || !out || pool->be != be) return FJ_INVALID_INPUT;
  const fj_dense_config& c = *config;
  if ((c.dtype != FJ_F32 && c.dtype != FJ_BF16 && c.dtype != FJ_F16) || c.layers == 0 || c.kv_heads == 0 || c.q_heads % c.kv_heads != 0 || c.head_dim % 2 != 0 || c.head_dim > 256 ||
      c.max_rows == 0 || c.hidden == 0 || c.vocab == 0 || c.intermediate == 0)
    return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const size_t esz = fj::dtype_size(c.dtype);
  auto* m = new fj_dense_model();
  m->be = be; m->pool = pool; m->cfg = c;
  bool ok = true;
  auto dev_alloc = [&](size_t bytes) -> void* {
    void* p = nullptr;
    if (!ok) return nullptr;
    if (be->limit_bytes && be->used_bytes + bytes > be->limit_bytes) { ok = false; return nullptr; }
    if (cudaMalloc(&p, std::max<size_t>(bytes, 16)) != cudaSuccess) { cudaGetLastError(); ok = false; return nullptr; }
    cudaMemsetAsync(p, 0, std::max<size_t>(bytes, 16), be->stream);
    be->used_bytes += bytes;
    m->owned.push_back(p);
    return p;
  };
  auto weight = [&](uint64_t id, uint64_t elements) -> const void* {
    fj_buffer_rec* r = find_buffer(be, id);
    if (!r || r->bytes < elements * esz) { ok = false; return nullptr; }
    return r->ptr;
  };
  const uint64_t qd = static_cast<uint64_t>(c.q_heads) * c.head_dim, kd = static_cast<uint64_t>(c.kv_heads) * c.head_dim;
  m->embed = weight(embed, static_cast<uint64_t>(c.vocab) * c.hidden);
  m->final_norm = weight(final_norm, c.hidden);
  const size_t plane_bytes = static_cast<size_t>(pool->dev.physical_pages) * pool->dev.page_tokens * kd * esz;
  m->plane_bytes = plane_bytes;
  m->layers.resize(c.layers);
  for (uint32_t l = 0; l < c.layers && ok; ++l) {
    const fj_dense_layer_weights& w = layers[l];
    auto& L = m->layers[l];
    L.input_norm = weight(w.input_norm, c.hidden);
    L.post_norm = weight(w.post_norm, c.hidden);
    L.wo = weight(w.wo, static_cast<uint64_t>(c.hidden) * qd);
    L.w_down = weight(w.w_down, static_cast<uint64_t>(c.hidden) * c.intermediate);
    L.q_norm = c.qk_norm ? weight(w.q_norm, c.head_dim) : nullptr;
    L.k_norm = c.qk_norm ? weight(w.k_norm, c.head_dim) : nullptr;
    const void *wq = weight(w.wq, qd * c.hidden), *wk = weight(w.wk, kd * c.hidden), *wv = weight(w.wv, kd * c.hidden);
    const void *wg = weight(w.w_gate, static_cast<uint64_t>(c.intermediate) * c.hidden), *wu = weight(w.w_up, static_cast<uint64_t>(c.intermediate) * c.hidden);
    // stacked projection weights: one GEMM for q|k|v and one for gate|up (same per-element arithmetic)
    L.wqkv = dev_alloc((qd + 2 * kd) * c.hidden * esz);
    L.w_gate_up = dev_alloc(2ull * c.intermediate * c.hidden * esz);
    L.k_plane = dev_alloc(plane_bytes);
    L.v_plane = dev_alloc(plane_bytes);
    if (!ok) break;
    char* dst = static_cast<char*>(L.wqkv);
    cudaMemcpyAsync(dst, wq, qd * c.hidden * esz, cudaMemcpyDeviceToDevice, be->stream);
    cudaMemcpyAsync(dst + qd * c.hidden * esz, wk, kd * c.hidden * esz, cudaMemcpyDeviceToDevice, be->stream);
    cudaMemcpyAsync(dst + (qd + kd) * c.hidden * esz, wv, kd * c.hidden * esz, cudaMemcpyDeviceToDevice, be->stream);
    dst = static_cast<char*>(L.w_gate_up);
    cudaMemcpyAsync(dst, wg, static_cast<size_t>(c.intermediate) * c.hidden * esz, cudaMemcpyDeviceToDevice, be->stream);
    cudaMemcpyAsync(dst + static_cast<size_t>(c.intermediate) * c.hidden * esz, wu, static_cast<size_t>(c.intermediate) * c.hidden * esz, cudaMemcpyDeviceToDevice, be->stream);
  }
  const size_t R = c.max_rows, Lanes = pool->dev.lanes;
  m->hidden = dev_alloc(R * c.hidden * esz);
  m->hidden2 = dev_alloc(R * c.hidden * esz);
  m->normed = dev_alloc(R * c.hidden * esz);
  m->qkv = dev_alloc(R * (qd + 2 * kd) * esz);
  m->q = dev_alloc(R * qd * esz);
  m->attn = dev_alloc(R * qd * esz);
  m->proj = dev_alloc(R * c.hidden * esz);
  m->gate_up = dev_alloc(R * 2 * c.intermediate * esz);
  m->act = dev_alloc(R * c.intermediate * esz);
  m->last_hidden = dev_alloc(Lanes * c.hidden * esz);
  m->last_normed = dev_alloc(Lanes * c.hidden * esz);
  m->logits = dev_alloc(Lanes * c.vocab * esz);
  m->argmax_scratch = dev_alloc(fj::argmax_scratch_bytes(static_cast<unsigned>(Lanes), c.vocab));
  m->tokens_in = static_cast<unsigned*>(dev_alloc(R * 4));
  m->tokens_out = static_cast<unsigned*>(dev_alloc(Lanes * 4));
  m->seqs = static_cast<fj::AttnSeq*>(dev_alloc(Lanes * sizeof(fj::AttnSeq)));
  // work items: every lane may be split into table_pages * page_tokens / 64 chunks in the worst case;
  // the list is sized for the pool's token capacity instead, which bounds the sum over lanes
  const uint64_t token_capacity = static_cast<uint64_t>(pool->dev.physical_pages) * pool->dev.page_tokens;
  // Split-K work items of a step: at most ceil(length / chunk) per lane and KV head with chunk >= 64 and a length that the lane's
  // page table bounds, whatever prefixes are shared between lanes. Sized for that bound, the per-step check against work_cap
  // cannot fail on one rank only (it still can where the bound exceeds 2^22 items and is clipped).
  const uint64_t lane_items = (static_cast<uint64_t>(pool->dev.table_pages) * pool->dev.page_tokens + 63) / 64 + 1;
  m->work_cap = static_cast<uint32_t>(std::min<uint64_t>(std::max<uint64_t>((token_capacity / 64 + Lanes) * c.kv_heads, Lanes * lane_items * c.kv_heads), 1u << 22));
  m->work = static_cast<fj::AttnWork*>(dev_alloc(static_cast<size_t>(m->work_cap) * sizeof(fj::AttnWork)));
  m->n_work_dev = static_cast<unsigned*>(dev_alloc(16));
  m->prefill_items_cap = static_cast<uint32_t>(R + Lanes);
  m->prefill_items = static_cast<uint2*>(dev_alloc(static_cast<size_t>(m->prefill_items_cap) * sizeof(uint2)));
  if (ok) {
    m->inv_freq = c.qk_norm ? freq_table(be, c.theta, -2.0f / static_cast<float>(c.head_dim), c.head_dim / 2, false)
                            : freq_table(be, c.theta, 0.0f, c.head_dim / 2, true);
    ok = m->inv_freq != nullptr;
  }
  if (ok) ok = ensure_gemm_scratch(be, fj::gemm_scratch_bytes(static_cast<unsigned>(R), std::max<unsigned>({2 * c.intermediate, static_cast<unsigned>(qd + 2 * kd), c.hidden}), c.hidden));
  if (!ok || cudaStreamSynchronize(be->stream) != cudaSuccess) {
    for (void* p : m->owned) cudaFree(p);
    delete m;
    return FJ_ALLOCATION_FAILED;
  }
  *out = m;
  return FJ_OK;
}

void fj_dense_model_destroy(fj_dense_model* m) {
  if (!m) return;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  cudaStreamSynchronize(m->be->stream);
  for (auto& g : m->graphs) cudaGraphExecDestroy(g.exec);
  for (void* p : m->owned) cudaFree(p);
  for (auto& pair : m->pending) { cudaEventDestroy(pair.first); cudaEventDestroy(pair.second); }
  for (auto e : m->event_pool) cudaEventDestroy(e);
  delete m;
}

}  // extern "C"

namespace {

// Launch geometry of one step, fixed before anything is enqueued.
struct StepPlan {
  unsigned rows;          // rows every row-wise kernel runs (the packed rows, or the lane count when padded for replay)
  unsigned lanes;
  bool feedback;          // tokens come from the previous step's device-resident greedy tokens
  bool mma;               // split-K tensor-core decode attention
  unsigned max_q_len;
  unsigned chunk;         // tokens per split-K work item
  unsigned work_grid;     // CTAs of the decode attention launch (>= the live item count)
  const unsigned* n_work_dev;  // live item count on the device when work_grid is a rounded-up bound, else nullptr
  unsigned n_blocks;      // 128-row blocks of the chunked-prefill attention
  fj::AttnScratch scratch;
  void* logits;
};

// The launch sequence of one forward step (reference op order: engines/qwen3/src/lib.rs:391-452, 734-811;
// engines/smollm2/src/optimized.rs:97-245). Everything it touches is device-resident and every pointer it
// passes outlives the call, so the same sequence can be recorded into a CUDA graph and replayed.
void enqueue_dense_step(fj_dense_model* m, const StepPlan& plan) {
  fj_backend* be = m->be;
  fj_kvpool* pool = m->pool;
  const fj_dense_config& c = m->cfg;
  const int dt = static_cast<int>(c.dtype);
  const size_t esz = fj::dtype_size(dt);
  const unsigned qd = c.q_heads * c.head_dim, kd = c.kv_heads * c.head_dim, H = c.hidden, I = c.intermediate;
  const unsigned rows = plan.rows, lanes = plan.lanes;
  fj::Ctx& ctx = be->ctx;
  fj::AttnGeometry g;
  g.q_heads = c.q_heads; g.kv_heads = c.kv_heads; g.head_dim = c.head_dim; g.value_dim = c.head_dim; g.page_tokens = pool->dev.page_tokens;
  g.physical_pages = pool->dev.physical_pages; g.q_dtype = dt; g.kv_dtype = dt; g.out_dtype = dt;
  g.scale = 1.0f / sqrtf(static_cast<float>(c.head_dim));

  if (plan.feedback) launch_feedback_tokens(ctx, pool->pack.cu_seqlens, m->tokens_out, m->tokens_in, lanes);
  // attention plan for this step (shared by all layers: q and attn buffers do not move)
  fj::launch_build_attn_lists(ctx, pool->dev, pool->pack, lanes, c.kv_heads, plan.chunk, m->q, m->attn, c.q_heads, c.head_dim, static_cast<int>(esz), m->seqs,
                              m->work, m->n_work_dev, m->work_cap);
  fj::launch_embed(ctx, m->embed, dt, m->tokens_in, m->hidden, dt, c.vocab, H, rows, nullptr);
  void* hidden = m->hidden;
  void* other = m->hidden2;
  fj::launch_rms_norm(ctx, dense_view(hidden, dt, rows, H, H), weight_view(m->layers[0].input_norm, dt, rows, H), dense_view(m->normed, dt, rows, H, H), rows, H, c.eps);
  const unsigned plane_slots = pool->dev.physical_pages * pool->dev.page_tokens;
  for (uint32_t l = 0; l < c.layers; ++l) {
    const auto& L = m->layers[l];
    fj::launch_gemm_nt(ctx, m->normed, dt, H, L.wqkv, dt, H, m->qkv, dt, qd + 2 * kd, rows, qd + 2 * kd, H, be->gemm_scratch, be->gemm_scratch_bytes);
    fj::launch_qknorm_rope_append(ctx, m->qkv, dt, L.q_norm, L.k_norm, pool->pack.positions, pool->pack.slot_mapping, m->q, L.k_plane, L.v_plane, rows, c.q_heads, c.kv_heads,
                                  c.head_dim, c.eps, m->inv_freq, c.qk_norm ? 1 : 0, plane_slots);
    cudaEvent_t attn_begin = nullptr, attn_end = nullptr;
    if (m->profile_attention) { attn_begin = m->take_event(); attn_end = m->take_event(); cudaEventRecord(attn_begin, be->stream); }
    if (plan.mma) fj::launch_attn_decode_mma(ctx, g, m->seqs, m->work, plan.work_grid, L.k_plane, L.v_plane, pool->dev.generations, plan.scratch, nullptr, plan.n_work_dev);
    else if (plan.n_blocks) fj::launch_attn_prefill_mma(ctx, g, m->seqs, m->prefill_items, plan.n_blocks, L.k_plane, L.v_plane, pool->dev.generations, nullptr);
    else fj::launch_attn_generic(ctx, g, m->seqs, lanes, plan.max_q_len, L.k_plane, L.v_plane, pool->dev.generations, nullptr);
    if (m->profile_attention) { cudaEventRecord(attn_end, be->stream); m->pending.emplace_back(attn_begin, attn_end); }
    fj::launch_gemm_nt(ctx, m->attn, dt, qd, L.wo, dt, qd, m->proj, dt, H, rows, H, qd, be->gemm_scratch, be->gemm_scratch_bytes);
    // hidden' = hidden + attention ; normed = rms(hidden') * post_norm
    fj::launch_residual_norm(ctx, dense_view(hidden, dt, rows, H, H), dense_view(m->proj, dt, rows, H, H), weight_view(L.post_norm, dt, rows, H), dense_view(other, dt, rows, H, H),
                             dense_view(m->normed, dt, rows, H, H), rows, H, c.eps, c.qk_norm ? 0 : 1);
    std::swap(hidden, other);
    fj::launch_gemm_nt(ctx, m->normed, dt, H, L.w_gate_up, dt, H, m->gate_up, dt, 2 * I, rows, 2 * I, H, be->gemm_scratch, be->gemm_scratch_bytes);
    fj::launch_silu_mul(ctx, dense_view(m->gate_up, dt, rows, I, 2 * I), dense_view(static_cast<char*>(m->gate_up) + static_cast<size_t>(I) * esz, dt, rows, I, 2 * I),
                        dense_view(m->act, dt, rows, I, I), static_cast<size_t>(rows) * I);
    fj::launch_gemm_nt(ctx, m->act, dt, I, L.w_down, dt, I, m->proj, dt, H, rows, H, I, be->gemm_scratch, be->gemm_scratch_bytes);
    if (l + 1 < c.layers) {
      fj::launch_residual_norm(ctx, dense_view(hidden, dt, rows, H, H), dense_view(m->proj, dt, rows, H, H), weight_view(m->layers[l + 1].input_norm, dt, rows, H),
                               dense_view(other, dt, rows, H, H), dense_view(m->normed, dt, rows, H, H), rows, H, c.eps, c.qk_norm ? 0 : 1);
    } else {
      fj::launch_add(ctx, dense_view(hidden, dt, rows, H, H), dense_view(m->proj, dt, rows, H, H), dense_view(other, dt, rows, H, H), static_cast<size_t>(rows) * H);
    }
    std::swap(hidden, other);
  }
  // last row of every lane -> final norm -> tied lm_head -> greedy token
  launch_gather_last_rows(ctx, hidden, dt, pool->pack.cu_seqlens, m->last_hidden, lanes, H);
  fj::launch_rms_norm(ctx, dense_view(m->last_hidden, dt, lanes, H, H), weight_view(m->final_norm, dt, lanes, H), dense_view(m->last_normed, dt, lanes, H, H), lanes, H, c.eps);
  fj::launch_gemm_nt(ctx, m->last_normed, dt, H, m->embed, dt, H, plan.logits, dt, c.vocab, lanes, c.vocab, H, be->gemm_scratch, be->gemm_scratch_bytes);
  fj::launch_argmax(ctx, plan.logits, dt, c.vocab, m->tokens_out, lanes, c.vocab, m->argmax_scratch);
}

constexpr unsigned kWorkGridStep = 1024;  // recorded decode steps round their attention grid up to a multiple of this (a recording costs tens of ms)
constexpr size_t kMaxStepGraphs = 24;     // least recently used recordings beyond this are dropped

// Replays the recorded launch sequence of this step's bucket, recording it first when the bucket is new.
// false: nothing was enqueued (recording failed or is not possible); the caller runs the step directly.
bool replay_dense_step(fj_dense_model* m, const StepPlan& plan) {
  fj_backend* be = m->be;
  fj_dense_model::StepGraph wanted{};
  const uint64_t key[8] = {plan.lanes, plan.chunk, plan.work_grid, plan.feedback ? 1u : 0u, reinterpret_cast<uint64_t>(plan.logits),
                           reinterpret_cast<uint64_t>(be->gemm_scratch), reinterpret_cast<uint64_t>(plan.scratch.counters), reinterpret_cast<uint64_t>(m->pool->pack.positions)};
  ++m->graph_clock;
  for (auto& g : m->graphs) {
    if (memcmp(g.key, key, sizeof(key)) != 0) continue;
    if (cudaGraphLaunch(g.exec, be->stream) != cudaSuccess) { cudaGetLastError(); return false; }
    g.last_use = m->graph_clock;
    be->ctx.launches += g.kernels;
    ++m->graph_replays;
    return true;
  }
  if (m->graph_failures >= 3) return false;  // recording does not work here: stay on the direct path
  const unsigned long long before = be->ctx.launches;
  if (cudaStreamBeginCapture(be->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); ++m->graph_failures; return false; }
  enqueue_dense_step(m, plan);
  cudaGraph_t graph = nullptr;
  const cudaError_t ended = cudaStreamEndCapture(be->stream, &graph);
  const uint64_t kernels = be->ctx.launches - before;
  be->ctx.launches = before;  // nothing ran yet
  cudaGraphExec_t exec = nullptr;
  if (ended != cudaSuccess || graph == nullptr || cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
    cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    ++m->graph_failures;
    return false;
  }
  cudaGraphDestroy(graph);
  if (m->graphs.size() >= kMaxStepGraphs) {
    auto oldest = std::min_element(m->graphs.begin(), m->graphs.end(), [](const fj_dense_model::StepGraph& a, const fj_dense_model::StepGraph& b) { return a.last_use < b.last_use; });
    cudaGraphExecDestroy(oldest->exec);
    m->graphs.erase(oldest);
  }
  memcpy(wanted.key, key, sizeof(key));
  wanted.exec = exec; wanted.kernels = kernels; wanted.last_use = m->graph_clock;
  m->graphs.push_back(wanted);
  ++m->graph_captures;
  if (cudaGraphLaunch(exec, be->stream) != cudaSuccess) { cudaGetLastError(); return false; }
  be->ctx.launches += kernels;
  ++m->graph_replays;
  return true;
}

}  // namespace

extern "C" {

int32_t fj_dense_step(fj_dense_model* m, const uint32_t* token_ids, uint32_t* out_tokens, uint64_t logits_out) {
  if (!m) return FJ_INVALID_INPUT;
  fj_backend* be = m->be;
  fj_kvpool* pool = m->pool;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const fj_dense_config& c = m->cfg;
  const unsigned rows = pool->rows, lanes = pool->lanes_packed;
  if (rows == 0 || lanes == 0) return FJ_INVALID_INPUT;
  if (rows > c.max_rows) return FJ_INVALID_INPUT;
  const int dt = static_cast<int>(c.dtype);
  const size_t esz = fj::dtype_size(dt);
  fj::Ctx& ctx = be->ctx;
  const unsigned long long launches_before = ctx.launches;

  StepPlan plan{};
  plan.rows = rows; plan.lanes = lanes; plan.feedback = token_ids == nullptr;
  const unsigned group = c.q_heads / c.kv_heads;
  unsigned max_q_len = 0;
  uint64_t total_keys = 0;
  bool decode_only = true;
  for (unsigned l = 0; l < lanes; ++l) {
    max_q_len = std::max(max_q_len, pool->host_tokens[l]);
    decode_only = decode_only && pool->host_tokens[l] <= 1;
    if (pool->host_tokens[l]) total_keys += static_cast<uint64_t>(pool->host_starts[l]) + pool->host_tokens[l];
  }
  plan.max_q_len = max_q_len;
  fj::AttnGeometry g;
  g.q_heads = c.q_heads; g.kv_heads = c.kv_heads; g.head_dim = c.head_dim; g.value_dim = c.head_dim; g.page_tokens = pool->dev.page_tokens;
  g.physical_pages = pool->dev.physical_pages; g.q_dtype = dt; g.kv_dtype = dt; g.out_dtype = dt;
  plan.mma = fj::attn_decode_mma_supported(g, max_q_len) && max_q_len * group <= 16;
  uint64_t chunk = 64, n_work = 0;
  if (plan.mma) {
    const uint64_t target_items = static_cast<uint64_t>(ctx.sm_count) * 2 * 4;
    chunk = (total_keys * c.kv_heads + target_items - 1) / std::max<uint64_t>(target_items, 1);
    chunk = std::min<uint64_t>(std::max<uint64_t>((chunk + 63) / 64 * 64, 64), 1024);
    for (unsigned l = 0; l < lanes; ++l)
      if (pool->host_tokens[l]) n_work += ((static_cast<uint64_t>(pool->host_starts[l]) + pool->host_tokens[l] + chunk - 1) / chunk) * c.kv_heads;
    if (n_work > m->work_cap) return FJ_QUOTA_EXCEEDED;
  }
  plan.chunk = static_cast<unsigned>(chunk);
  plan.work_grid = static_cast<unsigned>(n_work);
  // A decode-only step can be replayed from a recording: every row-wise kernel then runs `lanes` rows (the packer pads the
  // rows past the packed count with refused slots) and the attention grid is rounded up, with the live count read on the device.
  const bool replay = m->graph_replay && plan.mma && decode_only && !m->profile_attention && lanes <= c.max_rows && lanes <= pool->rows_cap &&
                      m->direct_decode_steps > 0 && m->graph_failures < 3;
  if (replay) {
    plan.rows = lanes;
    plan.work_grid = static_cast<unsigned>(std::min<uint64_t>((n_work + kWorkGridStep - 1) / kWorkGridStep * kWorkGridStep, m->work_cap));
    plan.n_work_dev = m->n_work_dev;
  }
  // query runs too long for the decode kernel: 128-row tensor-core blocks, listed by the host from the packed step
  if (!plan.mma && fj::attn_prefill_mma_supported(g)) {
    const unsigned per_block = fj::attn_prefill_tokens_per_block(g);
    std::vector<uint2> items;
    for (unsigned l = 0; l < lanes; ++l)
      for (unsigned t = 0; t < pool->host_tokens[l]; t += per_block) items.push_back(make_uint2(l, t));
    if (items.size() > m->prefill_items_cap) return FJ_QUOTA_EXCEEDED;
    plan.n_blocks = static_cast<unsigned>(items.size());
    cudaMemcpyAsync(m->prefill_items, items.data(), items.size() * sizeof(uint2), cudaMemcpyHostToDevice, be->stream);  // pageable source: staged before the call returns
  }
  plan.scratch = fj::AttnScratch{nullptr, nullptr, nullptr};
  if (plan.mma) {
    const size_t groups = static_cast<size_t>(lanes) * c.kv_heads;
    const size_t counter_bytes = (groups * sizeof(unsigned) + 255) / 256 * 256;
    const size_t o_bytes = fj::attn_part_o_bytes(plan.work_grid, c.head_dim), ml_bytes = fj::attn_part_ml_bytes(plan.work_grid);
    if (!ensure_attn_scratch(be, counter_bytes + o_bytes + ml_bytes)) return FJ_ALLOCATION_FAILED;
    plan.scratch.counters = static_cast<unsigned*>(be->attn_scratch);
    plan.scratch.part_o = reinterpret_cast<float*>(static_cast<char*>(be->attn_scratch) + counter_bytes);
    plan.scratch.part_ml = reinterpret_cast<float*>(static_cast<char*>(be->attn_scratch) + counter_bytes + o_bytes);
  }
  plan.logits = m->logits;
  if (logits_out) {
    fj_buffer_rec* r = find_buffer(be, logits_out);
    if (!r || r->readonly || r->bytes < static_cast<uint64_t>(lanes) * c.vocab * esz) return FJ_INVALID_INPUT;
    plan.logits = r->ptr;
  }

  if (token_ids) cudaMemcpyAsync(m->tokens_in, token_ids, static_cast<size_t>(rows) * 4, cudaMemcpyHostToDevice, be->stream);
  if (!(replay && replay_dense_step(m, plan))) {
    if (replay) {  // the recording could not be made: run this step with its exact geometry
      plan.rows = rows; plan.work_grid = static_cast<unsigned>(n_work); plan.n_work_dev = nullptr;
    }
    enqueue_dense_step(m, plan);
    if (plan.mma && decode_only) ++m->direct_decode_steps;
  }
  m->last_kernels = ctx.launches - launches_before;
  m->last_work_items = n_work;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return FJ_DEVICE_EXECUTION_FAILED;
  if (out_tokens) {
    cudaMemcpyAsync(out_tokens, m->tokens_out, static_cast<size_t>(lanes) * 4, cudaMemcpyDeviceToHost, be->stream);
    return cuda_status(cudaStreamSynchronize(be->stream));
  }
  return FJ_OK;
}

// Graph replay for the decode step (the backend-specific tier behind Backend::prepare_graph / replay,
// crates/forja-core/src/backend.rs:858-967): with replay enabled, decode-only steps are recorded once per bucket
// {lanes, split-K chunk, attention grid rounded up to 1024 items, token source, logits target} as a CUDA graph and
// replayed, so a step costs one graph launch on the host instead of one launch per kernel.
int32_t fj_dense_graph_replay(fj_dense_model* m, uint32_t enabled) {
  if (!m) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  m->graph_replay = enabled != 0;
  return FJ_OK;
}

int32_t fj_dense_graph_stats(fj_dense_model* m, uint64_t* recordings, uint64_t* replays, uint64_t* failures) {
  if (!m) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  if (recordings) *recordings = m->graph_captures;
  if (replays) *replays = m->graph_replays;
  if (failures) *failures = m->graph_failures;
  return FJ_OK;
}

// The data half of cow_tail for this model's planes: the first `tokens` K and V rows of page `src_page` are copied to
// page `dst_page` in every layer (stream-ordered device copies).
int32_t fj_dense_copy_page(fj_dense_model* m, uint32_t src_page, uint32_t dst_page, uint32_t tokens) {
  if (!m) return FJ_INVALID_INPUT;
  fj_backend* be = m->be;
  const fj::KvPoolDevice& pool = m->pool->dev;
  if (src_page >= pool.physical_pages || dst_page >= pool.physical_pages || tokens > pool.page_tokens) return FJ_INVALID_INPUT;
  if (tokens == 0 || src_page == dst_page) return FJ_OK;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const size_t row = static_cast<size_t>(m->cfg.kv_heads) * m->cfg.head_dim * fj::dtype_size(static_cast<int>(m->cfg.dtype));
  const size_t from = static_cast<size_t>(src_page) * pool.page_tokens * row, to = static_cast<size_t>(dst_page) * pool.page_tokens * row;
  for (auto& L : m->layers) {
    cudaMemcpyAsync(static_cast<char*>(L.k_plane) + to, static_cast<const char*>(L.k_plane) + from, tokens * row, cudaMemcpyDeviceToDevice, be->stream);
    cudaMemcpyAsync(static_cast<char*>(L.v_plane) + to, static_cast<const char*>(L.v_plane) + from, tokens * row, cudaMemcpyDeviceToDevice, be->stream);
  }
  return cuda_status(cudaGetLastError());
}

int32_t fj_dense_kv_pages(fj_dense_model* m, uint32_t layer, uint32_t plane, uint32_t first_page, uint32_t count, void* host, uint32_t to_device) {
  if (!m || !host || layer >= m->layers.size() || plane > 1) return FJ_INVALID_INPUT;
  fj_backend* be = m->be;
  const fj::KvPoolDevice& pool = m->pool->dev;
  if (first_page > pool.physical_pages || count > pool.physical_pages - first_page) return FJ_INVALID_INPUT;
  if (count == 0) return FJ_OK;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const size_t page_bytes = static_cast<size_t>(pool.page_tokens) * m->cfg.kv_heads * m->cfg.head_dim * fj::dtype_size(static_cast<int>(m->cfg.dtype));
  char* dev = static_cast<char*>(plane == 0 ? m->layers[layer].k_plane : m->layers[layer].v_plane) + first_page * page_bytes;
  if (to_device) cudaMemcpyAsync(dev, host, count * page_bytes, cudaMemcpyHostToDevice, be->stream);
  else cudaMemcpyAsync(host, dev, count * page_bytes, cudaMemcpyDeviceToHost, be->stream);
  return cuda_status(cudaStreamSynchronize(be->stream));
}

int32_t fj_dense_step_stats(fj_dense_model* m, uint64_t* kernels, uint64_t* attn_work_items) {
  if (!m) return FJ_INVALID_INPUT;
  if (kernels) *kernels = m->last_kernels;
  if (attn_work_items) *attn_work_items = m->last_work_items;
  return FJ_OK;
}

int32_t fj_dense_fill_kv(fj_dense_model* m, uint64_t seed) {
  if (!m) return FJ_INVALID_INPUT;
  fj_backend* be = m->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const size_t elements = m->plane_bytes / fj::dtype_size(static_cast<int>(m->cfg.dtype));
  const unsigned grid = static_cast<unsigned>(be->ctx.sm_count) * 16;
  for (size_t l = 0; l < m->layers.size(); ++l) {
    fill_normal_kernel<<<grid, 256, 0, be->stream>>>(m->layers[l].k_plane, static_cast<int>(m->cfg.dtype), elements, seed * 131 + 2 * l);
    fill_normal_kernel<<<grid, 256, 0, be->stream>>>(m->layers[l].v_plane, static_cast<int>(m->cfg.dtype), elements, seed * 131 + 2 * l + 1);
    be->ctx.launches += 2;
  }
  return cuda_status(cudaStreamSynchronize(be->stream));
}

int32_t fj_tcgen05_wait_giveups(fj_backend* be, uint32_t* out) {
  if (!be || !out) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  cudaStreamSynchronize(be->stream);
  *out = fj::gemm_tma_giveups() + fj::grouped_tcgen05_giveups() + fj::attn_prefill_tc5_giveups();
  return FJ_OK;
}

int32_t fj_fill_random(fj_backend* be, uint64_t buffer, uint64_t offset_bytes, uint64_t elements, uint32_t dtype, uint64_t seed, float mean, float std) {
  if (!be || dtype > FJ_U32) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  fj_buffer_rec* r = find_buffer(be, buffer);
  const uint64_t esz = fj::dtype_size(static_cast<int>(dtype));
  if (!r || r->readonly || offset_bytes % esz != 0 || offset_bytes > r->bytes || elements > (r->bytes - offset_bytes) / esz) return FJ_INVALID_INPUT;
  if (elements == 0) return FJ_OK;
  const unsigned grid = static_cast<unsigned>(be->ctx.sm_count) * 16;
  char* base = static_cast<char*>(r->ptr) + offset_bytes;
  if (dtype == FJ_U32 || dtype == FJ_I32) fill_words_kernel<<<grid, 256, 0, be->stream>>>(reinterpret_cast<unsigned*>(base), elements, seed);
  else fill_normal_kernel<<<grid, 256, 0, be->stream>>>(base, static_cast<int>(dtype), elements, seed, mean, std);
  be->ctx.launches++;
  return cuda_status(cudaGetLastError());
}

int32_t fj_dense_profile_attention(fj_dense_model* m, uint32_t enabled) {
  if (!m) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  m->profile_attention = enabled != 0;
  return FJ_OK;
}

int32_t fj_dense_attention_time(fj_dense_model* m, uint64_t* total_ns, uint64_t* launches) {
  if (!m) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  for (auto& pair : m->pending) {
    float ms = 0.0f;
    if (cudaEventSynchronize(pair.second) == cudaSuccess && cudaEventElapsedTime(&ms, pair.first, pair.second) == cudaSuccess) {
      m->attention_ns += static_cast<uint64_t>(static_cast<double>(ms) * 1.0e6);
      m->attention_launches += 1;
    } else {
      cudaGetLastError();
    }
    m->event_pool.push_back(pair.first);
    m->event_pool.push_back(pair.second);
  }
  m->pending.clear();
  if (total_ns) *total_ns = m->attention_ns;
  if (launches) *launches = m->attention_launches;
  return FJ_OK;
}

}  // extern "C"
