// Host-side launch interface of the forja sm_100a kernels. Every launcher enqueues on ctx.stream
// and bumps ctx.launches by the number of kernels it started; none of them allocates.
#pragma once

#include <atomic>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fj_common.cuh"

namespace fj {

struct Ctx {
  cudaStream_t stream;
  unsigned long long launches;  // kernels started through this context
  int sm_count;
};

// Launch with the programmatic stream-serialisation attribute (see pdl_sync in fj_common.cuh): only
// for kernels whose first statement is pdl_sync().
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
}

// Raises a kernel's dynamic shared-memory limit once per device: cudaFuncAttributeMaxDynamicSharedMemorySize
// belongs to the (function, device) pair, so a process that opens a second GPU has to opt in there too.
// One SmemOptIn per kernel instantiation (a function-local static); safe to call from several host threads.
// Returns false when the attribute call fails; the CUDA error is left pending, so the launch that follows
// fails too and the submission reports FJ_DEVICE_EXECUTION_FAILED.
struct SmemOptIn {
  std::atomic<unsigned char> done[64] = {};
};
template <typename K>
inline bool opt_in_smem(SmemOptIn& state, K kernel, int bytes) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return false;
  if (device < 0 || device >= 64) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
  if (state.done[device].load(std::memory_order_acquire)) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  state.done[device].store(1, std::memory_order_release);
  return true;
}

// ---- fj_dense_ops.cu ------------------------------------------------------------------------
// Op::Sdpa over a contiguous cache (views [heads, tokens, width], any strides) and Op::GatherMatmul over dense experts.
// false: shape outside what the kernels take (head_dim > 256, value width > 256, inner beyond 12288).
bool launch_sdpa(Ctx& ctx, const View& q, const View& k, const View& v, const View& out, float scale, bool causal, unsigned q_start);
bool launch_gather_matmul(Ctx& ctx, const View& x, const View& w, const View& idx, const View& out, ErrorRecord* err);

// ---- fj_elementwise.cu ----------------------------------------------------------------------
void launch_copy(Ctx& ctx, const View& in, const View& out, size_t elements);
void launch_fill_zero(Ctx& ctx, void* ptr, size_t bytes);
// Map programs over `shape` (views broadcast to it): add, silu_mul, rope_pairs.
void launch_add(Ctx& ctx, const View& a, const View& b, const View& out, size_t elements);
void launch_silu_mul(Ctx& ctx, const View& gate, const View& up, const View& out, size_t elements);
// Row programs: rows = elements / width, reductions over the last axis.
void launch_rms_norm(Ctx& ctx, const View& x, const View& w, const View& out, size_t rows, unsigned width, float eps);
void launch_residual_norm(Ctx& ctx, const View& residual, const View& update, const View& w, const View& sum_out,
                          const View& norm_out, size_t rows, unsigned width, float eps, int round_sum = 0);
// qk_norm_rope over the half row: inputs lo, hi, weight_lo, weight_hi, positions (all views of the
// iteration shape [.., half]); inv_freq[i] = powf(theta, i * (-2/head_dim)) precomputed on the host.
void launch_qk_norm_rope(Ctx& ctx, const View& lo, const View& hi, const View& wlo, const View& whi, const View& pos,
                         const View& out_lo, const View& out_hi, size_t rows, unsigned half, float head_dim, float eps,
                         const float* inv_freq);
// rope_pairs map program / Op::Rope: first, second halves; positions view (float or u32 dtype).
void launch_rope_pairs(Ctx& ctx, const View& first, const View& second, const View& pos, const View& out_first,
                       const View& out_second, size_t elements, unsigned half, const float* inv_freq);
void launch_embed(Ctx& ctx, const void* table, int t_dt, const unsigned* ids, void* out, int out_dt, unsigned vocab,
                  unsigned width, unsigned count, ErrorRecord* err);
void launch_quant_embed(Ctx& ctx, const unsigned* packed, const void* scales, const void* biases, int p_dt,
                        const unsigned* ids, void* out, int out_dt, unsigned vocab, unsigned packed_width, unsigned count,
                        unsigned bits, unsigned group_size, ErrorRecord* err);
// argmax under IEEE total order, ties -> highest index. scratch: rows * chunks u64.
size_t argmax_scratch_bytes(unsigned rows, unsigned width);
void launch_argmax(Ctx& ctx, const void* x, int x_dt, size_t row_stride, unsigned* out, unsigned rows, unsigned width,
                   void* scratch);
// Op::Sample / SampleMasked: params = 5 device words (temperature, top_k, top_p, seed lo, seed hi), allow = bit mask or nullptr.
// Invalid parameters or mask: ERR_INVALID in err (value = row) and token 0.
void launch_sample(Ctx& ctx, const void* x, int x_dt, size_t row_stride, const unsigned* params, const unsigned* allow, unsigned* out, unsigned rows, unsigned width,
                   unsigned position, ErrorRecord* err);
// top-k: descending total order, ties -> lower index; optional softmax over the selected set.
void launch_top_k(Ctx& ctx, const void* x, int x_dt, void* values, int v_dt, unsigned* indices, unsigned rows,
                  unsigned width, unsigned k, bool normalize);
// Fused q/k RMS-norm + RoPE + KV append for the dense step. qkv [rows, (hq + 2 kvh) * d] in `dt`;
// q_out [rows, hq, d]; K/V rows go to the planes at slot_mapping[row] (slot 0xFFFFFFFF = skip).
// qk_norm == 0: plain half-split RoPE with inv_freq (Op::Rope semantics, u32 positions).
void launch_qknorm_rope_append(Ctx& ctx, const void* qkv, int dt, const void* q_norm_w, const void* k_norm_w,
                               const unsigned* positions, const unsigned* slot_mapping, void* q_out, void* k_plane,
                               void* v_plane, unsigned rows, unsigned q_heads, unsigned kv_heads, unsigned head_dim,
                               float eps, const float* inv_freq, int qk_norm, unsigned plane_slots);

// ---- fj_paged.cu ----------------------------------------------------------------------------
// One sequence (lane) of a ragged attention launch. Pointers are device addresses.
struct AttnSeq {
  const void* q;                // first query row of the lane
  void* out;
  const unsigned* table;        // [table_pages][2] {page, generation}
  const unsigned* activity;     // one word or nullptr (= active)
  unsigned q_len, q_start, key_length, table_pages;
  unsigned long long q_tok_stride, q_head_stride, o_tok_stride, o_head_stride;  // elements
  unsigned causal;
  unsigned err_index;           // which record of the launch's error array this lane reports to (its dispatch within a coalesced run)
};
// One lane of a batched single-token append (PagedSdpaAppend's copy half, crates/forja-cpu/src/lib.rs:262-307).
struct AppendLane {
  const void* k_new;            // [kv_heads * head_dim] and [kv_heads * value_dim] rows of the new token
  const void* v_new;
  const unsigned* table;
  const unsigned* activity;     // one word or nullptr (= active)
  unsigned table_pages, q_start, err_index;
  int k_dtype, v_dtype;
};
struct AttnWork {
  unsigned seq, kv_head, t_begin, t_end, split, n_splits, slot, group_index;
};
struct AttnGeometry {
  unsigned q_heads, kv_heads, head_dim, value_dim, page_tokens, physical_pages;
  int q_dtype, kv_dtype, out_dtype;
  float scale;
};
// Scratch layout for split-K partials (device memory owned by the caller).
struct AttnScratch {
  float* part_o;        // [slots][16][head_dim]
  float* part_ml;       // [slots][2][16]
  unsigned* counters;   // [groups] (zero before first use; kernels leave them zero)
};
size_t attn_part_o_bytes(unsigned slots, unsigned head_dim);
size_t attn_part_ml_bytes(unsigned slots);
// Decode / short-query attention on tensor cores: requires q_len * (q_heads / kv_heads) <= 16,
// head_dim == value_dim == 128, page_tokens == 16, 16-bit q/kv dtypes (same type).
bool attn_decode_mma_supported(const AttnGeometry& g, unsigned max_q_len);
void launch_attn_decode_mma(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, const AttnWork* work, unsigned n_work,
                            const void* kpool, const void* vpool, const unsigned* generations, const AttnScratch& scratch,
                            ErrorRecord* err, const unsigned* n_work_dev = nullptr);
// n_work_dev: optional device word holding the live item count; CTAs beyond it return at once, so a launch recorded
// once with a rounded-up grid (a replayed CUDA graph) serves steps whose work lists differ in length.
// Chunked-prefill attention on tensor cores for any q_len (tcgen05, fj_attn_tc5.cu): 16-bit q/kv of one type, head_dim ==
// value_dim == 128, 16-token pages, q_heads / kv_heads dividing 128. One CTA per item {sequence, first token of a block of
// attn_prefill_tokens_per_block tokens} and KV head (128 rows = tokens x query heads of the group); the caller lists every
// block of every sequence. The *_mma names are the entry points the callers use; they forward to the tcgen05 kernel.
bool attn_prefill_mma_supported(const AttnGeometry& g);
unsigned attn_prefill_tokens_per_block(const AttnGeometry& g);
bool attn_prefill_tc5_supported(const AttnGeometry& g);
unsigned attn_prefill_tc5_tokens_per_block(const AttnGeometry& g);
void launch_attn_prefill_tc5(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, const uint2* items, unsigned n_items, const void* kpool, const void* vpool,
                             const unsigned* generations, ErrorRecord* err);
unsigned attn_prefill_tc5_giveups();
void launch_attn_prefill_mma(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, const uint2* items, unsigned n_items, const void* kpool, const void* vpool,
                             const unsigned* generations, ErrorRecord* err);
// Generic f32-math attention for any float dtypes, head_dim <= 256, any q_len (one CTA per
// (sequence, head, query row)); used for f32 models and odd shapes.
void launch_attn_generic(Ctx& ctx, const AttnGeometry& g, const AttnSeq* seqs, unsigned n_seqs, unsigned max_q_len,
                         const void* kpool, const void* vpool, const unsigned* generations, ErrorRecord* err);
// Single-token appends of many lanes in one launch: lane i writes its new K and V rows at logical position q_start through its
// authenticated page table, or reports ERR_PAGE to err[err_index] and writes nothing.
void launch_paged_append_batch(Ctx& ctx, const AppendLane* lanes, unsigned count, void* kpool, void* vpool, int pool_dt, const unsigned* generations,
                               unsigned physical_pages, unsigned page_tokens, unsigned k_elements, unsigned v_elements, ErrorRecord* err);
// Split-K work list of a ragged decode launch, built on the device from the lanes' descriptors: chunks of `chunk` tokens per
// (lane, kv head), in lane-major, head, split order (the order the host loop used to upload).
void launch_build_work_from_seqs(Ctx& ctx, const AttnSeq* seqs, unsigned count, unsigned kv_heads, unsigned chunk, AttnWork* work, unsigned work_cap);
// Paged copy of `tokens` rows between an ordinary [tokens, elements] tensor and a plane.
void launch_paged_copy(Ctx& ctx, bool into_pages, void* ordinary, int o_dt, size_t o_row_stride, void* pool, int p_dt,
                       const unsigned* table, unsigned table_pages, const unsigned* generations, unsigned physical_pages,
                       unsigned start, unsigned tokens, unsigned page_tokens, unsigned elements, const unsigned* activity,
                       ErrorRecord* err);

// ---- fj_gemm.cu -----------------------------------------------------------------------------
// C[M,N] = A[M,K] * W[N,K]^T ("NT": both operands K-major), f32 accumulation, output rounded once.
// lda/ldw/ldc in elements. 16-bit path: the TMA-fed tcgen05 kernel for M > 16 (mma.sync split-K tiles when its
// alignment rules are not met), warp-per-column GEMV at 16 rows or fewer.
size_t gemm_scratch_bytes(unsigned m, unsigned n, unsigned k);
void launch_gemm_nt(Ctx& ctx, const void* a, int a_dt, size_t lda, const void* w, int w_dt, size_t ldw, void* c, int c_dt,
                    size_t ldc, unsigned m, unsigned n, unsigned k, void* scratch, size_t scratch_bytes);
// TMA-fed, warp-specialised tcgen05 GEMM (fj_gemm_tma.cu): 128 x {32, 64, 128, 256} tiles, one producer thread issuing
// cp.async.bulk.tensor loads, one thread issuing the MMAs, four epilogue warps. false from the launcher: no tensor map
// could be made (the caller takes another kernel).
bool gemm_nt_tma_supported(int a_dt, int w_dt, unsigned m, unsigned n, unsigned k, size_t lda, size_t ldw, const void* a, const void* w);
bool launch_gemm_nt_tma(Ctx& ctx, const void* a, int a_dt, size_t lda, const void* w, size_t ldw, void* c, int c_dt, size_t ldc, unsigned m, unsigned n, unsigned k);
unsigned gemm_tma_giveups();  // bounded waits that ran out since the library was loaded (0 in a healthy run)
unsigned grouped_tcgen05_giveups();  // the same for the expert-bucketed tcgen05 tiles
// Fully strided fallback (any layout, batch): one thread per output element.
void launch_matmul_generic(Ctx& ctx, const View& a, const View& b, const View& c, unsigned batch, unsigned m, unsigned n,
                           unsigned k);

// ---- fj_quant.cu ----------------------------------------------------------------------------
// y[m,n] = sum_k x[m,k] * (scale[n,k/g] * q[n,k] + bias[n,k/g]); packed u32 [N, K*bits/32], LSB first.
void launch_quant_matmul(Ctx& ctx, const void* x, int x_dt, const unsigned* packed, const void* scales, const void* biases,
                         int p_dt, void* out, int out_dt, unsigned m, unsigned k, unsigned n, unsigned bits,
                         unsigned group_size, void* workspace = nullptr, size_t workspace_bytes = 0, void* gemm_scratch = nullptr,
                         size_t gemm_scratch_bytes = 0);
// epilogue: 0 none; 1 silu(acc0) * acc1 (pair form); 2 acc0 + extra (weighted-sum form)
void launch_gather_quant_matmul(Ctx& ctx, const void* x, int x_dt, const unsigned* packed, const void* scales,
                                const void* biases, int p_dt, const unsigned* packed2, const void* scales2,
                                const void* biases2, const unsigned* indices, void* out, int out_dt, unsigned rows,
                                unsigned k, unsigned experts, unsigned n, unsigned routes, unsigned bits, unsigned group_size,
                                int epilogue, ErrorRecord* err);
void launch_gather_quant_weighted_sum(Ctx& ctx, const void* act, int a_dt, const unsigned* packed, const void* scales,
                                      const void* biases, int p_dt, const unsigned* indices, const void* weights, int w_dt,
                                      const void* extra, int e_dt, void* out, int out_dt, unsigned rows, unsigned routes,
                                      unsigned k, unsigned experts, unsigned n, unsigned bits, unsigned group_size,
                                      int epilogue, ErrorRecord* err);

// ---- fj_grouped.cu --------------------------------------------------------------------------
// Routes bucketed by expert and cut into tiles of tile_rows rows (64 for the tile GEMMs, 16 for the streaming form); `plan` is caller-owned device memory of
// route_plan_bytes(total_routes, experts). Ids >= experts are left out of every bucket.
size_t route_plan_bytes(unsigned total_routes, unsigned experts);
void launch_route_plan(Ctx& ctx, const unsigned* indices, unsigned total_routes, unsigned experts, void* plan, ErrorRecord* err, unsigned tile_rows = 64,
                       const unsigned* slab_counts = nullptr, unsigned slab_cap = 0, unsigned slab_offset = 0, unsigned slab_limit = 0);
bool grouped_q4_supported(unsigned k, unsigned n, unsigned bits, unsigned group_size, unsigned experts, const void* x, const void* packed);
// Rows per tile (64 or 128) the tile GEMMs should use for this many routes; pass it to launch_route_plan and to both launchers.
unsigned grouped_tile_rows(unsigned total_routes, unsigned experts);
// act_out[route, :] = silu(x_r . gate_e) * (x_r . up_e) in bf16, x_r = x[route / src_div]; bf16 x, bf16 scales/biases, group 64.
void launch_grouped_q4_pair(Ctx& ctx, const void* x, const unsigned* gate, const void* gate_scales, const void* gate_biases, const unsigned* up, const void* up_scales,
                            const void* up_biases, const void* plan, unsigned total_routes, unsigned experts, unsigned src_div, void* act_out, unsigned k, unsigned n,
                            unsigned tile_rows = 64);
// out[route, :] = x[route / src_div] . W_e, f32 or (out_bf16) bf16.
void launch_grouped_q4_single(Ctx& ctx, const void* x, const unsigned* packed, const void* scales, const void* biases, const void* plan, unsigned total_routes, unsigned experts,
                              unsigned src_div, void* out, bool out_bf16, unsigned k, unsigned n, unsigned tile_rows = 64);
// Streaming form of the two launchers above for few rows per expert; the plan must have been made with tile_rows = 16.
// live_routes (only a hint for the grid): how many of the routes are expected to carry a valid expert id.
// false: the kernel could not be configured on this device and nothing was launched.
bool expert_stream_supported(unsigned k, unsigned n, unsigned bits, unsigned group_size, unsigned experts, const void* x, const void* packed, const void* scales, const void* biases);
bool launch_expert_stream_pair(Ctx& ctx, const void* x, const unsigned* gate, const void* gate_scales, const void* gate_biases, const unsigned* up, const void* up_scales,
                               const void* up_biases, const void* plan, unsigned total_routes, unsigned experts, unsigned src_div, void* act_out, unsigned k, unsigned n,
                               unsigned live_routes = 0xFFFFFFFFu);
bool launch_expert_stream_single(Ctx& ctx, const void* x, const unsigned* packed, const void* scales, const void* biases, const void* plan, unsigned total_routes, unsigned experts,
                                 unsigned src_div, void* out, bool out_bf16, unsigned k, unsigned n, unsigned live_routes = 0xFFFFFFFFu);
// out[row] = (extra[row] +) sum_j weights[row, j] * per_route[slot], j ascending (slot = route_slot[row, j], or the route itself);
// per_route rows are f32 or bf16 (p_dt).
void launch_routes_combine(Ctx& ctx, const void* per_route, int p_dt, const unsigned* route_slot, const unsigned* expert_ids, unsigned experts, const void* weights, int w_dt, const void* extra,
                           int e_dt, void* out, int out_dt, unsigned rows, unsigned top_k, unsigned width);

// ---- fj_pack.cu -----------------------------------------------------------------------------
struct KvPoolDevice {
  unsigned* free_stack;   // [physical_pages]; top at free_count - 1
  unsigned* free_count;   // [1]
  unsigned* generations;  // [physical_pages]
  unsigned* tables;       // [lanes][table_pages][2]
  unsigned* lane_pages;   // [lanes] pages bound to each lane
  unsigned* refcounts;    // [physical_pages] owners of each page (0 = free)
  unsigned* immutable;    // [lanes][table_pages] 1 = this lane must not write the page (shared prefix)
  unsigned physical_pages, lanes, table_pages, page_tokens;
};
void launch_kvpool_init(Ctx& ctx, const KvPoolDevice& pool);
void launch_kvpool_reserve(Ctx& ctx, const KvPoolDevice& pool, const unsigned* lanes, const unsigned* tokens, unsigned count,
                           int* status);
void launch_kvpool_release(Ctx& ctx, const KvPoolDevice& pool, const unsigned* lanes, unsigned count);
// args (device) = {src lane, dst lane, prefix tokens, reserved tokens}; *status (device) = 0 / 1 quota / 3 overflow / 7 invalid.
void launch_kvpool_fork(Ctx& ctx, const KvPoolDevice& pool, const unsigned* args, int* status);
// args (device) = {lane, logical length}; result (device) = {status, copied, src page, dst page, tokens to copy}.
void launch_kvpool_cow_tail(Ctx& ctx, const KvPoolDevice& pool, const unsigned* args, int* result);
struct PackOutputs {
  unsigned *logical_lengths, *query_starts, *absolute_positions, *activity, *cu_seqlens, *positions, *slot_mapping, *row_lane;
};
// rewind check / checkpoint / rollback / checkpoint drop on the device pool; see kvpool_boundary_kernel for the argument words.
void launch_kvpool_boundary(Ctx& ctx, const KvPoolDevice& pool, const unsigned* args, int* result);
void launch_pack_step(Ctx& ctx, const KvPoolDevice& pool, const unsigned* starts, const unsigned* tokens, unsigned lanes,
                      const PackOutputs& out, unsigned rows_cap);
// Builds AttnSeq / AttnWork lists for the dense step from packed metadata (one CTA).
void launch_build_attn_lists(Ctx& ctx, const KvPoolDevice& pool, const PackOutputs& pack, unsigned lanes, unsigned kv_heads,
                             unsigned chunk_tokens, const void* q_base, void* out_base, unsigned q_heads, unsigned head_dim,
                             int elem_bytes, AttnSeq* seqs, AttnWork* work, unsigned* n_work, unsigned work_cap);

}  // namespace fj
