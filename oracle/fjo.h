/*
 * forja-cpu oracle: C ABI of the CPU restatement of forja's reference backend.
 *
 * TEST INFRASTRUCTURE ONLY. This library is the checker for the CUDA path: only the tests,
 * the smoke check and the CPU-baseline leg of the benchmark may load it. The product
 * library (libforja_cuda.so) never links, loads or calls anything declared here.
 *
 * Parity status: pinned. The arithmetic lives in-tree in the reference
 * (crates/forja-cpu/src/{lib,paged,interpreter}.rs, crates/forja-core/src/{paged,paged_pool}.rs,
 * crates/forja-serve/src/scheduler.rs); its only numeric dependency is the `half` crate 2.7.1
 * (round-to-nearest-even f32<->f16/bf16), restated in fjo_convert.h. Every function below is
 * checked against the known-answer vectors of the reference's own unit tests.
 *
 * Conventions: every tensor argument is the contiguous logical byte image of the tensor (what
 * the reference's `read()` gathers), together with a dtype code. All arithmetic is f32 on values
 * decoded from storage, accumulation is sequential in index order, and every output is rounded
 * once to its dtype (crates/forja-cpu/src/lib.rs:484-493, 1790-1847).
 */
#ifndef FJO_H
#define FJO_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes, in the order of wit/compute.wit:4-10 */
enum { FJO_F32 = 0, FJO_F16 = 1, FJO_BF16 = 2, FJO_I32 = 3, FJO_U32 = 4 };

/* status codes (subset of BackendError, crates/forja-core/src/backend.rs:362-426) */
enum {
  FJO_OK = 0,
  FJO_INVALID_INPUT = 1,
  FJO_EXECUTION_FAILED = 2,
  FJO_INDEX_OUT_OF_RANGE = 3, /* *bad_index holds the lowest offending index */
  FJO_QUOTA_EXCEEDED = 4,
  FJO_ARITHMETIC_OVERFLOW = 5,
  FJO_UNRESERVED_WRITE = 6,
  FJO_SHARED_TAIL = 7,
  FJO_BANK_IN_FLIGHT = 8,
  FJO_FOREIGN_RESOURCE = 9,
  FJO_INVALID_CHECKPOINT = 10,
  FJO_CORRUPT_STATE = 11,
  FJO_EMPTY_SLAB = 12
};

size_t fjo_dtype_size(int dtype);
void fjo_set_threads(int threads); /* OpenMP threads for the row/column-parallel loops; 1 = faithful */
int fjo_get_max_threads(void);

/* encode/decode, crates/forja-cpu/src/lib.rs:1790-1847 */
int fjo_decode(const void* src, int dtype, float* dst, size_t n);
int fjo_encode(const float* src, void* dst, int dtype, size_t n);

/* Op::Copy, lib.rs:171-187 */
int fjo_copy(const void* in, int in_dt, void* out, int out_dt, size_t n);
/* Op::RmsNorm, lib.rs:495-517 */
int fjo_rms_norm(const void* x, int x_dt, const void* w, int w_dt, void* out, int out_dt,
                 size_t rows, size_t width, float eps);
/* Op::Argmax, lib.rs:519-550 (ties -> highest index, IEEE total order) */
int fjo_argmax(const void* x, int x_dt, uint32_t* out, size_t rows, size_t width);
/* Op::TopK, lib.rs:552-608 */
int fjo_top_k(const void* x, int x_dt, void* values, int v_dt, uint32_t* indices, size_t rows,
              size_t width, uint32_t k, int normalize);
/* Op::Sample / SampleMasked, lib.rs:610-678, 1545-1700. params = 5 words; allow may be NULL */
int fjo_sample(const void* x, int x_dt, const uint32_t* params, const uint32_t* allow,
               uint32_t* out, size_t rows, size_t width, uint32_t position);
/* Op::Rope, lib.rs:681-710. x is [tokens, heads, width]; positions u32 [tokens] */
int fjo_rope(const void* x, int x_dt, const uint32_t* positions, void* out, int out_dt,
             size_t tokens, size_t heads, size_t width, float theta);
/* Op::Embed, lib.rs:712-745 */
int fjo_embed(const void* table, int t_dt, const uint32_t* ids, void* out, int out_dt,
              size_t vocab, size_t width, size_t count, uint32_t* bad_index);
/* Op::QuantEmbed, lib.rs:748-813 */
int fjo_quant_embed(const uint32_t* packed, const void* scales, const void* biases, int p_dt,
                    const uint32_t* ids, void* out, int out_dt, size_t vocab, size_t packed_width,
                    size_t count, uint32_t bits, uint32_t group_size, uint32_t* bad_index);
/* Op::Matmul, lib.rs:815-848. left [batch, rows, inner]; right [batch, inner, cols] logical.
 * right_transposed != 0: `right` is stored as [batch, cols, inner] (the same k-ascending
 * accumulation, cache-friendly; bit-identical results). */
int fjo_matmul(const void* left, int l_dt, const void* right, int r_dt, void* out, int out_dt,
               size_t batch, size_t rows, size_t inner, size_t cols, int right_transposed);
/* Op::QuantMatmul, lib.rs:914-962 + affine_quant_dot :1277-1310 */
int fjo_quant_matmul(const void* x, int x_dt, const uint32_t* packed, const void* scales,
                     const void* biases, int p_dt, void* out, int out_dt, size_t rows,
                     size_t inner, size_t cols, uint32_t bits, uint32_t group_size);
/* Op::GatherQuantMatmul 5-input projection, lib.rs:1025-1106. out [rows, k, cols] */
int fjo_gather_matmul(const void* x, int x_dt, const void* weights, int w_dt, const uint32_t* indices, void* out, int out_dt,
                      size_t rows, size_t inner, size_t experts, size_t cols, size_t routes, uint32_t* bad_index);
int fjo_gather_quant_matmul(const void* x, int x_dt, const uint32_t* packed, const void* scales,
                            const void* biases, int p_dt, const uint32_t* indices, void* out,
                            int out_dt, size_t rows, size_t inner, size_t experts, size_t cols,
                            size_t k, uint32_t bits, uint32_t group_size, uint32_t* bad_index);
/* Op::GatherQuantMatmul 6-input weighted sum, lib.rs:1108-1204. act [rows, routes, inner];
 * out [rows, cols] (before any epilogue; pass out_dt F32 to obtain raw accumulators) */
int fjo_gather_quant_weighted_sum(const void* act, int a_dt, const uint32_t* packed,
                                  const void* scales, const void* biases, int p_dt,
                                  const uint32_t* indices, const void* weights, int w_dt,
                                  void* out, int out_dt, size_t rows, size_t routes, size_t inner,
                                  size_t experts, size_t cols, uint32_t bits, uint32_t group_size,
                                  uint32_t* bad_index);
/* Op::Sdpa (contiguous cache), lib.rs:1206-1273. q [hq, T, d]; k [kvh, L, d]; v [kvh, L, dv] */
int fjo_sdpa(const void* q, int q_dt, const void* k, int k_dt, const void* v, int v_dt, void* out,
             int out_dt, size_t q_heads, size_t q_len, size_t width, size_t kv_heads,
             size_t kv_len, size_t value_width, float scale, int causal, uint32_t q_start);

/* Scalar program interpreter, crates/forja-cpu/src/interpreter.rs:38-396.
 * insts: n_insts x 4 words {tag, a, b, c}; tags: 0 Input(slot) 1 Const(f32 bits) 2 Index(axis)
 * 3 Extent(axis) 4 Unary(op, x) 5 Binary(op, l, r) 6 Select(c, t, f) 7 Cast(type, x)
 * 8 Reduce(op, x). kind: 0 Map, 1 Row. inputs: contiguous logical arrays already broadcast to
 * `shape`, dtype codes per input (floats decoded to f32, U32 kept). outputs: one array per slot. */
int fjo_program(int kind, const uint32_t* insts, size_t n_insts, const uint32_t* outputs /*slot,inst*/,
                size_t n_outputs, const uint32_t* shape, size_t rank, const void* const* inputs,
                const int* input_dtypes, size_t n_inputs, void* const* outs, const int* out_dtypes);

/* Direct restatements of the guest programs of crates/forja-sdk/src/nn/blocks.rs:380-444 with
 * the interpreter's evaluation order (bit-identical to fjo_program on the same IR). */
int fjo_prog_rms_norm(const void* x, int dt, const void* w, int w_dt, void* out, int out_dt,
                      size_t rows, size_t width, float eps);
int fjo_prog_residual_norm(const void* residual, const void* update, int dt, const void* w, int w_dt,
                           void* sum_out, void* norm_out, int out_dt, size_t rows, size_t width,
                           float eps);
int fjo_prog_add(const void* a, const void* b, int dt, void* out, int out_dt, size_t n);
int fjo_prog_silu_mul(const void* gate, const void* up, int dt, void* out, int out_dt, size_t n);
/* x [tokens, heads, 2*half] split lo/hi; weight [2*half] or [heads, 2*half] (per_head_weight);
 * positions f32 [tokens] */
int fjo_prog_qk_norm_rope(const void* x, int dt, const void* w, int w_dt, int per_head_weight,
                          const float* positions, void* out, int out_dt, size_t tokens,
                          size_t heads, size_t width, float eps, float theta);

/* Paged storage, crates/forja-cpu/src/paged.rs + lib.rs:189-380, 1519-1535.
 * table: table_pages x {page, generation}; generations: [physical_pages]. pool planes are
 * [physical_pages, page_tokens, elements]. activity: NULL or one u32. */
int fjo_paged_copy(int into_pages, void* ordinary, int o_dt, void* pool, int p_dt,
                   const uint32_t* table, size_t table_pages, const uint32_t* generations,
                   size_t physical_pages, uint32_t start, uint32_t tokens, uint32_t page_tokens,
                   size_t elements, const uint32_t* activity);
/* q/out [hq, T, d] logical */
int fjo_paged_sdpa(const void* q, int q_dt, const void* kpool, int k_dt, const void* vpool, int v_dt,
                   const uint32_t* table, size_t table_pages, const uint32_t* generations,
                   size_t physical_pages, void* out, int out_dt, uint32_t q_heads, uint32_t q_len,
                   uint32_t kv_heads, uint32_t width, uint32_t value_width, uint32_t key_length,
                   uint32_t q_start, float scale, int causal, uint32_t page_tokens,
                   const uint32_t* activity);
/* Op::PagedSdpaAppend, lib.rs:262-306: k_new [1, kvh, d], v_new [1, kvh, dv] */
int fjo_paged_sdpa_append(const void* q, int q_dt, const void* k_new, int kn_dt, const void* v_new,
                          int vn_dt, void* kpool, int k_dt, void* vpool, int v_dt,
                          const uint32_t* table, size_t table_pages, const uint32_t* generations,
                          size_t physical_pages, void* out, int out_dt, uint32_t q_heads,
                          uint32_t kv_heads, uint32_t width, uint32_t value_width, uint32_t q_start,
                          float scale, uint32_t page_tokens, const uint32_t* activity);
/* PagedLayout::plane_page_bytes, crates/forja-core/src/paged.rs:258-298 */
int fjo_paged_layout_page_bytes(uint32_t page_tokens, int dtype, uint64_t elements_per_token,
                                uint64_t alignment, uint64_t* page_bytes);
/* PageTable::resolve on a padded table, paged.rs:97-163: 0 ok, 1 logical OOB, 2 physical OOB, 3 stale */
int fjo_page_table_resolve(const uint32_t* table, size_t table_pages, const uint32_t* generations,
                           size_t physical_pages, uint32_t logical_page, uint32_t* physical);

/* Allocator, crates/forja-core/src/paged_pool.rs. One plane-geometry number stands for the
 * layout: total_page_bytes (sum of aligned page bytes over planes). */
typedef struct fjo_pool fjo_pool;
typedef struct fjo_seq fjo_seq;
typedef struct fjo_checkpoint fjo_checkpoint;
typedef struct fjo_banks fjo_banks;
int fjo_pool_new(uint32_t page_tokens, uint64_t total_page_bytes, uint32_t pages_per_slab,
                 uint64_t byte_limit, int fixed, fjo_pool** out);
void fjo_pool_free(fjo_pool*);
int fjo_pool_observe_completion(fjo_pool*, uint64_t serial);
int fjo_pool_reserve(fjo_pool*, uint64_t tokens, fjo_seq** out);
int fjo_pool_memory(fjo_pool*, uint64_t usage[5] /*slab,table,slot,graph,scratch*/, uint64_t* limit);
int fjo_pool_set_graph_arena_bytes(fjo_pool*, uint64_t bytes);
int fjo_pool_set_scratch_bytes(fjo_pool*, uint64_t primary, uint64_t overlap);
size_t fjo_pool_physical_pages(fjo_pool*);
int fjo_pool_generations(fjo_pool*, uint32_t* out, size_t n);
size_t fjo_pool_free_list(fjo_pool*, uint32_t* out, size_t cap);
int fjo_pool_debug_set_generation(fjo_pool*, uint32_t page, uint32_t generation);
void fjo_seq_drop(fjo_seq*);
uint64_t fjo_seq_logical_len(fjo_seq*);
uint64_t fjo_seq_reserved_tokens(fjo_seq*);
size_t fjo_seq_pages(fjo_seq*);
int fjo_seq_table(fjo_seq*, uint32_t* entries /* pages x 2 */, size_t cap_pages);
int fjo_seq_refcounts(fjo_seq*, uint32_t* out, size_t cap_pages);
int fjo_seq_validate_write(fjo_seq*, uint64_t start, uint64_t tokens);
int fjo_seq_validate_append(fjo_seq*, uint64_t win_start, uint64_t win_end, uint64_t start, uint64_t tokens);
int fjo_seq_commit_write(fjo_seq*, uint64_t tokens);
int fjo_seq_rewind_private(fjo_seq*, uint64_t logical_len);
int fjo_seq_mark_submitted(fjo_seq*, uint64_t serial);
int fjo_seq_fork_reserved(fjo_seq*, uint64_t prefix, uint64_t reserved, fjo_seq** out);
/* cow: *copied = 0/1; src/dst physical pages and token_count */
int fjo_seq_cow_tail(fjo_seq*, int* copied, uint32_t* src, uint32_t* dst, uint32_t* token_count);
int fjo_seq_checkpoint(fjo_seq*, fjo_checkpoint** out);
int fjo_seq_rollback(fjo_seq*, fjo_checkpoint*); /* consumes the checkpoint */
int fjo_checkpoint_belongs_to(fjo_checkpoint*, fjo_seq*);
void fjo_checkpoint_drop(fjo_checkpoint*);
int fjo_banks_new(fjo_pool*, size_t lanes, size_t table_pages, fjo_banks** out);
void fjo_banks_free(fjo_banks*);
int fjo_banks_bind(fjo_banks*, size_t bank, size_t lane, fjo_seq*);
int fjo_banks_bind_all(fjo_banks*, size_t lane, fjo_seq*);
int fjo_banks_poison(fjo_banks*, size_t bank, size_t lane);
int fjo_banks_open_append(fjo_banks*, size_t bank, size_t lane, uint64_t start, uint64_t logical_len);
int fjo_banks_mark_submitted(fjo_banks*, size_t bank, uint64_t serial);
/* slot snapshot: table entries [table_pages x 2], info {logical_len, append_start, active} */
int fjo_banks_slot(fjo_banks*, size_t bank, size_t lane, uint32_t* entries, uint64_t info[3]);

/* Scheduler, crates/forja-serve/src/scheduler.rs:16-196 */
typedef struct fjo_sched fjo_sched;
int fjo_sched_new(const uint32_t* buckets, size_t n, size_t active_limit, size_t prefill_limit,
                  uint32_t prompt_budget, uint32_t idle_prompt_budget, fjo_sched** out);
void fjo_sched_free(fjo_sched*);
void fjo_sched_chunk_multiple(fjo_sched*, uint32_t multiple);
void fjo_sched_enqueue(fjo_sched*, uint64_t id, uint64_t reserved_tokens);
void fjo_sched_reconcile_active(fjo_sched*, size_t active);
void fjo_sched_complete(fjo_sched*, uint64_t id);
void fjo_sched_retry_admission(fjo_sched*, uint64_t id, uint64_t reserved_tokens);
/* reserve predicate: admission succeeds when reserved_tokens < reserve_below */
size_t fjo_sched_admit_below(fjo_sched*, uint64_t reserve_below, uint64_t* ids, size_t cap);
/* reserve predicate driven by a pool: succeeds when pool pages remain (fixed-capacity accounting) */
size_t fjo_sched_admit_pages(fjo_sched*, uint32_t page_tokens, uint64_t* free_pages, uint64_t* ids, size_t cap);
int64_t fjo_sched_decode_bucket(fjo_sched*, const uint32_t* slots, size_t n);
void fjo_sched_ready_prompt(fjo_sched*, uint64_t id, uint32_t tokens);
size_t fjo_sched_prompt_batch(fjo_sched*, int decoding, uint64_t* ids, uint32_t* spend, size_t cap);
/* PromptChunking, crates/forja-host/src/prompt.rs:20-41 */
uint32_t fjo_chunk_work(uint32_t piece, uint32_t remaining, uint32_t allowance);
uint32_t fjo_chunk_merged_work(uint32_t piece, uint32_t remaining, uint32_t allowance);
/* reservations_fit, crates/forja-serve/src/engine/continuous/batch.rs:1139-1152 */
int fjo_reservations_fit(uint32_t page_tokens, uint32_t max_context, const uint64_t* reservations, size_t n);
/* prefill_plan, crates/forja-sdk/src/nn/blocks.rs:892-911: returns piece count, pieces in out */
size_t fjo_prefill_plan(uint32_t sequence, uint32_t chunk, uint32_t tail_chunk, uint32_t* out, size_t cap);
/* Ragged-batch packer reference: per-lane (start, tokens) or inactive -> metadata of
 * write_paged_lane_metadata (crates/forja-host/src/lib.rs:4977-5065) plus the derived
 * cu_seqlens / positions / slot_mapping / row_lane the CUDA packer emits.
 * lanes_start/lanes_tokens [lanes] (tokens == 0 -> inactive); tables [lanes, table_pages, 2].
 * Outputs: logical_lengths, query_starts, absolute_positions, activity [lanes];
 * cu_seqlens [lanes+1]; positions, slot_mapping, row_lane [rows]; returns rows or -1. */
int64_t fjo_pack_step(const uint32_t* lanes_start, const uint32_t* lanes_tokens,
                      const uint32_t* lanes_logical_len, size_t lanes, const uint32_t* tables,
                      size_t table_pages, uint32_t page_tokens, uint32_t* logical_lengths,
                      uint32_t* query_starts, uint32_t* absolute_positions, uint32_t* activity,
                      uint32_t* cu_seqlens, uint32_t* positions, uint32_t* slot_mapping,
                      uint32_t* row_lane, size_t rows_cap);

#ifdef __cplusplus
}
#endif
#endif
