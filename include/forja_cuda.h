/*
 * forja_cuda.h - C ABI of libforja_cuda.so, the sm_100a backend library behind forja's
 * `forja_core::Backend` / `Submission` traits (reference: crates/forja-core/src/backend.rs:609-984).
 *
 * A Rust `forja-cuda` crate implements `Backend` by forwarding to these entry points; views stay
 * pure layout arithmetic on the caller's side (crates/forja-core/src/layout.rs) and cross the
 * boundary as `fj_tensor` descriptors. Every function returns an `fj_status`; results come back
 * through out-parameters. There is no CPU fallback: a backend cannot be created without a CUDA
 * device, and unsupported operations answer FJ_UNSUPPORTED_OPERATION.
 *
 * Threading: one backend may be used from several host threads; calls serialise on an internal
 * mutex (the reference CPU backend does the same, crates/forja-cpu/src/lib.rs:22-24).
 * Submissions of one backend execute in submission order on one CUDA stream.
 */
#ifndef FORJA_CUDA_H
#define FORJA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums -------------------------------------------------------------------------------- */

/* BackendError, crates/forja-core/src/backend.rs:362-426 */
typedef enum fj_status {
  FJ_OK = 0,
  FJ_QUOTA_EXCEEDED = 1,
  FJ_ALLOCATION_FAILED = 2,
  FJ_EXECUTION_FAILED = 3,
  FJ_DEVICE_EXECUTION_FAILED = 4, /* fj_device_error.code = cudaError_t */
  FJ_DEVICE_ERROR_FLAG = 5,       /* data-dependent error reported by a kernel, see fj_sub_error */
  FJ_TIMEOUT = 6,
  FJ_INVALID_INPUT = 7,
  FJ_UNSUPPORTED_OPERATION = 8,
  FJ_INDEX_OUT_OF_RANGE = 9,      /* fj_device_error.value = lowest offending index */
  /* WeightError, crates/forja-host/src/weights.rs:337-358 (returned by the fj_safetensors_* calls only) */
  FJ_WEIGHTS_IO = 20,
  FJ_WEIGHTS_NOT_REGULAR_FILE = 21,
  FJ_WEIGHTS_MAPPING = 22,
  FJ_WEIGHTS_TRUNCATED = 23,
  FJ_WEIGHTS_INVALID_HEADER = 24,
  FJ_WEIGHTS_INVALID_INDEX = 25,
  FJ_WEIGHTS_HEADER_TOO_LARGE = 26,
  FJ_WEIGHTS_UNSUPPORTED_DTYPE = 27,
  FJ_WEIGHTS_INVALID_RANGE = 28,
  FJ_WEIGHTS_OVERLAPPING_RANGES = 29,
  /* PagePoolError, crates/forja-core/src/paged_pool.rs:30-70 (returned by the fj_kvpool_* boundary calls only) */
  FJ_POOL_SHARED_TAIL = 30,
  FJ_POOL_INVALID_CHECKPOINT = 31,
  FJ_POOL_CORRUPT_STATE = 32
} fj_status;

/* dtype, wit/compute.wit:4-10 */
typedef enum fj_dtype { FJ_F32 = 0, FJ_F16 = 1, FJ_BF16 = 2, FJ_I32 = 3, FJ_U32 = 4 } fj_dtype;

/* Op, crates/forja-core/src/ops.rs:163-302 (Op::State, the recurrent-state update, is not on this path) */
typedef enum fj_op {
  FJ_OP_PROGRAM = 1,            /* program = handle from fj_program_prepare */
  FJ_OP_COPY = 2,
  FJ_OP_PAGED_COPY = 3,         /* u0 = direction (0 into pages, 1 out of pages), u1 = start, u2 = page_tokens */
  FJ_OP_RMS_NORM = 4,           /* f0 = eps */
  FJ_OP_ARGMAX = 5,
  FJ_OP_TOP_K = 6,              /* u0 = k, u1 = normalize */
  FJ_OP_ROPE = 7,               /* f0 = theta */
  FJ_OP_EMBED = 8,
  FJ_OP_QUANT_EMBED = 9,        /* u0 = bits, u1 = group_size */
  FJ_OP_MATMUL = 10,
  FJ_OP_QUANT_MATMUL = 11,      /* u0 = bits, u1 = group_size */
  FJ_OP_GATHER_QUANT_MATMUL = 12, /* u0 = bits, u1 = group_size; 5-, 8- or 6-input form; program = epilogue or 0 */
  FJ_OP_PAGED_SDPA = 13,        /* f0 = scale, u0 = causal, u1 = q_start, u2 = key_length, u3 = page_tokens */
  FJ_OP_PAGED_SDPA_APPEND = 14, /* f0 = scale, u1 = q_start, u3 = page_tokens */
  FJ_OP_SDPA = 15,              /* contiguous cache: [q [hq, T, d], k [kvh, L, d], v [kvh, L, dv]] -> [hq, T, dv]; f0 = scale, u0 = causal, u1 = q_start */
  FJ_OP_GATHER_MATMUL = 17,     /* Op::GatherMatmul (dense experts): [x [rows, inner], weights [experts, inner, cols], idx u32 [rows, routes]]
                                   -> [rows, routes, cols]; an id >= experts leaves a zero row and reports the lowest such id */
  FJ_OP_SAMPLE = 16             /* Op::Sample / Op::SampleMasked (crates/forja-core/src/ops.rs:202-239): u0 = position; inputs [logits, params(5 x u32),
                                   (allow mask, (width + 31) / 32 x u32)]; invalid parameter words or mask fail the submission with FJ_INVALID_INPUT */
} fj_op;

/* ---- plain data ---------------------------------------------------------------------------- */

/* Tensor = BufferId + Layout, crates/forja-core/src/ops.rs:20-159, layout.rs:165-175 */
typedef struct fj_tensor {
  uint64_t buffer;     /* allocation id returned by fj_alloc / fj_import_readonly */
  uint32_t dtype;      /* fj_dtype */
  uint32_t rank;       /* <= 8 */
  uint64_t offset;     /* elements from the start of the allocation */
  uint32_t shape[8];
  uint64_t strides[8]; /* elements; 0 for broadcast axes */
} fj_tensor;

/* Dispatch, crates/forja-core/src/ops.rs:664-782: already validated by the caller (arity, dtype,
 * shape, aliasing); the library re-checks what it needs to stay memory-safe. Operand orders are
 * those of the reference: PagedCopy [ordinary-or-pool, table, generations, (activity)] -> out;
 * PagedSdpa [q, kpool, vpool, table, generations, (activity)] -> out; PagedSdpaAppend
 * [q, k_new, v_new, table, generations, (activity)] -> [out, kpool, vpool]; QuantMatmul
 * [x, packed, scales, biases]; GatherQuantMatmul [x, packed, scales, biases, idx] /
 * [x, p1, s1, b1, p2, s2, b2, idx] / [act, packed, scales, biases, idx, weights] (+ epilogue
 * extras); TopK [logits] -> [values, indices]. */
typedef struct fj_dispatch {
  uint32_t op; /* fj_op */
  uint32_t n_inputs;
  uint32_t n_outputs;
  uint32_t u0, u1, u2, u3;
  float f0;
  uint64_t program; /* Op::Program / epilogue handle, else 0 */
  const fj_tensor* inputs;
  const fj_tensor* outputs;
} fj_dispatch;

typedef struct fj_device_error {
  uint64_t submission; /* completion serial of the failing submission */
  uint32_t dispatch;   /* index within the submission */
  uint32_t op;         /* fj_op of that dispatch */
  uint32_t flag;       /* 1 = index out of range, 2 = page-table entry refused, 3 = internal wait gave up */
  uint32_t value;      /* lowest offending index / logical page */
  int64_t code;        /* cudaError_t for FJ_DEVICE_EXECUTION_FAILED */
} fj_device_error;

typedef struct fj_device_info_t {
  char name[128];
  uint32_t sm_count;
  uint32_t cc_major, cc_minor;
  uint64_t total_memory;
  uint64_t l2_bytes;
  uint32_t max_smem_per_block;
} fj_device_info_t;

typedef struct fj_dispatch_profile {
  uint32_t op;
  uint32_t kernels;   /* kernel launches issued for this dispatch */
  uint64_t ns;        /* device time, 0 when the submission was not profiled */
  /* KernelCost of the dispatch (crates/forja-core/src/cost.rs:109-153, cost/attention.rs:38-137): logical operand bytes read
   * and written and 2 flops per multiply-add, so achieved bytes/s or flop/s per dispatch = these / ns. Attention counts the
   * K/V rows attended plus 12 bytes per page of table and generation; other operators count their whole operands.
   * Filled for profiled submissions, else 0. */
  uint64_t read_bytes;
  uint64_t write_bytes;
  uint64_t flops;
} fj_dispatch_profile;

typedef struct fj_backend fj_backend;
typedef struct fj_submission fj_submission;

/* ---- backend: Backend trait, crates/forja-core/src/backend.rs:650-984 ------------------------ */

/* CudaBackend::new. memory_limit 0 = no quota. Fails with FJ_ALLOCATION_FAILED when no CUDA
 * device can be opened (there is no fallback). */
int32_t fj_backend_create(int32_t device, uint64_t memory_limit, fj_backend** out);
void fj_backend_destroy(fj_backend* be);
int32_t fj_device_info(fj_backend* be, fj_device_info_t* out);                     /* backend.rs:679 */
int32_t fj_set_memory_limit(fj_backend* be, uint64_t bytes);                      /* backend.rs:684 */
int32_t fj_memory_usage(fj_backend* be, uint64_t* used, uint64_t* limit);         /* backend.rs:669 */
/* alloc: zero-initialised device allocation (backend.rs:713). */
int32_t fj_alloc(fj_backend* be, uint64_t bytes, uint64_t* buffer);
/* import_readonly (backend.rs:719): copies `bytes` from host memory into a read-only buffer. */
int32_t fj_import_readonly(fj_backend* be, const void* host, uint64_t bytes, uint64_t* buffer);
int32_t fj_release(fj_backend* be, uint64_t buffer);                              /* backend.rs:777 */
/* write (backend.rs:756): contiguous bytes at a byte offset; refused on read-only buffers. */
int32_t fj_write(fj_backend* be, uint64_t buffer, uint64_t byte_offset, const void* src, uint64_t len);
/* read_buffer_range (backend.rs:728). */
int32_t fj_read(fj_backend* be, uint64_t buffer, uint64_t byte_offset, void* dst, uint64_t len);
/* read (backend.rs:762): gathers a strided view into contiguous logical bytes at dst. */
int32_t fj_read_strided(fj_backend* be, const fj_tensor* view, void* dst);
/* The byte range [lo, hi) of its allocation that a view can touch, with every product and sum
 * overflow-checked (the checked layout arithmetic of crates/forja-core/src/layout.rs:165-330);
 * FJ_INVALID_INPUT when rank or dtype is out of range or the arithmetic wraps 64 bits. Host logic,
 * needs no device: it is the test every tensor of a submission passes before a kernel sees it. */
int32_t fj_tensor_byte_span(const fj_tensor* view, uint64_t* lo, uint64_t* hi);
/* Device address of a buffer, for callers that stage data with their own copies or kernels. */
int32_t fj_buffer_device_ptr(fj_backend* be, uint64_t buffer, void** ptr, uint64_t* bytes);

/* prepare_program (backend.rs:693): structural recognition of the scalar programs the engines
 * submit (crates/forja-sdk/src/nn/blocks.rs:380-444, engines/qwen3-coder/src/lib.rs:26-54) with
 * their constants captured; anything else is FJ_UNSUPPORTED_OPERATION (no interpreter fallback).
 * kind: 0 Map, 1 Row. insts: n_insts x 4 words {tag, a, b, c} with tags 0 Input(slot),
 * 1 Const(f32 bits), 2 Index(axis), 3 Extent(axis), 4 Unary(op, x), 5 Binary(op, l, r),
 * 6 Select(c, t, f), 7 Cast(type, x), 8 Reduce(op, x); opcode numbering follows the declaration
 * order of UnOp/BinOp/RedOp/ValueType in crates/forja-core/src/program.rs:43-126.
 * outputs: n_outputs x {slot, inst}. */
int32_t fj_program_prepare(fj_backend* be, uint32_t kind, const uint32_t* insts, uint32_t n_insts,
                           const uint32_t* outputs, uint32_t n_outputs, uint64_t* handle);
/* The recognition step alone (host logic, needs no device): FJ_OK and *kernel / consts filled as
 * for fj_program_info, or FJ_UNSUPPORTED_OPERATION. */
int32_t fj_program_classify(uint32_t kind, const uint32_t* insts, uint32_t n_insts, const uint32_t* outputs,
                            uint32_t n_outputs, uint32_t* kernel, float consts[4]);
/* Which fused kernel a prepared program maps to: 1 add, 2 silu_mul, 3 rms_norm, 4 residual_norm,
 * 5 qk_norm_rope, 6 rope_pairs, 7 gated up (input 0 * silu(input 1), the matmul epilogue of
 * engines/smollm2/src/optimized.rs:249-252); consts receives the captured constants (eps, theta, head_dim).
 * As the epilogue of FJ_OP_MATMUL / FJ_OP_QUANT_MATMUL (fj_dispatch.program, one extra input of the output's shape after
 * the primitive inputs; crates/forja-cpu/src/lib.rs:443-493) the Map programs 1, 2 and 7 are taken: the program sees the
 * f32 accumulator as input 0 and the extra operand as input 1, and its result is rounded once to the output dtype. */
int32_t fj_program_info(fj_backend* be, uint64_t handle, uint32_t* kernel, float consts[4]);

/* submit (backend.rs:783) / submit_profiled (backend.rs:800). Work is enqueued and the call
 * returns; runs of per-lane paged-attention dispatches over the same planes are executed as one
 * ragged launch. */
int32_t fj_submit(fj_backend* be, const fj_dispatch* dispatches, uint32_t count, uint32_t profiled,
                  fj_submission** out);
/* Graph templates: prepare_graph / replay / replay_profiled (backend.rs:858-920; GraphTemplate,
 * crates/forja-core/src/graph.rs:1062-1617). A template is a validated command list in which scalar operation
 * parameters (TemplateOp: q_start, key_length, copy start, sample position) and tensor layouts (TemplateTensor::
 * Symbolic: element offset, extents) may be affine in up to 16 replay parameters: value = offset + scale *
 * values[param] (Affine, crates/forja-core/src/symbolic.rs:207-262, checked arithmetic). fj_graph_prepare copies
 * the dispatches; fj_graph_replay instantiates them with this call's values and submits them - the reference's
 * own default tier - so a replay answers exactly like the equivalent fj_submit (fj_dense_graph_replay below is
 * the device-side tier for whole decode steps). Field codes: */
enum {
  FJ_GRAPH_FIELD_U0 = 0, FJ_GRAPH_FIELD_U1 = 1, FJ_GRAPH_FIELD_U2 = 2, FJ_GRAPH_FIELD_U3 = 3, /* fj_dispatch.u0 .. u3 */
  FJ_GRAPH_FIELD_INPUT_OFFSET = 0x100,  /* | operand << 4 : element offset of input `operand` */
  FJ_GRAPH_FIELD_OUTPUT_OFFSET = 0x200, /* | operand << 4 */
  FJ_GRAPH_FIELD_INPUT_EXTENT = 0x300,  /* | operand << 4 | axis : shape[axis] of input `operand` */
  FJ_GRAPH_FIELD_OUTPUT_EXTENT = 0x400  /* | operand << 4 | axis */
};
typedef struct fj_graph_binding {
  uint32_t dispatch; /* index into the template's dispatches */
  uint32_t field;    /* one of the codes above */
  uint32_t param;    /* index into the replay values */
  uint32_t scale;
  uint64_t offset;
} fj_graph_binding;
typedef struct fj_graph fj_graph;
int32_t fj_graph_prepare(fj_backend* be, const fj_dispatch* dispatches, uint32_t count, const fj_graph_binding* bindings,
                         uint32_t n_bindings, uint32_t n_params, fj_graph** out);
int32_t fj_graph_replay(fj_graph* graph, const uint32_t* values, uint32_t n_values, uint32_t profiled, fj_submission** out);
void fj_graph_destroy(fj_graph* graph);
/* Submission, backend.rs:609-647 */
int32_t fj_sub_wait(fj_submission* sub, uint64_t timeout_ns); /* 0 = wait forever; FJ_TIMEOUT leaves the submission alive */
int32_t fj_sub_gpu_time_ns(fj_submission* sub, uint64_t* ns);
uint64_t fj_sub_completion_serial(fj_submission* sub);
int32_t fj_sub_error(fj_submission* sub, fj_device_error* out);
uint32_t fj_sub_kernel_launches(fj_submission* sub);
int32_t fj_sub_profile(fj_submission* sub, fj_dispatch_profile* out, uint32_t cap, uint32_t* count);
void fj_sub_destroy(fj_submission* sub);

/* Device-wide synchronisation of the backend's stream (tests and benchmarks). */
int32_t fj_synchronize(fj_backend* be);
/* Number of kernels this backend has launched since creation. */
uint64_t fj_kernel_launch_count(fj_backend* be);

/* Timers on the backend's stream (CUDA events): benchmarks time the stream the kernels run on. */
int32_t fj_timer_create(fj_backend* be, uint64_t* timer);
int32_t fj_timer_record(fj_backend* be, uint64_t timer);
int32_t fj_timer_elapsed_ns(fj_backend* be, uint64_t start_timer, uint64_t stop_timer, uint64_t* ns);

/* ---- weight sources: safetensors import, crates/forja-host/src/weights.rs ------------------- */

/* WeightTensor, weights.rs:27-84. `name` points into the source and lives as long as it. */
typedef struct fj_weight_tensor {
  const char* name;
  uint32_t dtype;        /* fj_dtype: F32, F16, BF16 or U32 (anything else is FJ_WEIGHTS_UNSUPPORTED_DTYPE at open) */
  uint32_t rank;
  uint32_t shape[8];
  uint64_t byte_offset;  /* from the start of the data region */
  uint64_t byte_len;
  uint32_t dtype_aligned; /* is_dtype_aligned, weights.rs:72 */
} fj_weight_tensor;
typedef struct fj_safetensors fj_safetensors;

/* Safetensors::open (weights.rs:175-226): validates one file - regular file, 8-byte length prefix, header of at
 * most 100 MiB, JSON object without duplicate names (nesting deeper than 128 is refused), supported dtypes, byte
 * ranges equal to shape x element size, inside the file and non-overlapping. Tensors are kept sorted by offset.
 * Host-only: needs no device. On failure fj_weights_last_error() holds the message for the calling thread. */
int32_t fj_safetensors_open(const char* path, fj_safetensors** out);
/* Safetensors::open_all (weights.rs:114-168): `path` ending in .json is a shard index {"weight_map": {tensor: file}}
 * (at most 100 MiB, at most 1024 shards, shard names without separators ending in .safetensors, resolving inside the
 * index's directory, each shard holding exactly the tensors the map assigns to it); shards come back ordered by
 * file name. Any other path opens as a single file. *count receives the number of sources; FJ_QUOTA_EXCEEDED when
 * `cap` is too small (nothing is returned then). */
int32_t fj_safetensors_open_all(const char* path, fj_safetensors** out, uint32_t cap, uint32_t* count);
void fj_safetensors_close(fj_safetensors* source);
uint32_t fj_safetensors_tensor_count(const fj_safetensors* source);
const char* fj_safetensors_shard_name(const fj_safetensors* source); /* NULL for an unsharded file (weights.rs:235) */
uint64_t fj_safetensors_file_len(const fj_safetensors* source);      /* weights.rs:241 */
uint64_t fj_safetensors_data_start(const fj_safetensors* source);
int32_t fj_safetensors_tensor(const fj_safetensors* source, uint32_t index, fj_weight_tensor* out);
int32_t fj_safetensors_find(const fj_safetensors* source, const char* name, fj_weight_tensor* out);
const char* fj_weights_last_error(void);
/* mapped_region + import_readonly (weights.rs:326-333, crates/forja-host/src/lib.rs:5885-5900): maps the file,
 * refuses it when its length changed since validation, and copies the data region into one read-only buffer. */
int32_t fj_safetensors_import(fj_backend* be, const fj_safetensors* source, uint64_t* buffer);
/* WeightTensor::layout (weights.rs:76-83): the named tensor as a contiguous view of the imported buffer. */
int32_t fj_safetensors_view(const fj_safetensors* source, const char* name, uint64_t buffer, fj_tensor* out);
/* An MLX affine-quantised matrix (or stack of expert matrices) by checkpoint prefix: `<prefix>.weight` u32
 * [.., out, in * bits / 32], `<prefix>.scales` and `<prefix>.biases` f16/bf16 [.., out, in / group_size]
 * (engines/qwen3-coder/src/lib.rs:174-188, 430-437); shapes and dtypes are cross-checked like
 * QuantizedMatrix::new (crates/forja-core/src/quantized.rs:78-121). */
int32_t fj_safetensors_quant_views(const fj_safetensors* source, const char* prefix, uint64_t buffer, uint32_t bits,
                                   uint32_t group_size, fj_tensor* packed, fj_tensor* scales, fj_tensor* biases);

/* ---- fast path: device-resident ragged batching -------------------------------------------- */

/* Paged-KV allocator on the device (replaces the host mutex of PagePool::reserve/release,
 * crates/forja-core/src/paged_pool.rs:204-232, 308-327, 1229-1326, for fixed-capacity pools).
 * One pool owns: free stack (LIFO, page 0 on top), generations[physical_pages], and
 * `lanes` page tables of `table_pages` entries {page, generation}, poisoned when unbound. */
typedef struct fj_kvpool fj_kvpool;
int32_t fj_kvpool_create(fj_backend* be, uint32_t page_tokens, uint32_t physical_pages, uint32_t lanes,
                         uint32_t table_pages, fj_kvpool** out);
void fj_kvpool_destroy(fj_kvpool* pool);
/* reserve: lane <- ceil(tokens/page_tokens) pages popped from the stack, generation bumped
 * (never 0xFFFFFFFF); refusal (not enough pages, lane bound, table too small) changes nothing and
 * is reported in status[i] (FJ_OK / FJ_QUOTA_EXCEEDED / FJ_INVALID_INPUT) after the call.
 * Requests are applied in order by one CTA so page ids equal the host allocator's. */
int32_t fj_kvpool_reserve(fj_kvpool* pool, const uint32_t* lanes, const uint32_t* tokens, uint32_t count,
                          int32_t* status);
/* release: pages of the lane return to the stack in table order; table re-poisoned. */
int32_t fj_kvpool_release(fj_kvpool* pool, const uint32_t* lanes, uint32_t count);
/* Snapshots for parity checks: table [table_pages x 2] of one lane, generations, free stack. */
int32_t fj_kvpool_read_table(fj_kvpool* pool, uint32_t lane, uint32_t* entries);
int32_t fj_kvpool_read_generations(fj_kvpool* pool, uint32_t* generations);
int32_t fj_kvpool_read_free(fj_kvpool* pool, uint32_t* pages, uint32_t cap, uint32_t* count);
int32_t fj_kvpool_read_refcounts(fj_kvpool* pool, uint32_t* refcounts); /* [physical_pages]: owners of each page, 0 = free */
/* Prefix sharing (PagedSequence::fork_reserved / cow_tail, crates/forja-core/src/paged_pool.rs:949-1054).
 * fork: the unbound lane dst shares the first ceil(prefix_tokens / page_tokens) pages of src (reference counts + 1, the
 * pages become immutable for both) and gets private pages up to reserved_tokens; src_logical_len = tokens src has
 * committed. Returns FJ_OK, FJ_QUOTA_EXCEEDED (not enough free pages; nothing changed) or FJ_INVALID_INPUT.
 * cow_tail: before a lane writes at logical_len, a shared page holding token logical_len - 1 is replaced in its table by
 * a fresh private page; out4 = {copied (0/1), source page, destination page, rows to copy}; the caller copies the rows
 * (fj_dense_copy_page). Both calls are synchronous control-path calls. */
int32_t fj_kvpool_fork(fj_kvpool* pool, uint32_t src_lane, uint64_t src_logical_len, uint32_t dst_lane, uint64_t prefix_tokens, uint64_t reserved_tokens);
int32_t fj_kvpool_cow_tail(fj_kvpool* pool, uint32_t lane, uint64_t logical_len, uint32_t* out4);
/* Sequence boundaries on the device pool (PagedSequence::rewind_private / checkpoint / rollback and SequenceCheckpoint,
 * crates/forja-core/src/paged_pool.rs:864-883, 1061-1175). The logical length of a lane lives with the caller, as
 * everywhere in this interface.
 * rewind_private: may the lane go back from current_len to new_len? FJ_POOL_INVALID_CHECKPOINT unless new_len < current_len;
 *   FJ_POOL_SHARED_TAIL when a page between the two boundaries is immutable for the lane or referenced by another owner.
 * checkpoint: records the lane's length and tail page; a tail that is shared is retained (reference count + 1) so that a
 *   later copy-on-write cannot free it.
 * rollback: consumes a checkpoint of this lane: the recorded tail page goes back into the table (a private copy made since
 *   is released), the immutable mark is restored and *logical_len receives the recorded length. A checkpoint of another
 *   pool or lane, or one whose lane was released since, is refused with FJ_POOL_INVALID_CHECKPOINT and dropped.
 * checkpoint_drop: gives up a checkpoint that was not rolled back (releases the retained tail). */
typedef struct fj_kv_checkpoint {
  uint64_t pool, lane_epoch, logical_len;
  uint32_t lane, active, has_tail, index, page, immutable, retained, reserved;
} fj_kv_checkpoint;
int32_t fj_kvpool_rewind_private(fj_kvpool* pool, uint32_t lane, uint64_t current_len, uint64_t new_len);
int32_t fj_kvpool_checkpoint(fj_kvpool* pool, uint32_t lane, uint64_t logical_len, fj_kv_checkpoint* out);
int32_t fj_kvpool_rollback(fj_kvpool* pool, uint32_t lane, fj_kv_checkpoint* checkpoint, uint64_t* logical_len);
int32_t fj_kvpool_checkpoint_drop(fj_kvpool* pool, fj_kv_checkpoint* checkpoint);
uint64_t fj_kvpool_tables_buffer(fj_kvpool* pool);      /* buffer id: [lanes, table_pages, 2] u32 */
uint64_t fj_kvpool_generations_buffer(fj_kvpool* pool); /* buffer id: [physical_pages] u32 */

/* Ragged-batch packer on the device: lane descriptors -> the metadata of
 * write_paged_lane_metadata (crates/forja-host/src/lib.rs:4977-5065) plus cu_seqlens, positions,
 * slot_mapping and row_lane. starts/tokens are host arrays [lanes] (tokens 0 = inactive lane);
 * logical lengths are taken as start (the lane's committed length when the step begins).
 * All outputs are u32 device buffers owned by the pool; read them back with fj_kvpool_read_pack. */
typedef struct fj_pack_view {
  uint32_t rows;
  uint32_t lanes;
  uint64_t logical_lengths, query_starts, absolute_positions, activity; /* buffer ids, [lanes] */
  uint64_t cu_seqlens;                                                  /* [lanes + 1] */
  uint64_t positions, slot_mapping, row_lane;                           /* [rows] */
} fj_pack_view;
int32_t fj_pack_step(fj_kvpool* pool, const uint32_t* starts, const uint32_t* tokens, uint32_t lanes,
                     fj_pack_view* out);

/* Continuous-batching policy on the host; replaces SchedulerPolicy
 * (crates/forja-serve/src/scheduler.rs:16-196). Integer bookkeeping, bit-exact with the reference:
 *   create            SchedulerPolicy::new :30-66 (buckets sorted + deduplicated, must start at 1 and
 *                     reach active_limit; limits and budgets positive, else FJ_INVALID_INPUT)
 *   set_prompt_chunk_multiple  with_prompt_chunk_multiple :67-76 (switches to merged chunking)
 *   enqueue / reconcile_active / complete / retry_admission   :78-107
 *   admit             :109-152: FIFO; a head that cannot be reserved may be overtaken at most 8 times
 *                     by the first strictly smaller request that can; `reserve` returns nonzero when
 *                     it has reserved room for (id, reserved_tokens). Returns how many were admitted
 *                     and writes up to cap ids in admission order.
 *   admit_pages       admit with the page arithmetic of the continuous engine: a request needs
 *                     ceil(reserved_tokens / page_tokens) pages out of *free_pages (decremented).
 *   decode_bucket     :89-95: smallest bucket >= max(slot) + 1 (saturating), -1 when none / empty
 *   ready_prompt / prompt_batch  :154-195: round-robin over ascending ids starting after the id
 *                     served last, at most prefill_limit entries, spending prompt_budget (decoding)
 *                     or idle_prompt_budget through PromptChunking::work / merged_work
 *                     (crates/forja-host/src/prompt.rs:20-41). */
typedef struct fj_sched fj_sched;
typedef int32_t (*fj_sched_reserve_fn)(void* user, uint64_t id, uint64_t reserved_tokens);
int32_t fj_sched_create(const uint32_t* buckets, uint32_t bucket_count, uint64_t active_limit, uint64_t prefill_limit,
                        uint32_t prompt_budget, uint32_t idle_prompt_budget, fj_sched** out);
void fj_sched_destroy(fj_sched* sched);
void fj_sched_set_prompt_chunk_multiple(fj_sched* sched, uint32_t multiple);
void fj_sched_enqueue(fj_sched* sched, uint64_t id, uint64_t reserved_tokens);
void fj_sched_reconcile_active(fj_sched* sched, uint64_t active);
void fj_sched_complete(fj_sched* sched, uint64_t id);
void fj_sched_retry_admission(fj_sched* sched, uint64_t id, uint64_t reserved_tokens);
uint64_t fj_sched_admit(fj_sched* sched, fj_sched_reserve_fn reserve, void* user, uint64_t* ids, uint64_t cap);
uint64_t fj_sched_admit_pages(fj_sched* sched, uint32_t page_tokens, uint64_t* free_pages, uint64_t* ids, uint64_t cap);
int64_t fj_sched_decode_bucket(const fj_sched* sched, const uint32_t* slots, uint64_t count);
void fj_sched_ready_prompt(fj_sched* sched, uint64_t id, uint32_t tokens);
uint64_t fj_sched_prompt_batch(fj_sched* sched, int32_t decoding, uint64_t* ids, uint32_t* spend, uint64_t cap);
uint64_t fj_sched_waiting(const fj_sched* sched);
uint64_t fj_sched_active(const fj_sched* sched);
/* PromptChunking::work / merged_work (crates/forja-host/src/prompt.rs:20-41). */
uint32_t fj_prompt_chunk_work(uint32_t piece, uint32_t remaining, uint32_t allowance);
uint32_t fj_prompt_chunk_merged_work(uint32_t piece, uint32_t remaining, uint32_t allowance);
/* reservations_fit (crates/forja-serve/src/engine/continuous/batch.rs:1139-1152): 1 when the pages of
 * all reservations fit ceil(max_context / page_tokens), 0 otherwise or on overflow. */
int32_t fj_reservations_fit(uint32_t page_tokens, uint32_t max_context, const uint64_t* reservations, uint64_t count);
/* Chunk lengths of a chunked prefill (crates/forja-sdk/src/nn/blocks.rs:892-911): full chunks, then
 * tail_chunk-sized pieces; returns the number of pieces (0 = no valid plan). */
uint64_t fj_prefill_plan(uint32_t sequence, uint32_t chunk, uint32_t tail_chunk, uint32_t* out, uint64_t cap);

/* Dense decoder (SmolLM2 / Qwen3-dense shapes; reference op order: engines/qwen3/src/lib.rs:391-452,
 * 734-811 and engines/smollm2/src/optimized.rs:97-245). Weights are buffers of this backend in the
 * activation dtype: embed [vocab, hidden] (tied lm_head), per layer wq [hq*d, hidden],
 * wk/wv [kvh*d, hidden], wo [hidden, hq*d], w_gate/w_up [inter, hidden], w_down [hidden, inter],
 * norms [hidden], optional q_norm/k_norm [d]. */
typedef struct fj_dense_config {
  uint32_t dtype;        /* FJ_F32 or FJ_BF16: activations, weights and KV planes */
  uint32_t layers, hidden, q_heads, kv_heads, head_dim, intermediate, vocab;
  uint32_t qk_norm;      /* 1: per-head RMSNorm on q and k before RoPE (guest program), 0: plain Op::Rope */
  float eps, theta;
  uint32_t max_rows;     /* largest number of token rows in one step */
} fj_dense_config;
typedef struct fj_dense_layer_weights {
  uint64_t input_norm, wq, wk, wv, q_norm, k_norm, wo, post_norm, w_gate, w_up, w_down;
} fj_dense_layer_weights;
typedef struct fj_dense_model fj_dense_model;
int32_t fj_dense_model_create(fj_backend* be, const fj_dense_config* config, uint64_t embed, uint64_t final_norm,
                              const fj_dense_layer_weights* layers, fj_kvpool* pool, fj_dense_model** out);
void fj_dense_model_destroy(fj_dense_model* model);
/* One continuous-batching forward step over the lanes packed by the last fj_pack_step:
 * embed -> layers (qkv, qk-norm+rope+KV append, paged attention, o, residual+norm, MLP) -> final
 * norm -> lm_head on each lane's last row -> greedy argmax. token_ids: host u32 [rows] or NULL to
 * feed back each lane's previous greedy token (device-resident). out_tokens: host u32 [lanes] or
 * NULL. logits_out: buffer id receiving [lanes, vocab] in the activation dtype, or 0. The call
 * returns after the step completed when out_tokens != NULL, else it only enqueues. */
int32_t fj_dense_step(fj_dense_model* model, const uint32_t* token_ids, uint32_t* out_tokens, uint64_t logits_out);
/* Launch count of the last step and the number of split-K work items of its attention launches. */
/* Copies the first `tokens` K/V rows of page src_page to page dst_page in every layer (the data half of cow_tail). */
int32_t fj_dense_copy_page(fj_dense_model* model, uint32_t src_page, uint32_t dst_page, uint32_t tokens);
int32_t fj_dense_step_stats(fj_dense_model* model, uint64_t* kernels, uint64_t* attn_work_items);
/* Graph replay of the decode step: the backend-specific tier behind Backend::prepare_graph / replay
 * (crates/forja-core/src/backend.rs:858-967; the reference's default tier re-instantiates and re-submits the
 * template). With replay enabled, a decode-only step (every active lane appends one token) is recorded once per
 * bucket {lanes, split-K chunk, attention grid rounded up to 1024 work items, token source, logits target} as a
 * CUDA graph and replayed afterwards: one graph launch on the host instead of one launch per kernel. Every
 * row-wise kernel of a replayed step runs `lanes` rows (rows past the packed count are padding whose appends are
 * refused), the attention kernel reads the live work-item count on the device. Steps that mix prompt pieces, or
 * run while attention profiling is on, take the direct path. Results are identical on both paths.
 * fj_dense_graph_stats: recordings made, steps replayed, recordings that failed (after 3 the model stays direct). */
int32_t fj_dense_graph_replay(fj_dense_model* model, uint32_t enabled);
int32_t fj_dense_graph_stats(fj_dense_model* model, uint64_t* recordings, uint64_t* replays, uint64_t* failures);
/* Host access to the model's KV planes (which the library owns, like the host-owned page planes of
 * crates/forja-host/src/lib.rs:4323-4360): copies the rows of `count` consecutive physical pages of
 * one layer's K plane (plane 0) or V plane (plane 1) to host memory (to_device 0) or from it
 * (to_device 1); page_tokens * kv_heads * head_dim elements of the model dtype per page.
 * Synchronous; for checkpointing a sequence's cache and for checkers that replay a lane elsewhere. */
int32_t fj_dense_kv_pages(fj_dense_model* model, uint32_t layer, uint32_t plane, uint32_t first_page, uint32_t count,
                          void* host, uint32_t to_device);
/* Fills every K/V plane of the model with seeded pseudo-random N(0, 1) values in the plane dtype
 * (synthetic contexts for benchmarks: any page a lane is given already holds finite random rows). */
int32_t fj_dense_fill_kv(fj_dense_model* model, uint64_t seed);
/* Attention timing: when enabled, every paged-attention launch of fj_dense_step is bracketed by
 * CUDA events on the backend's stream. fj_dense_attention_time drains the recorded pairs
 * (synchronising on them), adds their durations and launch count to the totals and returns them. */
int32_t fj_dense_profile_attention(fj_dense_model* model, uint32_t enabled);
int32_t fj_dense_attention_time(fj_dense_model* model, uint64_t* total_ns, uint64_t* launches);

/* ---- decode attention without any allocation ----------------------------------------------- */

/* This entry point has no counterpart in the reference. It exists for hosts that cannot let the
 * library allocate at step time: a server that has already given all device memory to the KV
 * planes and holds the backend to a fixed quota, or a decode loop that must never enter the
 * driver's allocator (cudaMalloc / cudaFree may stall the whole device). It runs the same
 * split-K paged GQA decode attention as FJ_OP_PAGED_SDPA for one token per lane, but every piece
 * of scratch it needs (lane descriptors, work list, split partials, counters) lives in a fixed
 * array inside the library image, about 8.6 MB that each GPU loading the library holds until the
 * process exits. It calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Limits (beyond them the call is refused with FJ_QUOTA_EXCEEDED and nothing runs):
 * lanes <= FJ_STATIC_ATTENTION_MAX_LANES, lanes * kv_heads <= FJ_STATIC_ATTENTION_MAX_GROUPS; the
 * key range is cut into at most FJ_STATIC_ATTENTION_MAX_ITEMS chunks (chunks grow with the batch).
 *
 * All pointers are device addresses of the backend's GPU except key_lengths (host array [lanes],
 * tokens attended per lane, i.e. position + 1): q, out [lanes, q_heads, 128] and kpool, vpool
 * [physical_pages, 16, kv_heads, 128] in `dtype` (FJ_BF16 or FJ_F16); tables
 * [lanes, table_pages, 2] {page, generation}; generations [physical_pages]; status: two u32 words
 * that receive {flag, lowest offending logical page} with the meaning of the fj_device_error
 * fields: flag 2 = page entry refused, and that lane's output is zero. May be NULL. The work is enqueued on the backend's stream.
 *
 * The first call on a device also looks up the array's device address and raises the kernel's
 * shared-memory limit; make that first call before starting any stream capture. All calls share
 * the one array, which still holds the previous call's contents (the counters are cleared on
 * every call): two calls whose GPU work overlaps - other streams, other threads, other backends
 * on the same device - race on it. Calls on one backend are ordered by its stream and are safe. */
#define FJ_STATIC_ATTENTION_MAX_LANES 64
#define FJ_STATIC_ATTENTION_MAX_GROUPS 512
#define FJ_STATIC_ATTENTION_MAX_ITEMS 1024
int32_t fj_paged_decode_attention_static(fj_backend* be, const void* q, void* out, const void* kpool, const void* vpool,
                                         const uint32_t* tables, const uint32_t* generations, const uint32_t* key_lengths,
                                         uint32_t lanes, uint32_t table_pages, uint32_t physical_pages, uint32_t q_heads,
                                         uint32_t kv_heads, uint32_t dtype, float scale, uint32_t* status);

/* Health counter of the tcgen05 kernels (dense GEMM, grouped expert GEMM, prefill attention; no counterpart in the
 * reference): how many of their bounded mbarrier waits ran out since the library was loaded. 0 in a healthy run; a
 * nonzero value means a kernel gave up, freed its tensor memory and left its output tile unwritten (the attention kernel
 * writes zeros for its rows). Synchronises the stream. */
int32_t fj_tcgen05_wait_giveups(fj_backend* be, uint32_t* out);

/* Synthetic contents for benchmarks (no counterpart in the reference, whose weights come from
 * checkpoints): fills `elements` values of a buffer starting at offset_bytes with a counter-based
 * generator: normal(mean, std) for float dtypes, uniform 32-bit words for FJ_U32 / FJ_I32. */
int32_t fj_fill_random(fj_backend* be, uint64_t buffer, uint64_t offset_bytes, uint64_t elements, uint32_t dtype, uint64_t seed,
                       float mean, float std);

/* Expert parallelism over the GPUs of one node. The reference is single-GPU, so these entry points
 * have no counterpart there; they carry the all-to-all of the sparse-MoE step below. NCCL is opened
 * at run time (path of libnccl.so.2, or NULL for the loader's search path); one rank creates the
 * 128-byte id, every rank of the group passes the same id to the create call. */
typedef struct fj_ep fj_ep;
int32_t fj_ep_load(const char* libnccl_path);
int32_t fj_ep_unique_id(uint8_t* out128);
int32_t fj_ep_create(fj_backend* be, const uint8_t* id128, uint32_t rank, uint32_t world, fj_ep** out);
void fj_ep_destroy(fj_ep* ep);
/* Every rank sends bytes_per_peer bytes of `send` to each rank and receives as many from each into
 * `recv` (buffer ids; world * bytes_per_peer bytes each), ordered on the backend's stream. */
int32_t fj_ep_all_to_all(fj_ep* ep, uint64_t send, uint64_t recv, uint64_t bytes_per_peer);
/* Every host wait on an exchange of this group (the per-layer row counts of large steps, the tokens of a step) polls with a
 * deadline, 60 s unless set here (0 = none). When it runs out - a peer never posted its half - the communicator is aborted
 * (ncclCommAbort), the call and every later exchange of the group answer FJ_TIMEOUT, and the backend stays usable. */
int32_t fj_ep_set_timeout(fj_ep* ep, uint64_t timeout_ms);
/* Host-only check of that bounded wait against a simulated clock (needs no device): a condition that turns true at its
 * ready_after_polls-th poll (0 = never) is waited for with a clock that advances tick_ms per reading; returns 1 when the
 * condition was seen, 0 when the wait gave up at timeout_ms; *polls = how often the condition was asked. */
int32_t fj_ep_poll_selftest(uint64_t timeout_ms, uint64_t ready_after_polls, uint64_t tick_ms, uint64_t* polls);

/* Sparse-MoE decoder (Qwen3-Coder-30B-A3B shape family; reference op order:
 * engines/qwen3-coder/src/lib.rs:886-947 forward_batch, :505-603 SparseMoe::route / forward_decode,
 * crates/forja-sdk/src/nn.rs:29-45 moe_router_with). All projections are MLX affine-quantised
 * (packed u32 [N, K * bits / 32], scales and biases bf16 [N, K / group]): q4 everywhere except the
 * router (router_bits, 8 in the reference). Expert tensors are stacked [experts_local, N, ...].
 * Activations and KV are bf16; router logits, routing weights and per-route down projections f32.
 * With an fj_ep the experts are sharded: this rank holds experts
 * [rank * experts / world, (rank + 1) * experts / world) and runs its own lanes. */
typedef struct fj_quant_weight {
  uint64_t packed, scales, biases; /* buffer ids */
} fj_quant_weight;
typedef struct fj_moe_config {
  uint32_t layers, hidden, q_heads, kv_heads, head_dim, experts, top_k, expert_intermediate, vocab;
  uint32_t group_size, router_bits;
  float eps, theta;
  uint32_t max_rows; /* largest number of token rows in one step */
  /* Expert projections switch from one pass per route to expert-bucketed forms at this many routes
   * (0 = 64); a value above max_rows * top_k keeps the per-route path. Bucketed routes run as 16-row
   * tiles that stream each active expert once (int8 tensor cores) while routes < stream_rows_per_expert
   * * experts (0 = 72), and as tile GEMMs (128 rows on tcgen05, weights rounded to bf16) from there on. */
  uint32_t grouped_min_routes;
  uint32_t stream_rows_per_expert;
  /* Expert parallelism only: nonzero = the experts' owners return their per-route rows rounded to bf16 instead of f32.
   * Halves the larger of the two exchanges; the logits then agree with one GPU within the bf16 tolerance instead of bit for bit. */
  uint32_t ep_return_bf16;
  /* Expert parallelism with the direct exchange only: every layer's rows are split into this many chunks (0 or 1 = no
   * split, at most 8) that go through dispatch, experts and return one behind the other on streams of their own, so that one
   * chunk's transfer over NVLink runs while another chunk's experts compute. All ranks must use the same value. */
  uint32_t ep_chunks;
} fj_moe_config;
typedef struct fj_moe_layer_weights {
  uint64_t input_norm, q_norm, k_norm, post_norm; /* bf16 [hidden], [head_dim], [head_dim], [hidden] */
  fj_quant_weight qkv;                            /* [(q_heads + 2 kv_heads) * head_dim, hidden] */
  fj_quant_weight o;                              /* [hidden, q_heads * head_dim] */
  fj_quant_weight router;                         /* [experts, hidden], router_bits */
  fj_quant_weight gate, up;                       /* [experts_local, expert_intermediate, hidden] */
  fj_quant_weight down;                           /* [experts_local, hidden, expert_intermediate] */
} fj_moe_layer_weights;
typedef struct fj_moe_model fj_moe_model;
int32_t fj_moe_model_create(fj_backend* be, const fj_moe_config* config, const fj_quant_weight* embed, uint64_t final_norm,
                            const fj_quant_weight* lm_head, const fj_moe_layer_weights* layers, fj_kvpool* pool, fj_ep* ep,
                            fj_moe_model** out);
void fj_moe_model_destroy(fj_moe_model* model);
/* One forward step over the lanes packed by the last fj_pack_step; arguments as fj_dense_step
 * (logits_out, when nonzero, receives [lanes, vocab] bf16). Under expert parallelism every rank of
 * the group must call it for the same step, even with no active lane of its own (pack zero tokens). */
int32_t fj_moe_step(fj_moe_model* model, const uint32_t* token_ids, uint32_t* out_tokens, uint64_t logits_out);
int32_t fj_moe_step_stats(fj_moe_model* model, uint64_t* kernels, uint64_t* attn_work_items);
/* Direct exchange between the ranks of one node (no counterpart in the single-GPU reference): instead of NCCL sends and
 * receives with a host round trip for the row counts, every rank maps four of the others' buffers (CUDA IPC). A layer's
 * dispatch is plain peer stores over NVLink by the kernel that assigns the slots, followed by one flag per (source,
 * destination) carrying the row count, which the receiver polls in its own memory with a bound. On the way back either the
 * owner only publishes "results ready" and the origin's combine reads the per-route rows from the owner's memory (fewer
 * passes over local memory; used up to 3 ranks), or the owner writes them into the origin's memory (writes load NVLink
 * better than reads when every rank talks to every other; used from 4 ranks on); fj_moe_ep_return_mode overrides the choice.
 * No multicast is used. Results are bit-identical to the NCCL exchange and to one GPU (same slots, same arithmetic).
 *   fj_moe_ep_export     writes this rank's 5 x 64-byte buffer handles to out320.
 *   fj_moe_ep_connect    takes every rank's 320 bytes in rank order ([world][320]; gathered by the caller over any host
 *                        channel) and maps the peers' buffers; FJ_UNSUPPORTED_OPERATION when a mapping is refused.
 *   fj_moe_ep_direct     switches the model's steps to this exchange (1) or back to NCCL (0). All ranks must choose alike:
 *                        enable only after every rank reported a successful connect.
 *   fj_moe_ep_disconnect unmaps the peers' buffers. Every rank calls it and then meets the others at a host barrier before
 *                        any of them destroys its model: a mapping has to be closed before its owner frees the memory.
 *   fj_moe_ep_wait_polls bound of the device-side waits in polls (default 2^24, about ten seconds). A wait that runs out
 *                        makes the step compute on zero rows, fj_moe_step answer FJ_TIMEOUT from then on, and leaves the
 *                        context usable; the model has to be rebuilt.
 *   fj_ep_wait_selftest  runs that wait on a flag nothing sets and returns FJ_TIMEOUT when the kernel gave up and said so. */
int32_t fj_moe_ep_export(fj_moe_model* model, uint8_t* out320);
int32_t fj_moe_ep_connect(fj_moe_model* model, const uint8_t* table);
int32_t fj_moe_ep_direct(fj_moe_model* model, uint32_t enabled);
int32_t fj_moe_ep_disconnect(fj_moe_model* model);
int32_t fj_moe_ep_wait_polls(fj_moe_model* model, uint32_t polls);
int32_t fj_moe_ep_return_mode(fj_moe_model* model, uint32_t mode); /* 0 or 1 = the origin reads, 2 = the owner writes; same on all ranks */
/* Rows this rank received for its experts in the last finished step of the direct exchange, per (layer, chunk):
 * out[layers * max(ep_chunks, 1)]. Shows how evenly the router spreads work over the ranks. */
int32_t fj_moe_ep_received(fj_moe_model* model, uint32_t* out, uint32_t words);
int32_t fj_ep_wait_selftest(fj_backend* be, uint32_t polls);
/* Measurement aid: while enabled, every layer of a step records CUDA events around its four phases; fj_moe_read_phase_ms
 * waits for the step and returns the time summed over the layers: [0] attention block and router, [1] dispatch (slot plan,
 * row scatter, exchange to the experts' owners; ~0 on one GPU), [2] expert projections, [3] exchange back and weighted combine. */
int32_t fj_moe_phase_timing(fj_moe_model* model, uint32_t enabled);
int32_t fj_moe_read_phase_ms(fj_moe_model* model, float* out4);
/* Measurement aid: while enabled, the router still runs but its choice is replaced by an even spread (every row takes top_k
 * distinct experts from a hash of layer and row, weight 1 / top_k). A model with random weights routes most rows of a prompt to
 * the same few experts, which a trained, load-balanced router does not; this switch shows what the step costs without that. */
int32_t fj_moe_uniform_routing(fj_moe_model* model, uint32_t enabled);
/* Parity aid: while enabled, every layer's routing of a step (TopK output: expert ids and normalised
 * weights, [rows, top_k] in packed row order) is kept and can be read back after the step. */
int32_t fj_moe_capture_routes(fj_moe_model* model, uint32_t enabled);
int32_t fj_moe_read_routes(fj_moe_model* model, uint32_t layer, uint32_t rows, uint32_t* experts, float* weights);

#ifdef __cplusplus
}
#endif
#endif /* FORJA_CUDA_H */
