// Internal state of the CUDA backend shared by the C ABI translation units.
#pragma once

#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/forja_cuda.h"
#include "fj_kernels.h"

struct fj_buffer_rec {
  void* ptr = nullptr;
  uint64_t bytes = 0;
  bool readonly = false;
};

// A recognised scalar program: which fused kernel runs it and the constants captured from the IR.
struct fj_program_rec {
  uint32_t kernel = 0;  // 1 add, 2 silu_mul, 3 rms_norm, 4 residual_norm, 5 qk_norm_rope, 6 rope_pairs
  float eps = 0.0f, theta = 0.0f, head_dim = 0.0f, exponent_scale = 0.0f;
};

struct fj_backend {
  int device = 0;
  cudaStream_t stream = nullptr;
  fj::Ctx ctx{};
  std::mutex mutex;
  std::unordered_map<uint64_t, fj_buffer_rec> buffers;
  uint64_t next_buffer = 1;
  uint64_t used_bytes = 0, limit_bytes = 0;
  std::vector<fj_program_rec> programs;  // handle = index + 1
  uint64_t next_serial = 1;
  cudaDeviceProp prop{};
  std::vector<cudaEvent_t> timers;
  // device tables of rotary frequencies, keyed by (theta bits, scale bits, count, reciprocal form)
  std::map<std::string, float*> freq_tables;
  // persistent scratch, grown on demand while the stream is idle-ordered (single stream)
  void* gemm_scratch = nullptr;
  size_t gemm_scratch_bytes = 0;
  void* attn_scratch = nullptr;
  size_t attn_scratch_bytes = 0;
  // recycled pinned blocks for the per-submission error records (pointer, capacity in records)
  std::vector<std::pair<void*, size_t>> pinned_pool;
  std::mutex pinned_mutex;
};

// Paged-KV pool: device allocator state, page tables and the metadata of the last packed step.
struct fj_kvpool {
  fj_backend* be = nullptr;
  fj::KvPoolDevice dev{};
  uint64_t buf_free = 0, buf_count = 0, buf_gens = 0, buf_tables = 0, buf_lane_pages = 0, buf_refcounts = 0, buf_immutable = 0;
  // packer state
  uint64_t buf_lane_meta[5] = {0, 0, 0, 0, 0};  // logical_lengths, query_starts, absolute_positions, activity, cu_seqlens
  uint64_t buf_rows[3] = {0, 0, 0};             // positions, slot_mapping, row_lane
  uint64_t buf_stage = 0;                       // starts | tokens staged on the device
  uint32_t rows_cap = 0;
  fj::PackOutputs pack{};
  std::vector<uint32_t> host_starts, host_tokens;  // last packed step (host copy for grid sizing)
  uint32_t rows = 0, lanes_packed = 0;
  std::vector<uint64_t> lane_epoch;  // bumped when a lane is released: identity of the sequence a checkpoint was taken from
};

namespace fjb {

// Row-major [rows, width] view with the given row stride (elements), and its broadcast form for a
// [width] weight vector shared by every row.
inline fj::View dense_view(void* base, int dtype, unsigned rows, unsigned width, size_t row_stride) {
  fj::View v;
  v.base = base; v.dtype = dtype; v.rank = 2;
  for (int a = 0; a < 8; ++a) { v.shape[a] = 1; v.strides[a] = 0; }
  v.shape[0] = rows; v.shape[1] = width; v.strides[0] = row_stride; v.strides[1] = 1;
  return v;
}
inline fj::View weight_view(const void* base, int dtype, unsigned rows, unsigned width) {
  return dense_view(const_cast<void*>(base), dtype, rows, width, 0);
}
// Tokens of the previous step fed back as this step's inputs (last row of each lane), and the
// gather of every lane's last row into [lanes, width] (inactive lanes: zeros).
void launch_feedback_tokens(fj::Ctx& ctx, const unsigned* cu_seqlens, const unsigned* previous, unsigned* tokens, unsigned lanes);
void launch_gather_last_rows(fj::Ctx& ctx, const void* hidden, int dtype, const unsigned* cu_seqlens, void* out, unsigned lanes, unsigned width);

// Looks up a buffer; nullptr when unknown.
fj_buffer_rec* find_buffer(fj_backend* be, uint64_t id);
// Allocates a zeroed device buffer and registers it (quota checked). Returns an fj_status.
int32_t alloc_buffer(fj_backend* be, uint64_t bytes, uint64_t* id);
// Device pointer of a tensor's first element after bounds validation; nullptr on failure.
bool tensor_byte_span(const fj_tensor& t, uint64_t* lo, uint64_t* hi);
void* tensor_ptr(fj_backend* be, const fj_tensor& t, bool for_write);
bool make_view(fj_backend* be, const fj_tensor& t, bool for_write, fj::View* out);
bool is_contiguous(const fj_tensor& t);
uint64_t element_count(const fj_tensor& t);
// Rotary frequency table on the device: reciprocal == false: powf(theta, i * scale) (guest programs);
// reciprocal == true: 1 / powf(theta, 2 i / width) with width = count * 2 (Op::Rope).
const float* freq_table(fj_backend* be, float theta, float scale, unsigned count, bool reciprocal);
// Ensures the persistent scratch areas are at least this large (zero-filled when (re)allocated).
bool ensure_gemm_scratch(fj_backend* be, size_t bytes);
bool ensure_attn_scratch(fj_backend* be, size_t bytes);
int32_t cuda_status(cudaError_t e);

}  // namespace fjb
