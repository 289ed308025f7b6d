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

namespace fjb {

// Looks up a buffer; nullptr when unknown.
fj_buffer_rec* find_buffer(fj_backend* be, uint64_t id);
// Allocates a zeroed device buffer and registers it (quota checked). Returns an fj_status.
int32_t alloc_buffer(fj_backend* be, uint64_t bytes, uint64_t* id);
// Device pointer of a tensor's first element after bounds validation; nullptr on failure.
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
