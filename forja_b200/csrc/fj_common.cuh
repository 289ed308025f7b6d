// Shared device helpers for the forja sm_100a kernels: storage <-> f32 conversion with the
// reference's rounding (round to nearest even on every store, crates/forja-cpu/src/lib.rs:1836-1847),
// IEEE total-order keys, warp/block reductions and the per-dispatch error record.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fj {

enum DType : int { F32 = 0, F16 = 1, BF16 = 2, I32 = 3, U32 = 4 };

__host__ __device__ inline size_t dtype_size(int dt) { return (dt == F16 || dt == BF16) ? 2 : 4; }

// Per-dispatch error record written by kernels: never a trap, always a flag the host reads after
// completion (the reference's device contract: crates/forja-metal/src/paged.metal:39-55).
struct ErrorRecord {
  unsigned int flag;   // 0 ok, 1 index out of range, 2 page entry refused, 3 wait gave up
  unsigned int value;  // lowest offending value (initialised to 0xFFFFFFFF)
};
enum : unsigned int { ERR_INDEX = 1, ERR_PAGE = 2, ERR_WAIT = 3, ERR_INVALID = 4 };  // ERR_INVALID: a device-resident parameter failed validation

// Programmatic dependent launch: a kernel started with the stream-serialisation attribute may begin
// while its predecessor in the stream is still draining. `griddepcontrol.wait` blocks until that
// predecessor has completed and its writes are visible, so it must come before the first access to
// anything the predecessor wrote (or still reads); `launch_dependents` lets the successor start its
// own launch early. Both are no-ops for kernels started without the attribute.
__device__ inline void pdl_sync() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

__device__ inline void report_error(ErrorRecord* rec, unsigned int flag, unsigned int value) {
  if (rec == nullptr) return;
  atomicMax(&rec->flag, flag);
  atomicMin(&rec->value, value);
}

template <typename T> __device__ inline float to_f32(T v);
template <> __device__ inline float to_f32<float>(float v) { return v; }
template <> __device__ inline float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ inline float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ inline T from_f32(float v);
template <> __device__ inline float from_f32<float>(float v) { return v; }
template <> __device__ inline __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ inline __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Runtime-dtype element access (cold paths and generic kernels).
__device__ inline float load_as_f32(const void* base, int dt, size_t index) {
  switch (dt) {
    case F32: return static_cast<const float*>(base)[index];
    case F16: return __half2float(static_cast<const __half*>(base)[index]);
    default: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[index]);
  }
}
__device__ inline void store_from_f32(void* base, int dt, size_t index, float v) {
  switch (dt) {
    case F32: static_cast<float*>(base)[index] = v; break;
    case F16: static_cast<__half*>(base)[index] = __float2half_rn(v); break;
    default: static_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(v); break;
  }
}
// Rounds an f32 value through a storage dtype (re-inserts the rounding of a materialised tensor).
__device__ inline float round_through(float v, int dt) {
  switch (dt) {
    case F16: return __half2float(__float2half_rn(v));
    case BF16: return __bfloat162float(__float2bfloat16_rn(v));
    default: return v;
  }
}

// f32::total_cmp as an unsigned key (larger key = greater under IEEE total order). Keys are built
// from raw bits: routing a NaN through a float register before taking its bits lost the ordering
// of positive NaNs on sm_100a builds, so no float value is involved.
// Bits of element `index` widened to f32 with integer arithmetic only, so NaN sign and payload
// reach the ordering key untouched (the reference decodes f16/bf16 NaNs as sign | quiet | payload).
__device__ inline unsigned int load_f32_bits(const void* base, int dt, size_t index) {
  if (dt == F32) return static_cast<const unsigned int*>(base)[index];
  const unsigned int h = static_cast<const unsigned short*>(base)[index];
  if (dt == BF16) return ((h & 0x7FFFu) > 0x7F80u) ? ((h | 0x0040u) << 16) : (h << 16);
  const unsigned int sign = (h & 0x8000u) << 16, exp = h & 0x7C00u, man = h & 0x03FFu;
  if (exp == 0x7C00u) return man == 0 ? (sign | 0x7F800000u) : (sign | 0x7FC00000u | (man << 13));
  return static_cast<unsigned int>(__float_as_int(__half2float(__ushort_as_half(static_cast<unsigned short>(h)))));
}
__device__ inline unsigned int total_order_key_bits(unsigned int bits) {
  int b = static_cast<int>(bits);
  b ^= static_cast<int>(static_cast<unsigned int>(b >> 31) >> 1);
  return static_cast<unsigned int>(b) ^ 0x80000000u;
}
__device__ inline unsigned int key_to_bits(unsigned int key) {
  int b = static_cast<int>(key ^ 0x80000000u);
  b ^= static_cast<int>(static_cast<unsigned int>(b >> 31) >> 1);
  return static_cast<unsigned int>(b);
}

__device__ inline float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ inline unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}
// Block-wide sum; `scratch` holds 32 floats of shared memory. All threads get the result.
__device__ inline float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = lane < warps ? scratch[lane] : 0.0f;
  total = warp_sum(total);
  return total;
}

// Strided view descriptor passed by value to generic kernels.
struct View {
  void* base;          // allocation base pointer (already offset by the view's element offset)
  int dtype;
  int rank;
  unsigned int shape[8];
  unsigned long long strides[8];
};
__device__ inline size_t view_offset(const View& v, size_t linear) {
  if (v.rank == 1) return linear * v.strides[0];
  size_t off = 0;
#pragma unroll 1
  for (int a = v.rank - 1; a >= 0; --a) {
    off += (linear % v.shape[a]) * v.strides[a];
    linear /= v.shape[a];
  }
  return off;
}

}  // namespace fj
