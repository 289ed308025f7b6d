// Device-resident forward step of the sparse-MoE decoder (Qwen3-Coder-30B-A3B shape family) and
// expert parallelism over several GPUs.
//
// Reference op order (engines/qwen3-coder/src/lib.rs:886-947 forward_batch, :505-603 SparseMoe,
// crates/forja-sdk/src/nn.rs:29-45 moe_router_with):
//   QuantEmbed(q4) -> RmsNorm -> per layer { QuantMatmul qkv -> qk_norm_rope -> PagedSdpaAppend ->
//   QuantMatmul o -> residual_norm -> QuantMatmul(q8) router -> TopK{k, normalize} ->
//   GatherQuantMatmul pair (gate, up) + silu(gate)*up -> GatherQuantMatmul weighted sum (down)
//   + residual -> rms_norm } -> QuantMatmul lm_head -> Argmax.
// Activations are bf16 (the reference engine keeps f32 tensors); router logits, routing weights and
// the per-route down projections stay f32, as the fused epilogues of the reference see them.
//
// Expert parallelism (no reference counterpart: the reference is single-GPU). Experts are sharded
// contiguously, expert e lives on rank e / (experts / world); attention, router and the dense
// projections are replicated and every rank runs its own lanes. Per MoE layer:
//   1. route locally; each route's activation row goes into the slab of the rank that owns its
//      expert, slots handed out in (row, j) order; the per-peer row counts are exchanged and read
//      back by the host (one small copy per layer) so that only live rows travel;
//   2. all-to-all of the rows (NCCL send/recv over NVLink) with the local expert id of every row;
//   3. the owner runs gate/up/silu and down for the rows it received (f32 results);
//   4. all-to-all back; the origin adds  residual + sum_j w_j * down_j  in ascending j.
// Each route's arithmetic is the same kernel code as in the single-GPU path, so both paths give
// identical bits. Received rows land in local memory before any kernel reads them.
#include "fj_backend.h"

#include <chrono>
#include <thread>

#include <dlfcn.h>
#include <string.h>

#include <algorithm>
#include <vector>

using namespace fjb;

// ---- NCCL through dlopen: the library keeps no link-time dependency on it ----------------------
namespace {

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(void* id) = nullptr;
  int (*CommInitRank)(void** comm, int nranks, const void* id_by_value_128, int rank) = nullptr;
  int (*CommDestroy)(void* comm) = nullptr;
  int (*Send)(const void* buf, size_t count, int dtype, int peer, void* comm, cudaStream_t stream) = nullptr;
  int (*Recv)(void* buf, size_t count, int dtype, int peer, void* comm, cudaStream_t stream) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*CommAbort)(void* comm) = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mutex;

// ncclUniqueId is a 128-byte struct passed by value to ncclCommInitRank.
struct UniqueId { char bytes[128]; };
using CommInitRankFn = int (*)(void** comm, int nranks, UniqueId id, int rank);
constexpr int kNcclInt8 = 0;  // ncclInt8 / ncclChar

}  // namespace

// Polls `done()` until it answers true or `timeout_ms` has passed (0 = no limit); sleeps briefly between polls once the
// first millisecond is over. Returns false on expiry. The clock is injectable so that the expiry path can be exercised
// on the host without a device (fj_ep_poll_selftest).
template <typename Done, typename Clock>
bool poll_until(Done done, uint64_t timeout_ms, Clock now_ms) {
  const uint64_t begin = now_ms();
  for (;;) {
    if (done()) return true;
    const uint64_t waited = now_ms() - begin;
    if (timeout_ms != 0 && waited >= timeout_ms) return false;
    if (waited >= 1) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}
inline uint64_t steady_ms() {
  return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}

struct fj_ep {
  fj_backend* be = nullptr;
  void* comm = nullptr;
  uint32_t rank = 0, world = 1;
  uint64_t wait_timeout_ms = 60000;  // host waits on an exchange give up after this long (fj_ep_set_timeout)
  bool aborted = false;              // the communicator was aborted after a wait ran out: every later exchange answers FJ_TIMEOUT
  cudaEvent_t wait_event = nullptr;
};

extern "C" {

int32_t fj_ep_load(const char* libnccl_path) {
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.handle) return FJ_OK;
  void* h = dlopen(libnccl_path && libnccl_path[0] ? libnccl_path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return FJ_UNSUPPORTED_OPERATION;
  NcclApi api;
  api.handle = h;
  api.GetUniqueId = reinterpret_cast<int (*)(void*)>(dlsym(h, "ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<int (*)(void**, int, const void*, int)>(dlsym(h, "ncclCommInitRank"));
  api.CommDestroy = reinterpret_cast<int (*)(void*)>(dlsym(h, "ncclCommDestroy"));
  api.Send = reinterpret_cast<int (*)(const void*, size_t, int, int, void*, cudaStream_t)>(dlsym(h, "ncclSend"));
  api.Recv = reinterpret_cast<int (*)(void*, size_t, int, int, void*, cudaStream_t)>(dlsym(h, "ncclRecv"));
  api.GroupStart = reinterpret_cast<int (*)()>(dlsym(h, "ncclGroupStart"));
  api.GroupEnd = reinterpret_cast<int (*)()>(dlsym(h, "ncclGroupEnd"));
  api.CommAbort = reinterpret_cast<int (*)(void*)>(dlsym(h, "ncclCommAbort"));  // optional: only the watchdog uses it
  if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.Send || !api.Recv || !api.GroupStart || !api.GroupEnd) { dlclose(h); return FJ_UNSUPPORTED_OPERATION; }
  g_nccl = api;
  return FJ_OK;
}

int32_t fj_ep_unique_id(uint8_t* out128) {
  if (!out128 || !g_nccl.handle) return FJ_INVALID_INPUT;
  UniqueId id;
  memset(&id, 0, sizeof(id));
  if (g_nccl.GetUniqueId(&id) != 0) return FJ_DEVICE_EXECUTION_FAILED;
  memcpy(out128, id.bytes, 128);
  return FJ_OK;
}

int32_t fj_ep_create(fj_backend* be, const uint8_t* id128, uint32_t rank, uint32_t world, fj_ep** out) {
  if (!be || !id128 || !out || world == 0 || rank >= world || !g_nccl.handle) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  UniqueId id;
  memcpy(id.bytes, id128, 128);
  void* comm = nullptr;
  if (reinterpret_cast<CommInitRankFn>(g_nccl.CommInitRank)(&comm, static_cast<int>(world), id, static_cast<int>(rank)) != 0) return FJ_DEVICE_EXECUTION_FAILED;
  auto* ep = new fj_ep();
  ep->be = be; ep->comm = comm; ep->rank = rank; ep->world = world;
  *out = ep;
  return FJ_OK;
}

void fj_ep_destroy(fj_ep* ep) {
  if (!ep) return;
  {
    std::lock_guard<std::mutex> lock(ep->be->mutex);
    cudaSetDevice(ep->be->device);
    if (!ep->aborted) cudaStreamSynchronize(ep->be->stream);
    if (ep->comm) g_nccl.CommDestroy(ep->comm);
    if (ep->wait_event) cudaEventDestroy(ep->wait_event);
  }
  delete ep;
}

int32_t fj_ep_set_timeout(fj_ep* ep, uint64_t timeout_ms) {
  if (!ep) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(ep->be->mutex);
  ep->wait_timeout_ms = timeout_ms;
  return FJ_OK;
}

// Host-only check of the bounded wait: a condition that turns true after `ready_after_polls` polls (0 = never) is polled
// against a simulated clock that advances `tick_ms` per reading. Returns 1 when the wait saw the condition, 0 when it gave
// up at the deadline; *polls receives how often the condition was asked.
int32_t fj_ep_poll_selftest(uint64_t timeout_ms, uint64_t ready_after_polls, uint64_t tick_ms, uint64_t* polls) {
  uint64_t asked = 0, clock = 0;
  const bool ok = poll_until([&]() { ++asked; return ready_after_polls != 0 && asked >= ready_after_polls; }, timeout_ms, [&]() { clock += tick_ms; return clock; });
  if (polls) *polls = asked;
  return ok ? 1 : 0;
}

}  // extern "C"

namespace {

// Waits for everything enqueued on the backend's stream, but only so long: a peer that never posts its half of an exchange
// leaves the NCCL kernel waiting on the device for ever, and a plain stream synchronisation would hang the host with it.
// On expiry the communicator is aborted (ncclCommAbort ends its kernels), the group is marked dead and FJ_TIMEOUT comes back.
int32_t ep_wait_stream(fj_ep* ep) {
  cudaStream_t stream = ep->be->stream;
  if (ep->aborted) return FJ_TIMEOUT;
  if (!ep->wait_event && cudaEventCreateWithFlags(&ep->wait_event, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return FJ_DEVICE_EXECUTION_FAILED; }
  if (cudaEventRecord(ep->wait_event, stream) != cudaSuccess) { cudaGetLastError(); return FJ_DEVICE_EXECUTION_FAILED; }
  cudaError_t last = cudaSuccess;
  const bool finished = poll_until([&]() { last = cudaEventQuery(ep->wait_event); return last != cudaErrorNotReady; }, ep->wait_timeout_ms, steady_ms);
  if (finished) { if (last != cudaSuccess) { cudaGetLastError(); return FJ_DEVICE_EXECUTION_FAILED; } return FJ_OK; }
  cudaGetLastError();
  ep->aborted = true;
  if (g_nccl.CommAbort && ep->comm) { g_nccl.CommAbort(ep->comm); ep->comm = nullptr; }
  return FJ_TIMEOUT;
}

// Every rank sends bytes_per_peer to each peer and receives as much from each, on the backend's
// stream; the block for the rank itself is a device copy. Caller holds the backend mutex.
int32_t ep_all_to_all(fj_ep* ep, const void* send, void* recv, size_t bytes_per_peer) {
  if (ep->aborted || !ep->comm) return FJ_TIMEOUT;
  cudaStream_t stream = ep->be->stream;
  if (g_nccl.GroupStart() != 0) return FJ_DEVICE_EXECUTION_FAILED;
  int failed = 0;
  for (uint32_t peer = 0; peer < ep->world; ++peer) {
    const char* s = static_cast<const char*>(send) + static_cast<size_t>(peer) * bytes_per_peer;
    char* r = static_cast<char*>(recv) + static_cast<size_t>(peer) * bytes_per_peer;
    if (peer == ep->rank) { cudaMemcpyAsync(r, s, bytes_per_peer, cudaMemcpyDeviceToDevice, stream); continue; }
    failed |= g_nccl.Send(s, bytes_per_peer, kNcclInt8, static_cast<int>(peer), ep->comm, stream);
    failed |= g_nccl.Recv(r, bytes_per_peer, kNcclInt8, static_cast<int>(peer), ep->comm, stream);
  }
  if (g_nccl.GroupEnd() != 0 || failed) return FJ_DEVICE_EXECUTION_FAILED;
  return FJ_OK;
}

// Variable-size form: rank p gets send_counts[p] rows of row_bytes from send + send_rows_at[p] rows, and
// its recv_counts[p] rows land at recv + recv_rows_at[p] rows. Counts are host values.
int32_t ep_all_to_all_rows(fj_ep* ep, const void* send, const unsigned* send_rows_at, const unsigned* send_counts, void* recv, const unsigned* recv_rows_at,
                           const unsigned* recv_counts, size_t row_bytes, const void* send2 = nullptr, void* recv2 = nullptr, size_t row_bytes2 = 0) {
  if (ep->aborted || !ep->comm) return FJ_TIMEOUT;
  cudaStream_t stream = ep->be->stream;
  if (g_nccl.GroupStart() != 0) return FJ_DEVICE_EXECUTION_FAILED;
  int failed = 0;
  // a second array with the same row layout (the expert id of every row) travels in the same group
  for (int pass = 0; pass < (send2 ? 2 : 1); ++pass) {
  if (pass == 1) { send = send2; recv = recv2; row_bytes = row_bytes2; }
  for (uint32_t peer = 0; peer < ep->world; ++peer) {
    const char* s = static_cast<const char*>(send) + static_cast<size_t>(send_rows_at[peer]) * row_bytes;
    char* r = static_cast<char*>(recv) + static_cast<size_t>(recv_rows_at[peer]) * row_bytes;
    if (peer == ep->rank) {
      if (send_counts[peer]) cudaMemcpyAsync(r, s, static_cast<size_t>(send_counts[peer]) * row_bytes, cudaMemcpyDeviceToDevice, stream);
      continue;
    }
    if (send_counts[peer]) failed |= g_nccl.Send(s, static_cast<size_t>(send_counts[peer]) * row_bytes, kNcclInt8, static_cast<int>(peer), ep->comm, stream);
    if (recv_counts[peer]) failed |= g_nccl.Recv(r, static_cast<size_t>(recv_counts[peer]) * row_bytes, kNcclInt8, static_cast<int>(peer), ep->comm, stream);
  }
  }
  if (g_nccl.GroupEnd() != 0 || failed) return FJ_DEVICE_EXECUTION_FAILED;
  return FJ_OK;
}

// ---- expert-parallel dispatch / combine kernels -------------------------------------------------
// Every route takes the next free slot of its destination's slab (atomic counter per destination,
// zeroed by the caller). Which slot a route gets does not matter: results come back by slot.
__global__ void ep_plan_kernel(const unsigned* __restrict__ indices, unsigned routes, unsigned experts_local, unsigned world, unsigned capacity,
                               unsigned* send_experts, unsigned* route_slot, unsigned* send_counts) {
  for (unsigned r = blockIdx.x * blockDim.x + threadIdx.x; r < routes; r += gridDim.x * blockDim.x) {
    const unsigned expert = indices[r];
    const unsigned dest = expert / experts_local;
    if (dest >= world) { route_slot[r] = 0xFFFFFFFFu; continue; }  // bad expert id: contributes nothing
    const unsigned slot = dest * capacity + atomicAdd(&send_counts[dest], 1u);
    route_slot[r] = slot;
    if (send_experts) send_experts[slot] = expert - dest * experts_local;
  }
}

// Router logits for many rows on the tensor cores without giving up f32 weights: every dequantised
// router weight w = s * q + b (f32, rounded like the reference, crates/forja-cpu/src/lib.rs:878-962)
// is split into hi = bf16(w) and lo = bf16(w - hi), stacked as 2 * experts rows; x . hi and x . lo
// come out of one dense GEMM with f32 accumulators and are added afterwards (|w - hi - lo| <= 2^-17 |w|).
__global__ void router_split_kernel(const unsigned* __restrict__ packed, const unsigned short* __restrict__ scales, const unsigned short* __restrict__ biases, unsigned experts,
                                    unsigned k, unsigned bits, unsigned group_size, unsigned short* __restrict__ out /*[2 * experts][k]*/) {
  fj::pdl_sync();
  const unsigned vpw = 32 / bits, mask = (1u << bits) - 1, words_per_row = k / vpw, groups = k / group_size;
  const size_t total = static_cast<size_t>(experts) * words_per_row;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const unsigned row = static_cast<unsigned>(idx / words_per_row), wi = static_cast<unsigned>(idx % words_per_row);
    const unsigned word = packed[idx];
    const size_t g = static_cast<size_t>(row) * groups + (wi * vpw) / group_size;
    const float s = __uint_as_float(static_cast<unsigned>(scales[g]) << 16), b = __uint_as_float(static_cast<unsigned>(biases[g]) << 16);
    for (unsigned i = 0; i < vpw; ++i) {
      const float w = __fadd_rn(__fmul_rn(s, static_cast<float>((word >> (i * bits)) & mask)), b);
      const __nv_bfloat16 hi = __float2bfloat16_rn(w);
      const __nv_bfloat16 lo = __float2bfloat16_rn(w - __bfloat162float(hi));
      out[static_cast<size_t>(row) * k + wi * vpw + i] = __bfloat16_as_ushort(hi);
      out[static_cast<size_t>(experts + row) * k + wi * vpw + i] = __bfloat16_as_ushort(lo);
    }
  }
}

__global__ void router_sum_kernel(const float* __restrict__ halves /*[rows][2 * experts]*/, float* __restrict__ logits, unsigned rows, unsigned experts) {
  fj::pdl_sync();
  const size_t total = static_cast<size_t>(rows) * experts;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = idx / experts, e = idx % experts;
    logits[idx] = halves[row * 2 * experts + e] + halves[row * 2 * experts + experts + e];
  }
}

// Measurement aid: replaces a step's routing by an even spread: row r of layer l takes top_k distinct experts
// (start + j * stride) mod experts from a hash of (l, r), each with weight 1 / top_k.
__global__ void route_uniform_kernel(unsigned* route_experts, float* route_weights, unsigned rows, unsigned top_k, unsigned experts, unsigned layer) {
  const unsigned r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  unsigned h = (r + 1u) * 2654435761u ^ (layer + 1u) * 40503u;
  h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
  const unsigned start = h % experts, stride = experts > 1 ? 1u + 2u * ((h >> 8) % max(experts / 2, 1u)) : 0u;  // odd: no repeat within a power-of-two expert count
  for (unsigned j = 0; j < top_k; ++j) {
    route_experts[r * top_k + j] = static_cast<unsigned>((start + static_cast<unsigned long long>(j) * stride) % experts);
    route_weights[r * top_k + j] = 1.0f / static_cast<float>(top_k);
  }
}

// Copies each route's activation row (bf16, width % 8 == 0) into its slot, 16 bytes per thread step.
__global__ void ep_scatter_rows_kernel(const unsigned short* __restrict__ normed, const unsigned* __restrict__ route_slot, unsigned routes, unsigned top_k,
                                       unsigned width, unsigned short* send_rows) {
  const unsigned vecs = width / 8;
  for (unsigned r = blockIdx.x; r < routes; r += gridDim.x) {
    const unsigned slot = route_slot[r];
    if (slot == 0xFFFFFFFFu) continue;
    const uint4* src = reinterpret_cast<const uint4*>(normed + static_cast<size_t>(r / top_k) * width);
    uint4* dst = reinterpret_cast<uint4*>(send_rows + static_cast<size_t>(slot) * width);
    for (unsigned i = threadIdx.x; i < vecs; i += blockDim.x) dst[i] = src[i];
  }
}

// ---- direct exchange: rows are stored straight into the owner's memory over NVLink ----------------
// Ranks of one node map each other's receive buffers (CUDA IPC) and a layer's exchange becomes plain peer
// stores plus one 64-bit flag per (source, destination): {exchange number, row count}. The kernel that wrote
// the rows publishes the flag after a system-scope fence from its last block; the receiver polls its own
// memory, with a bound, and hands the counts to the kernels that follow on its stream. No host round trip,
// no staging copy, no multicast. Why no back-pressure flag is needed: a rank overwrites a peer's slab for
// exchange e + 1 only after it received that peer's results of exchange e, which the peer sent after it
// finished reading the slab.
struct EpPeers {
  unsigned short* const* rows;        // [world] every rank's recv_rows
  unsigned* const* experts;           // [world] every rank's recv_experts
  unsigned long long* const* flags;   // [world] every rank's flag words: [world] dispatch | [world] return
  const unsigned char* const* results;  // [world] every rank's per-route results (down_ep), read by the origin's combine
  unsigned char* const* returned;       // [world] every rank's `returned`, written by the owners when results are pushed
};

__device__ inline void st_release_sys(unsigned long long* p, unsigned long long v) { asm volatile("st.release.sys.global.u64 [%0], %1;\n" ::"l"(p), "l"(v) : "memory"); }
__device__ inline unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// The last block to finish publishes what the whole grid stored: true in exactly one block, after every block's
// stores were fenced at system scope. `ticket` returns to zero for the next launch.
__device__ inline bool ep_last_block(unsigned* ticket) {
  __shared__ bool s_last;
  __syncthreads();  // orders the block's stores before thread 0's fence: one system fence per block, not one per thread
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    if (s_last) *ticket = 0;
    __threadfence_system();
  }
  __syncthreads();
  return s_last;
}

// Dispatch: every route takes a slot of its destination's slab (which one does not matter, results are read back by slot):
// a block counts its routes per destination in shared memory and reserves the ranges with one atomic per destination, so the
// global counters see a few hundred atomics instead of one per route. Each route's activation row and local expert id then go
// into slot (rank * capacity + slot) of the owner's buffers, one warp per row with eight 16-byte pieces in flight per lane;
// finally flag[rank] of every peer = {exchange, rows sent to it}. Zeroes the send counters for the next layer.
// A chunk covers routes [route_begin, route_end) and owns slots [chunk_base, chunk_base + chunk_capacity) of every slab, its own
// counters, ticket and flag words (flag_base): chunks of one layer travel independently of each other.
__global__ void __launch_bounds__(256) ep_push_dispatch_kernel(const unsigned short* __restrict__ normed, const unsigned* __restrict__ route_experts, unsigned route_begin,
                                                               unsigned route_end, unsigned top_k, unsigned width, unsigned capacity, unsigned chunk_base, unsigned chunk_capacity,
                                                               unsigned rank, unsigned world, unsigned experts_local, EpPeers peers, unsigned* route_slot, unsigned* send_counts,
                                                               unsigned* ticket, unsigned flag_base, unsigned exchange) {
  __shared__ unsigned s_count[64], s_base[64], s_slot[256];
  const unsigned vecs = width / 8, lane = threadIdx.x & 31u, warp = threadIdx.x / 32, warps = blockDim.x / 32;
  const unsigned routes = route_end - route_begin;
  const unsigned per_block = (routes + gridDim.x - 1) / gridDim.x;
  const unsigned begin = route_begin + min(routes, blockIdx.x * per_block), end = min(route_end, begin + per_block);
  for (unsigned chunk = begin; chunk < end; chunk += blockDim.x) {
    if (threadIdx.x < 64) s_count[threadIdx.x] = 0;
    __syncthreads();
    const unsigned r = chunk + threadIdx.x;
    unsigned expert = 0, dest = 0xFFFFFFFFu, local = 0;
    if (r < end) {
      expert = route_experts[r];
      dest = expert / experts_local;
      if (dest < world) local = atomicAdd(&s_count[dest], 1u);
    }
    __syncthreads();
    if (threadIdx.x < world) s_base[threadIdx.x] = s_count[threadIdx.x] ? atomicAdd(&send_counts[threadIdx.x], s_count[threadIdx.x]) : 0u;
    __syncthreads();
    if (r < end) {
      unsigned slot = 0xFFFFFFFFu;  // bad expert id: contributes nothing
      if (dest < world) {
        const unsigned in = s_base[dest] + local;
        if (in < chunk_capacity) {
          slot = dest * capacity + chunk_base + in;
          peers.experts[dest][rank * capacity + chunk_base + in] = expert - dest * experts_local;
        }
      }
      route_slot[r] = slot;
      s_slot[threadIdx.x] = slot;
    }
    __syncthreads();
    const unsigned n = min(blockDim.x, end - chunk);
    for (unsigned i = warp; i < n; i += warps) {
      const unsigned slot = s_slot[i];
      if (slot == 0xFFFFFFFFu) continue;
      const unsigned to = slot / capacity, at = rank * capacity + slot % capacity;
      const uint4* src = reinterpret_cast<const uint4*>(normed + static_cast<size_t>((chunk + i) / top_k) * width);
      uint4* dst = reinterpret_cast<uint4*>(peers.rows[to] + static_cast<size_t>(at) * width);
      for (unsigned base = 0; base < vecs; base += 256) {
        uint4 v[8];
#pragma unroll
        for (unsigned u = 0; u < 8; ++u) {
          const unsigned k = base + u * 32 + lane;
          if (k < vecs) v[u] = src[k];
        }
#pragma unroll
        for (unsigned u = 0; u < 8; ++u) {
          const unsigned k = base + u * 32 + lane;
          if (k < vecs) dst[k] = v[u];
        }
      }
    }
    __syncthreads();
  }
  if (ep_last_block(ticket) && threadIdx.x < world) {
    const unsigned count = min(send_counts[threadIdx.x], chunk_capacity);
    send_counts[threadIdx.x] = 0;
    st_release_sys(peers.flags[threadIdx.x] + flag_base + rank, (static_cast<unsigned long long>(exchange) << 32) | count);
  }
}

// Waits, with a bound, until every source's flag carries this exchange number; stores the row counts for the
// kernels that follow. A wait that runs out sets *wait_err (and every later wait returns at once): the step then
// computes on zero rows and the host answers FJ_TIMEOUT; the context stays usable.
// signal_flags != nullptr: before waiting, publish {exchange, 0} in word signal_at of every peer's flags (the owner's "results
// of this exchange are ready": everything earlier on the stream has completed and the fence orders it before the flag).
// `capacity` bounds a count (the chunk's share of a slab); the chunk's ids of source s start at recv_experts[s * slab_stride].
__global__ void ep_wait_kernel(const unsigned long long* flags, unsigned world, unsigned exchange, unsigned capacity, unsigned* counts_out, unsigned* stale_counts, unsigned* recv_experts,
                               unsigned* live_total_host, unsigned* wait_err, unsigned max_polls, unsigned long long* const* signal_flags = nullptr, unsigned signal_at = 0,
                               unsigned slab_stride = 0) {
  __shared__ unsigned s_counts[64];
  const unsigned src = threadIdx.x;
  unsigned count = 0;
  if (signal_flags && src < world) {
    __threadfence_system();
    st_release_sys(signal_flags[src] + signal_at, static_cast<unsigned long long>(exchange) << 32);
  }
  if (src < world) {
    bool seen = false;
    for (unsigned poll = 0; poll < max_polls && *reinterpret_cast<volatile unsigned*>(wait_err) == 0; ++poll) {
      const unsigned long long v = ld_acquire_sys(flags + src);
      if (static_cast<unsigned>(v >> 32) == exchange) { count = min(static_cast<unsigned>(v), capacity); seen = true; break; }
      __nanosleep(poll < 64 ? 20 : 500);
    }
    if (!seen) atomicExch(wait_err, exchange ? exchange : 1u);
    if (counts_out) counts_out[src] = count;
  }
  if (src < 64) s_counts[src] = src < world ? count : 0;
  __syncthreads();
  if (recv_experts) {
    // ids left over from an earlier, longer slab must not look valid to kernels that read the whole slab
    for (unsigned s = 0; s < world; ++s) {
      const unsigned now = s_counts[s], before = stale_counts[s];
      for (unsigned i = now + threadIdx.x; i < before; i += blockDim.x) recv_experts[static_cast<size_t>(s) * slab_stride + i] = 0xFFFFFFFFu;
    }
    __syncthreads();
    if (src < world) stale_counts[src] = count;
  }
  if (threadIdx.x == 0 && live_total_host) {
    unsigned total = 0;
    for (unsigned s = 0; s < world; ++s) total += s_counts[s];
    *live_total_host = total;
  }
}

// Return by writing: the result row of slot (src * capacity + chunk_base + i), i < counts[src], goes to slot
// (rank * capacity + chunk_base + i) of src's `returned`; then return-flag[rank] of every peer = {exchange, 0}. The alternative to
// the reading combine below; it costs an extra pass over local memory on both sides and measured slower on 2 and on 8 GPUs
// (57.7 against 54.8 ms and 71.3 against 68.2 ms per step of the sparse-MoE benchmark), so it is not the default.
__global__ void ep_push_return_kernel(const unsigned char* __restrict__ results, unsigned row_bytes, unsigned capacity, unsigned chunk_base, unsigned chunk_capacity, unsigned rank,
                                      unsigned world, const unsigned* __restrict__ counts, EpPeers peers, unsigned* ticket, unsigned flag_base, unsigned exchange) {
  const unsigned vecs = row_bytes / 16, lane = threadIdx.x & 31u, warp = threadIdx.x / 32, warps = blockDim.x / 32;
  unsigned most = 0;
  for (unsigned src = 0; src < world; ++src) most = max(most, min(counts[src], chunk_capacity));
  // consecutive warps write to consecutive destinations, starting behind this rank: at any moment every destination is being
  // written by every source, instead of all sources converging on one destination after the other
  for (unsigned item = blockIdx.x * warps + warp; item < most * world; item += gridDim.x * warps) {
    const unsigned src = (rank + 1 + item % world) % world, i = item / world;
    if (i >= min(counts[src], chunk_capacity)) continue;
    {
      const uint4* from = reinterpret_cast<const uint4*>(results + (static_cast<size_t>(src) * capacity + chunk_base + i) * row_bytes);
      uint4* to = reinterpret_cast<uint4*>(peers.returned[src] + (static_cast<size_t>(rank) * capacity + chunk_base + i) * row_bytes);
      for (unsigned base = 0; base < vecs; base += 256) {
        uint4 v[8];
#pragma unroll
        for (unsigned u = 0; u < 8; ++u) {
          const unsigned k = base + u * 32 + lane;
          if (k < vecs) v[u] = from[k];
        }
#pragma unroll
        for (unsigned u = 0; u < 8; ++u) {
          const unsigned k = base + u * 32 + lane;
          if (k < vecs) to[k] = v[u];
        }
      }
    }
  }
  if (ep_last_block(ticket) && threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + flag_base + rank, static_cast<unsigned long long>(exchange) << 32);
}

// Return by reading instead of writing: the owner only publishes "results of this exchange are ready" (ep_wait_kernel's
// signal), and the origin's
// combine reads each route's result row from the owner's memory (peer loads over NVLink; all top_k rows of a column group are
// in flight before the first is used). Same arithmetic as routes_combine_kernel: sum over j ascending of the rounded products
// w_j * row_j, then the residual. Nothing is staged on either side. The owner overwrites its results for exchange e + 1 only
// after every peer's dispatch of e + 1 arrived, which each peer issues after this kernel of exchange e.
template <bool kBf16>
__global__ void __launch_bounds__(256) ep_pull_combine_kernel(const unsigned char* const* __restrict__ results /*[world] every rank's per-route results*/,
                                                              const unsigned* __restrict__ route_slot, const float* __restrict__ weights, const void* __restrict__ extra, int e_dt, void* out,
                                                              int out_dt, unsigned rows, unsigned top_k, unsigned width, unsigned capacity, unsigned rank) {
  constexpr unsigned kBatch = 8;
  for (unsigned row = blockIdx.x; row < rows; row += gridDim.x) {
    for (unsigned c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
      float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (unsigned j0 = 0; j0 < top_k; j0 += kBatch) {
        float4 v[kBatch];
        float w[kBatch];
        unsigned valid = 0;
#pragma unroll
        for (unsigned b = 0; b < kBatch; ++b) {
          const unsigned j = j0 + b;
          const unsigned slot = j < top_k ? route_slot[row * top_k + j] : 0xFFFFFFFFu;
          w[b] = 0.0f;
          v[b] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (slot == 0xFFFFFFFFu) continue;
          valid |= 1u << b;
          w[b] = weights[row * top_k + j];
          const size_t at = (static_cast<size_t>(rank) * capacity + slot % capacity) * width + c;
          const unsigned char* base = results[slot / capacity];
          if (kBf16) {
            const uint2 h = *reinterpret_cast<const uint2*>(base + at * 2);
            v[b] = make_float4(__uint_as_float(h.x << 16), __uint_as_float(h.x & 0xFFFF0000u), __uint_as_float(h.y << 16), __uint_as_float(h.y & 0xFFFF0000u));
          } else {
            v[b] = *reinterpret_cast<const float4*>(base + at * 4);
          }
        }
#pragma unroll
        for (unsigned b = 0; b < kBatch; ++b) {
          if (!(valid >> b & 1u)) continue;
          total[0] = __fadd_rn(total[0], __fmul_rn(w[b], v[b].x));
          total[1] = __fadd_rn(total[1], __fmul_rn(w[b], v[b].y));
          total[2] = __fadd_rn(total[2], __fmul_rn(w[b], v[b].z));
          total[3] = __fadd_rn(total[3], __fmul_rn(w[b], v[b].w));
        }
      }
      const size_t o = static_cast<size_t>(row) * width + c;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (extra) total[i] = total[i] + fj::load_as_f32(extra, e_dt, o + i);
        fj::store_from_f32(out, out_dt, o + i, total[i]);
      }
    }
  }
}

}  // namespace

// ---- the model ------------------------------------------------------------------------------------
namespace {
struct QuantW {
  const unsigned* packed = nullptr;
  const void* scales = nullptr;
  const void* biases = nullptr;
};
}  // namespace

struct fj_moe_model {
  fj_backend* be = nullptr;
  fj_kvpool* pool = nullptr;
  fj_ep* ep = nullptr;
  fj_moe_config cfg{};
  uint32_t experts_local = 0, world = 1, capacity = 0;
  QuantW embed, lm_head;
  const void* final_norm = nullptr;
  struct Layer {
    const void *input_norm, *q_norm, *k_norm, *post_norm;
    QuantW qkv, o, router, gate, up, down;
    void *k_plane, *v_plane;
  };
  std::vector<Layer> layers;
  std::vector<void*> owned;
  // workspace (bf16 unless noted)
  void *hidden = nullptr, *hidden2 = nullptr, *normed = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *proj = nullptr, *act = nullptr;
  float *router_logits = nullptr, *route_weights = nullptr;
  float* router_halves = nullptr;          // [max_rows][2 * experts] f32: x . hi | x . lo
  unsigned short* router_split = nullptr;  // [2 * experts][hidden] bf16, rebuilt per layer
  unsigned* route_experts = nullptr;
  void *last_hidden = nullptr, *last_normed = nullptr, *logits = nullptr, *argmax_scratch = nullptr, *dequant = nullptr;
  size_t dequant_bytes = 0;
  unsigned *tokens_in = nullptr, *tokens_out = nullptr;
  // expert parallelism: slabs of `capacity` slots per peer
  unsigned short *send_rows = nullptr, *recv_rows = nullptr, *act_ep = nullptr;
  unsigned *send_experts = nullptr, *recv_experts = nullptr, *route_slot = nullptr;
  float *down_ep = nullptr, *returned = nullptr;
  unsigned *ep_counts = nullptr;       // device: per chunk, send counts [world] | receive counts [world]
  unsigned* ep_counts_host = nullptr;  // pinned copy of both
  // direct exchange (peer stores; fj_moe_ep_connect): tables of every rank's buffers, this rank's flag words
  bool ep_direct = false;
  std::vector<void*> ep_opened;        // peer mappings to close
  void** ep_tables = nullptr;          // device: [5][world] pointers (rows | experts | flags | per-route results | returned)
  unsigned long long* ep_flags = nullptr;  // device: [chunks][2 * world] (dispatch | return), written by the peers
  unsigned* ep_state = nullptr;        // device: wait_err [1] | dispatch tickets [chunks] | return tickets [chunks] | stale counts [chunks][world]
  uint32_t ep_return_mode = 0;         // 0 or 1 = the origin reads the results, 2 = the owner writes them
  uint32_t ep_chunks = 1, ep_chunk_capacity = 0;  // chunks per layer and each chunk's share of a slab (capacity = chunks * share)
  std::vector<cudaStream_t> ep_streams;  // streams of chunks 1.. (chunk 0 runs on the backend's stream)
  std::vector<cudaEvent_t> ep_events;    // [0] router done | [1 + 3 c + {0 pushed, 1 experts done, 2 combined}]
  std::vector<void*> ep_plans;           // route plan of every chunk
  unsigned* ep_live_host = nullptr;    // mapped pinned: rows received per (layer, chunk) in the previous step, then wait_err copy [1]
  unsigned* ep_live_dev = nullptr;     // the same memory as the device sees it
  uint32_t ep_exchange = 0;            // exchanges done so far (all ranks count alike)
  uint32_t ep_max_polls = 1u << 24;    // about ten seconds of polling before a wait gives up (fj_moe_ep_wait_polls)
  // grouped expert path (many routes): route plan and per-route f32 down projections
  void* route_plan = nullptr;
  float* down_routes = nullptr;
  fj::AttnSeq* seqs = nullptr;
  fj::AttnWork* work = nullptr;
  unsigned* n_work_dev = nullptr;
  uint32_t work_cap = 0;
  uint2* prefill_items = nullptr;  // {lane, first token} blocks of the chunked-prefill attention
  uint32_t prefill_items_cap = 0;
  const float* inv_freq = nullptr;
  uint64_t last_kernels = 0, last_work_items = 0;
  // optional record of every layer's routing of the last step (parity checks): [layers][max_rows * top_k]
  std::vector<cudaEvent_t> phase_events;  // [layers][5] when phase timing is on
  unsigned* captured_experts = nullptr;
  float* captured_weights = nullptr;
  bool uniform_routing = false;  // measurement aid (fj_moe_uniform_routing)
};

extern "C" {

int32_t fj_ep_all_to_all(fj_ep* ep, uint64_t send, uint64_t recv, uint64_t bytes_per_peer) {
  if (!ep) return FJ_INVALID_INPUT;
  fj_backend* be = ep->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  fj_buffer_rec *s = find_buffer(be, send), *r = find_buffer(be, recv);
  const uint64_t total = bytes_per_peer * ep->world;
  if (!s || !r || r->readonly || s->bytes < total || r->bytes < total || s == r) return FJ_INVALID_INPUT;
  return ep_all_to_all(ep, s->ptr, r->ptr, bytes_per_peer);
}

int32_t fj_moe_model_create(fj_backend* be, const fj_moe_config* config, const fj_quant_weight* embed, uint64_t final_norm, const fj_quant_weight* lm_head,
                            const fj_moe_layer_weights* layers, fj_kvpool* pool, fj_ep* ep, fj_moe_model** out) {
  if (!be || !config || !embed || !lm_head || !layers || !pool || !out || pool->be != be || (ep && ep->be != be)) return FJ_INVALID_INPUT;
  const fj_moe_config& c = *config;
  const uint32_t world = ep ? ep->world : 1;
  if (c.layers == 0 || c.kv_heads == 0 || c.q_heads % c.kv_heads != 0 || c.head_dim % 2 != 0 || c.head_dim > 256 || c.max_rows == 0 || c.hidden % 8 != 0 || c.vocab == 0 ||
      c.experts == 0 || c.experts % world != 0 || c.top_k == 0 || c.top_k > c.experts || c.expert_intermediate == 0 || (c.group_size != 32 && c.group_size != 64 && c.group_size != 128) ||
      (c.router_bits != 4 && c.router_bits != 8) || c.hidden % c.group_size != 0 || c.expert_intermediate % c.group_size != 0 || (c.q_heads * c.head_dim) % c.group_size != 0)
    return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  auto* m = new fj_moe_model();
  m->be = be; m->pool = pool; m->ep = ep; m->cfg = c; m->world = world;
  m->experts_local = c.experts / world;
  m->ep_chunks = world > 1 ? std::min<uint32_t>(std::max<uint32_t>(c.ep_chunks, 1), 8) : 1;
  m->ep_chunk_capacity = (c.max_rows + m->ep_chunks - 1) / m->ep_chunks * c.top_k;
  m->capacity = m->ep_chunks * m->ep_chunk_capacity;  // >= max_rows * top_k
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
  auto vec = [&](uint64_t id, uint64_t elements) -> const void* {
    fj_buffer_rec* r = find_buffer(be, id);
    if (!r || r->bytes < elements * 2) { ok = false; return nullptr; }
    return r->ptr;
  };
  // a quantised tensor of `count` stacked [n, k] matrices
  auto quant = [&](const fj_quant_weight& w, uint64_t count, uint64_t n, uint64_t k, uint32_t bits) -> QuantW {
    QuantW q;
    fj_buffer_rec *p = find_buffer(be, w.packed), *s = find_buffer(be, w.scales), *b = find_buffer(be, w.biases);
    const uint64_t groups = count * n * (k / c.group_size);
    if (!p || !s || !b || p->bytes < count * n * (k * bits / 32) * 4 || s->bytes < groups * 2 || b->bytes < groups * 2) { ok = false; return q; }
    q.packed = static_cast<const unsigned*>(p->ptr); q.scales = s->ptr; q.biases = b->ptr;
    return q;
  };
  const uint64_t H = c.hidden, I = c.expert_intermediate, qd = static_cast<uint64_t>(c.q_heads) * c.head_dim, kd = static_cast<uint64_t>(c.kv_heads) * c.head_dim;
  m->embed = quant(*embed, 1, c.vocab, H, 4);
  m->lm_head = quant(*lm_head, 1, c.vocab, H, 4);
  m->final_norm = vec(final_norm, H);
  const size_t plane_bytes = static_cast<size_t>(pool->dev.physical_pages) * pool->dev.page_tokens * kd * 2;
  m->layers.resize(c.layers);
  for (uint32_t l = 0; l < c.layers && ok; ++l) {
    const fj_moe_layer_weights& w = layers[l];
    auto& L = m->layers[l];
    L.input_norm = vec(w.input_norm, H);
    L.post_norm = vec(w.post_norm, H);
    L.q_norm = vec(w.q_norm, c.head_dim);
    L.k_norm = vec(w.k_norm, c.head_dim);
    L.qkv = quant(w.qkv, 1, qd + 2 * kd, H, 4);
    L.o = quant(w.o, 1, H, qd, 4);
    L.router = quant(w.router, 1, c.experts, H, c.router_bits);
    L.gate = quant(w.gate, m->experts_local, I, H, 4);
    L.up = quant(w.up, m->experts_local, I, H, 4);
    L.down = quant(w.down, m->experts_local, H, I, 4);
    L.k_plane = dev_alloc(plane_bytes);
    L.v_plane = dev_alloc(plane_bytes);
  }
  const size_t R = c.max_rows, Lanes = pool->dev.lanes, K = c.top_k;
  m->hidden = dev_alloc(R * H * 2);
  m->hidden2 = dev_alloc(R * H * 2);
  m->normed = dev_alloc(R * H * 2);
  m->qkv = dev_alloc(R * (qd + 2 * kd) * 2);
  m->q = dev_alloc(R * qd * 2);
  m->attn = dev_alloc(R * qd * 2);
  m->proj = dev_alloc(R * H * 2);
  m->act = dev_alloc(R * K * I * 2);
  m->router_logits = static_cast<float*>(dev_alloc(R * c.experts * 4));
  if (R > 16) {
    m->router_halves = static_cast<float*>(dev_alloc(R * 2 * c.experts * 4));
    m->router_split = static_cast<unsigned short*>(dev_alloc(2 * static_cast<size_t>(c.experts) * H * 2));
  }
  m->route_weights = static_cast<float*>(dev_alloc(R * K * 4));
  m->route_experts = static_cast<unsigned*>(dev_alloc(R * K * 4));
  m->last_hidden = dev_alloc(Lanes * H * 2);
  m->last_normed = dev_alloc(Lanes * H * 2);
  m->logits = dev_alloc(Lanes * c.vocab * 2);
  m->argmax_scratch = dev_alloc(fj::argmax_scratch_bytes(static_cast<unsigned>(Lanes), c.vocab));
  m->tokens_in = static_cast<unsigned*>(dev_alloc(R * 4));
  m->tokens_out = static_cast<unsigned*>(dev_alloc(Lanes * 4));
  m->seqs = static_cast<fj::AttnSeq*>(dev_alloc(Lanes * sizeof(fj::AttnSeq)));
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
  if (std::max(R, Lanes) > 16) {
    // slab of dequantised weights for projections with more than 16 rows (tensor-core GEMM path)
    const uint64_t widest = std::max<uint64_t>({qd + 2 * kd, H, static_cast<uint64_t>(c.vocab)});
    m->dequant_bytes = static_cast<size_t>(std::min<uint64_t>(widest * std::max<uint64_t>(H, qd) * 2, uint64_t(64) << 20));
    m->dequant = dev_alloc(m->dequant_bytes);
  }
  if (world > 1) {
    const size_t slots = static_cast<size_t>(world) * m->capacity;
    m->send_rows = static_cast<unsigned short*>(dev_alloc(slots * H * 2));
    m->recv_rows = static_cast<unsigned short*>(dev_alloc(slots * H * 2));
    m->act_ep = static_cast<unsigned short*>(dev_alloc(slots * I * 2));
    m->send_experts = static_cast<unsigned*>(dev_alloc(slots * 4));
    m->recv_experts = static_cast<unsigned*>(dev_alloc(slots * 4));
    m->route_slot = static_cast<unsigned*>(dev_alloc(R * K * 4));
    m->down_ep = static_cast<float*>(dev_alloc(slots * H * 4));
    m->returned = static_cast<float*>(dev_alloc(slots * H * 4));
    const uint32_t chunks = m->ep_chunks;
    m->ep_counts = static_cast<unsigned*>(dev_alloc(static_cast<size_t>(chunks) * 2 * world * 4));
    if (cudaMallocHost(reinterpret_cast<void**>(&m->ep_counts_host), 2 * world * 4) != cudaSuccess) { cudaGetLastError(); ok = false; }
    m->ep_flags = static_cast<unsigned long long*>(dev_alloc(static_cast<size_t>(chunks) * 2 * world * 8));
    m->ep_state = static_cast<unsigned*>(dev_alloc((1 + 2 * chunks + static_cast<size_t>(chunks) * world) * 4));
    m->ep_tables = static_cast<void**>(dev_alloc(5 * world * sizeof(void*)));
    for (uint32_t ch = 1; ch < chunks && ok; ++ch) {
      cudaStream_t extra = nullptr;
      if (cudaStreamCreateWithFlags(&extra, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); ok = false; break; }
      m->ep_streams.push_back(extra);
      m->ep_plans.push_back(dev_alloc(fj::route_plan_bytes(static_cast<unsigned>(slots), m->experts_local)));
    }
    for (uint32_t e = 0; e < 1 + 3 * chunks && ok && chunks > 1; ++e) {
      cudaEvent_t ev = nullptr;
      if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); ok = false; break; }
      m->ep_events.push_back(ev);
    }
    if (ok) {
      cudaMemsetAsync(m->recv_experts, 0xFF, slots * 4, be->stream);
      const size_t words = static_cast<size_t>(c.layers) * chunks + 1;
      if (cudaHostAlloc(reinterpret_cast<void**>(&m->ep_live_host), words * 4, cudaHostAllocMapped) != cudaSuccess ||
          cudaHostGetDevicePointer(reinterpret_cast<void**>(&m->ep_live_dev), m->ep_live_host, 0) != cudaSuccess) { cudaGetLastError(); ok = false; }
      else memset(m->ep_live_host, 0, words * 4);
    }
    m->route_plan = dev_alloc(fj::route_plan_bytes(static_cast<unsigned>(slots), m->experts_local));
    m->ep_plans.insert(m->ep_plans.begin(), m->route_plan);
  } else {
    m->route_plan = dev_alloc(fj::route_plan_bytes(static_cast<unsigned>(R * K), c.experts));
    m->down_routes = static_cast<float*>(dev_alloc(R * K * H * 4));
  }
  if (ok) {
    m->inv_freq = freq_table(be, c.theta, -2.0f / static_cast<float>(c.head_dim), c.head_dim / 2, false);
    ok = m->inv_freq != nullptr;
  }
  if (ok) ok = ensure_gemm_scratch(be, fj::gemm_scratch_bytes(static_cast<unsigned>(std::max(R, Lanes)), static_cast<unsigned>(std::max<uint64_t>(qd + 2 * kd, H)), static_cast<unsigned>(std::max<uint64_t>(H, qd))));
  if (!ok || cudaStreamSynchronize(be->stream) != cudaSuccess) {
    for (void* p : m->owned) { cudaFree(p); }
    for (cudaStream_t st : m->ep_streams) cudaStreamDestroy(st);
    for (cudaEvent_t ev : m->ep_events) cudaEventDestroy(ev);
    if (m->ep_counts_host) cudaFreeHost(m->ep_counts_host);
    if (m->ep_live_host) cudaFreeHost(m->ep_live_host);
    delete m;
    return ok ? FJ_ALLOCATION_FAILED : FJ_INVALID_INPUT;
  }
  *out = m;
  return FJ_OK;
}

void fj_moe_model_destroy(fj_moe_model* m) {
  if (!m) return;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  cudaStreamSynchronize(m->be->stream);
  for (cudaStream_t st : m->ep_streams) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
  for (cudaEvent_t ev : m->ep_events) cudaEventDestroy(ev);
  for (void* p : m->ep_opened) cudaIpcCloseMemHandle(p);  // normally closed earlier by fj_moe_ep_disconnect, before any rank frees
  for (void* p : m->owned) cudaFree(p);
  for (cudaEvent_t e : m->phase_events) cudaEventDestroy(e);
  if (m->ep_counts_host) cudaFreeHost(m->ep_counts_host);
  if (m->ep_live_host) cudaFreeHost(m->ep_live_host);
  delete m;
}

// ---- direct exchange: connecting the ranks of one node -------------------------------------------------
// fj_moe_ep_export writes this rank's five buffer handles (5 x 64 bytes: received rows, received expert ids,
// flag words, per-route results, returned rows); the caller gathers every rank's 320 bytes in rank order (any host channel) and
// hands the whole table to fj_moe_ep_connect, which maps the peers' buffers. Every rank then passes whether its
// connect succeeded through the same channel and calls fj_moe_ep_direct(model, 1) only if all did: the choice
// between this exchange and the NCCL one must be the same on all ranks. Before any rank destroys its model,
// all call fj_moe_ep_disconnect and meet at a host barrier: a mapping must be closed before its owner frees.
int32_t fj_moe_ep_export(fj_moe_model* m, uint8_t* out320) {
  if (!m || !out320 || m->world < 2) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* bufs[5] = {m->recv_rows, m->recv_experts, m->ep_flags, m->down_ep, m->returned};
  for (int i = 0; i < 5; ++i) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, bufs[i]) != cudaSuccess) { cudaGetLastError(); return FJ_UNSUPPORTED_OPERATION; }
    memcpy(out320 + 64 * i, &h, 64);
  }
  return FJ_OK;
}

int32_t fj_moe_ep_connect(fj_moe_model* m, const uint8_t* table /*[world][320]*/) {
  if (!m || !table || m->world < 2 || m->world > 64 || !m->ep) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  if (!m->ep_opened.empty() || m->ep_direct) return FJ_INVALID_INPUT;
  const uint32_t W = m->world, rank = m->ep->rank;
  std::vector<void*> host(5 * static_cast<size_t>(W), nullptr);
  void* own[5] = {m->recv_rows, m->recv_experts, m->ep_flags, m->down_ep, m->returned};
  for (uint32_t p = 0; p < W; ++p)
    for (int i = 0; i < 5; ++i) {
      if (p == rank) { host[static_cast<size_t>(i) * W + p] = own[i]; continue; }
      cudaIpcMemHandle_t h;
      memcpy(&h, table + 320 * static_cast<size_t>(p) + 64 * i, 64);
      void* mapped = nullptr;
      if (cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        for (void* q : m->ep_opened) cudaIpcCloseMemHandle(q);
        m->ep_opened.clear();
        return FJ_UNSUPPORTED_OPERATION;
      }
      m->ep_opened.push_back(mapped);
      host[static_cast<size_t>(i) * W + p] = mapped;
    }
  if (cudaMemcpyAsync(m->ep_tables, host.data(), host.size() * sizeof(void*), cudaMemcpyHostToDevice, m->be->stream) != cudaSuccess ||
      cudaStreamSynchronize(m->be->stream) != cudaSuccess) { cudaGetLastError(); return FJ_DEVICE_EXECUTION_FAILED; }
  return FJ_OK;
}

int32_t fj_moe_ep_direct(fj_moe_model* m, uint32_t enabled) {
  if (!m || m->world < 2) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  if (enabled && m->ep_opened.size() != 5 * static_cast<size_t>(m->world - 1)) return FJ_INVALID_INPUT;
  m->ep_direct = enabled != 0;
  return FJ_OK;
}

int32_t fj_moe_ep_disconnect(fj_moe_model* m) {
  if (!m) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  cudaStreamSynchronize(m->be->stream);
  m->ep_direct = false;
  for (void* p : m->ep_opened) cudaIpcCloseMemHandle(p);
  m->ep_opened.clear();
  return FJ_OK;
}

// Bound of the device-side waits of the direct exchange, in polls (about half a microsecond each).
int32_t fj_moe_ep_wait_polls(fj_moe_model* m, uint32_t polls) {
  if (!m || polls == 0) return FJ_INVALID_INPUT;
  m->ep_max_polls = polls;
  return FJ_OK;
}

// How results travel back in the direct exchange: 0 or 1 = the origin's combine reads them from the owner's memory (default),
// 2 = the owner writes them into the origin's memory. All ranks must choose alike.
int32_t fj_moe_ep_return_mode(fj_moe_model* m, uint32_t mode) {
  if (!m || mode > 2) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  m->ep_return_mode = mode;
  return FJ_OK;
}

// Rows this rank received for its experts in the last finished step, per (layer, chunk): out[layers * chunks]. Tells how evenly
// the router spreads the work over the ranks; a rank with more rows than the others makes everybody wait at that layer's return.
int32_t fj_moe_ep_received(fj_moe_model* m, uint32_t* out, uint32_t words) {
  if (!m || !out || !m->ep_live_host || words < m->cfg.layers * m->ep_chunks) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  if (cudaStreamSynchronize(m->be->stream) != cudaSuccess) { cudaGetLastError(); return FJ_DEVICE_EXECUTION_FAILED; }
  memcpy(out, m->ep_live_host, static_cast<size_t>(m->cfg.layers) * m->ep_chunks * 4);
  return FJ_OK;
}

// Self-test of the bounded wait (no peer involved): waits on a flag that nothing sets, with `polls` polls,
// and answers FJ_TIMEOUT when the kernel gave up and reported it, FJ_OK if it did not. The context stays usable.
int32_t fj_ep_wait_selftest(fj_backend* be, uint32_t polls) {
  if (!be || polls == 0) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  void* mem = nullptr;
  if (cudaMalloc(&mem, 64) != cudaSuccess) { cudaGetLastError(); return FJ_ALLOCATION_FAILED; }
  cudaMemsetAsync(mem, 0, 64, be->stream);
  unsigned long long* flag = static_cast<unsigned long long*>(mem);
  unsigned* err = reinterpret_cast<unsigned*>(flag + 2);
  ep_wait_kernel<<<1, 64, 0, be->stream>>>(flag, 1, 7, 1, nullptr, nullptr, nullptr, nullptr, err, polls);
  unsigned host_err = 0;
  cudaMemcpyAsync(&host_err, err, 4, cudaMemcpyDeviceToHost, be->stream);
  const cudaError_t e = cudaStreamSynchronize(be->stream);
  cudaFree(mem);
  if (e != cudaSuccess) { cudaGetLastError(); return FJ_DEVICE_EXECUTION_FAILED; }
  return host_err == 7 ? FJ_TIMEOUT : FJ_OK;
}

int32_t fj_moe_phase_timing(fj_moe_model* m, uint32_t enabled) {
  if (!m) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  cudaStreamSynchronize(m->be->stream);
  for (cudaEvent_t e : m->phase_events) cudaEventDestroy(e);
  m->phase_events.clear();
  if (enabled) {
    m->phase_events.resize(static_cast<size_t>(m->cfg.layers) * 5);
    for (cudaEvent_t& e : m->phase_events)
      if (cudaEventCreate(&e) != cudaSuccess) return FJ_ALLOCATION_FAILED;
  }
  return FJ_OK;
}

int32_t fj_moe_read_phase_ms(fj_moe_model* m, float* out4) {
  if (!m || !out4 || m->phase_events.empty()) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  cudaSetDevice(m->be->device);
  if (cudaStreamSynchronize(m->be->stream) != cudaSuccess) return FJ_DEVICE_EXECUTION_FAILED;
  for (int i = 0; i < 4; ++i) out4[i] = 0.0f;
  for (uint32_t l = 0; l < m->cfg.layers; ++l)
    for (int i = 0; i < 4; ++i) {
      float ms = 0.0f;
      if (cudaEventElapsedTime(&ms, m->phase_events[l * 5 + i], m->phase_events[l * 5 + i + 1]) != cudaSuccess) { cudaGetLastError(); return FJ_INVALID_INPUT; }
      out4[i] += ms;
    }
  return FJ_OK;
}

int32_t fj_moe_uniform_routing(fj_moe_model* m, uint32_t enabled) {
  if (!m) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(m->be->mutex);
  m->uniform_routing = enabled != 0;
  return FJ_OK;
}

int32_t fj_moe_capture_routes(fj_moe_model* m, uint32_t enabled) {
  if (!m) return FJ_INVALID_INPUT;
  fj_backend* be = m->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  if (enabled && !m->captured_experts) {
    const size_t bytes = static_cast<size_t>(m->cfg.layers) * m->cfg.max_rows * m->cfg.top_k * 4;
    void *a = nullptr, *b = nullptr;
    if (cudaMalloc(&a, bytes) != cudaSuccess || cudaMalloc(&b, bytes) != cudaSuccess) { cudaGetLastError(); if (a) cudaFree(a); return FJ_ALLOCATION_FAILED; }
    m->owned.push_back(a);
    m->owned.push_back(b);
    m->captured_experts = static_cast<unsigned*>(a);
    m->captured_weights = static_cast<float*>(b);
  }
  if (!enabled) { m->captured_experts = nullptr; m->captured_weights = nullptr; }  // the buffers stay owned by the model
  return FJ_OK;
}

int32_t fj_moe_read_routes(fj_moe_model* m, uint32_t layer, uint32_t rows, uint32_t* experts, float* weights) {
  if (!m || !m->captured_experts || layer >= m->cfg.layers || rows > m->cfg.max_rows || !experts || !weights) return FJ_INVALID_INPUT;
  fj_backend* be = m->be;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const size_t at = static_cast<size_t>(layer) * m->cfg.max_rows * m->cfg.top_k, count = static_cast<size_t>(rows) * m->cfg.top_k;
  cudaMemcpyAsync(experts, m->captured_experts + at, count * 4, cudaMemcpyDeviceToHost, be->stream);
  cudaMemcpyAsync(weights, m->captured_weights + at, count * 4, cudaMemcpyDeviceToHost, be->stream);
  return cuda_status(cudaStreamSynchronize(be->stream));
}

int32_t fj_moe_step_stats(fj_moe_model* m, uint64_t* kernels, uint64_t* attn_work_items) {
  if (!m) return FJ_INVALID_INPUT;
  if (kernels) *kernels = m->last_kernels;
  if (attn_work_items) *attn_work_items = m->last_work_items;
  return FJ_OK;
}

}  // extern "C"

extern "C" int32_t fj_moe_step(fj_moe_model* m, const uint32_t* token_ids, uint32_t* out_tokens, uint64_t logits_out) {
  if (!m) return FJ_INVALID_INPUT;
  fj_backend* be = m->be;
  fj_kvpool* pool = m->pool;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const fj_moe_config& c = m->cfg;
  const unsigned rows = pool->rows, lanes = pool->lanes_packed;
  if (lanes == 0 || rows > c.max_rows) return FJ_INVALID_INPUT;
  if (rows == 0 && m->world == 1) return FJ_INVALID_INPUT;
  const int dt = FJ_BF16;
  const unsigned qd = c.q_heads * c.head_dim, kd = c.kv_heads * c.head_dim, H = c.hidden, I = c.expert_intermediate, K = c.top_k, G = c.group_size;
  fj::Ctx& ctx = be->ctx;
  const unsigned long long launches_before = ctx.launches;
  auto q4 = [&](const void* x, const QuantW& w, void* out, int out_dt, unsigned m_rows, unsigned k, unsigned n, unsigned bits) {
    fj::launch_quant_matmul(ctx, x, dt, w.packed, w.scales, w.biases, dt, out, out_dt, m_rows, k, n, bits, G, m_rows > 16 ? m->dequant : nullptr,
                            m_rows > 16 ? m->dequant_bytes : 0, be->gemm_scratch, be->gemm_scratch_bytes);
  };

  // attention plan for this step (shared by all layers)
  const unsigned group = c.q_heads / c.kv_heads;
  unsigned max_q_len = 0;
  uint64_t total_keys = 0;
  for (unsigned l = 0; l < lanes; ++l) {
    max_q_len = std::max(max_q_len, pool->host_tokens[l]);
    if (pool->host_tokens[l]) total_keys += static_cast<uint64_t>(pool->host_starts[l]) + pool->host_tokens[l];
  }
  fj::AttnGeometry g;
  g.q_heads = c.q_heads; g.kv_heads = c.kv_heads; g.head_dim = c.head_dim; g.value_dim = c.head_dim; g.page_tokens = pool->dev.page_tokens;
  g.physical_pages = pool->dev.physical_pages; g.q_dtype = dt; g.kv_dtype = dt; g.out_dtype = dt;
  g.scale = 1.0f / sqrtf(static_cast<float>(c.head_dim));
  const bool mma = rows != 0 && fj::attn_decode_mma_supported(g, max_q_len) && max_q_len * group <= 16;
  uint64_t chunk = 64, n_work = 0;
  fj::AttnScratch scratch{nullptr, nullptr, nullptr};
  unsigned n_blocks = 0;
  if (rows != 0) {
    if (mma) {
      const uint64_t target_items = static_cast<uint64_t>(ctx.sm_count) * 2 * 4;
      chunk = (total_keys * c.kv_heads + target_items - 1) / std::max<uint64_t>(target_items, 1);
      chunk = std::min<uint64_t>(std::max<uint64_t>((chunk + 63) / 64 * 64, 64), 1024);
      for (unsigned l = 0; l < lanes; ++l)
        if (pool->host_tokens[l]) n_work += ((static_cast<uint64_t>(pool->host_starts[l]) + pool->host_tokens[l] + chunk - 1) / chunk) * c.kv_heads;
      if (n_work > m->work_cap) return FJ_QUOTA_EXCEEDED;
    }
    fj::launch_build_attn_lists(ctx, pool->dev, pool->pack, lanes, c.kv_heads, static_cast<unsigned>(chunk), m->q, m->attn, c.q_heads, c.head_dim, 2, m->seqs, m->work,
                                m->n_work_dev, m->work_cap);
    if (mma) {
      const size_t groups = static_cast<size_t>(lanes) * c.kv_heads;
      const size_t counter_bytes = (groups * sizeof(unsigned) + 255) / 256 * 256;
      const size_t o_bytes = fj::attn_part_o_bytes(static_cast<unsigned>(n_work), c.head_dim), ml_bytes = fj::attn_part_ml_bytes(static_cast<unsigned>(n_work));
      if (!ensure_attn_scratch(be, counter_bytes + o_bytes + ml_bytes)) return FJ_ALLOCATION_FAILED;
      scratch.counters = static_cast<unsigned*>(be->attn_scratch);
      scratch.part_o = reinterpret_cast<float*>(static_cast<char*>(be->attn_scratch) + counter_bytes);
      scratch.part_ml = reinterpret_cast<float*>(static_cast<char*>(be->attn_scratch) + counter_bytes + o_bytes);
    }
    if (!mma && fj::attn_prefill_mma_supported(g)) {
      const unsigned per_block = fj::attn_prefill_tokens_per_block(g);
      std::vector<uint2> items;
      for (unsigned l = 0; l < lanes; ++l)
        for (unsigned t = 0; t < pool->host_tokens[l]; t += per_block) items.push_back(make_uint2(l, t));
      if (items.size() > m->prefill_items_cap) return FJ_QUOTA_EXCEEDED;
      n_blocks = static_cast<unsigned>(items.size());
      cudaMemcpyAsync(m->prefill_items, items.data(), items.size() * sizeof(uint2), cudaMemcpyHostToDevice, be->stream);  // pageable source: staged before the call returns
    }
    if (token_ids) cudaMemcpyAsync(m->tokens_in, token_ids, static_cast<size_t>(rows) * 4, cudaMemcpyHostToDevice, be->stream);
    else launch_feedback_tokens(ctx, pool->pack.cu_seqlens, m->tokens_out, m->tokens_in, lanes);
    fj::launch_quant_embed(ctx, m->embed.packed, m->embed.scales, m->embed.biases, dt, m->tokens_in, m->hidden, dt, c.vocab, H / 8, rows, 4, G, nullptr);
    fj::launch_rms_norm(ctx, dense_view(m->hidden, dt, rows, H, H), weight_view(m->layers[0].input_norm, dt, rows, H), dense_view(m->normed, dt, rows, H, H), rows, H, c.eps);
  }
  void* hidden = m->hidden;
  void* other = m->hidden2;
  const unsigned plane_slots = pool->dev.physical_pages * pool->dev.page_tokens;
  int32_t status = FJ_OK;
  for (uint32_t l = 0; l < c.layers && status == FJ_OK; ++l) {
    const auto& L = m->layers[l];
    auto mark = [&](int phase) {
      if (!m->phase_events.empty()) cudaEventRecord(m->phase_events[static_cast<size_t>(l) * 5 + phase], be->stream);
    };
    mark(0);
    if (rows != 0) {
      q4(m->normed, L.qkv, m->qkv, dt, rows, H, qd + 2 * kd, 4);
      fj::launch_qknorm_rope_append(ctx, m->qkv, dt, L.q_norm, L.k_norm, pool->pack.positions, pool->pack.slot_mapping, m->q, L.k_plane, L.v_plane, rows, c.q_heads, c.kv_heads,
                                    c.head_dim, c.eps, m->inv_freq, 1, plane_slots);
      if (mma) fj::launch_attn_decode_mma(ctx, g, m->seqs, m->work, static_cast<unsigned>(n_work), L.k_plane, L.v_plane, pool->dev.generations, scratch, nullptr);
      else if (n_blocks) fj::launch_attn_prefill_mma(ctx, g, m->seqs, m->prefill_items, n_blocks, L.k_plane, L.v_plane, pool->dev.generations, nullptr);
      else fj::launch_attn_generic(ctx, g, m->seqs, lanes, max_q_len, L.k_plane, L.v_plane, pool->dev.generations, nullptr);
      q4(m->attn, L.o, m->proj, dt, rows, qd, H, 4);
      fj::launch_residual_norm(ctx, dense_view(hidden, dt, rows, H, H), dense_view(m->proj, dt, rows, H, H), weight_view(L.post_norm, dt, rows, H), dense_view(other, dt, rows, H, H),
                               dense_view(m->normed, dt, rows, H, H), rows, H, c.eps, 0);
      std::swap(hidden, other);  // `hidden` is now the post-attention residual stream
      if (rows > 16 && m->router_split != nullptr) {
        const size_t words = static_cast<size_t>(c.experts) * (H * c.router_bits / 32);
        fj::launch_pdl(router_split_kernel, dim3(static_cast<unsigned>(std::min<size_t>((words + 255) / 256, 4096))), dim3(256), 0, be->stream, L.router.packed,
                       static_cast<const unsigned short*>(L.router.scales), static_cast<const unsigned short*>(L.router.biases), c.experts, H, c.router_bits, G,
                       m->router_split);
        ctx.launches++;
        fj::launch_gemm_nt(ctx, m->normed, dt, H, m->router_split, dt, H, m->router_halves, FJ_F32, 2 * c.experts, rows, 2 * c.experts, H, be->gemm_scratch,
                           be->gemm_scratch_bytes);
        fj::launch_pdl(router_sum_kernel, dim3(static_cast<unsigned>(std::min<size_t>((static_cast<size_t>(rows) * c.experts + 255) / 256, 2048))), dim3(256), 0, be->stream,
                       static_cast<const float*>(m->router_halves), m->router_logits, rows, c.experts);
        ctx.launches++;
      } else {
        q4(m->normed, L.router, m->router_logits, FJ_F32, rows, H, c.experts, c.router_bits);
      }
      fj::launch_top_k(ctx, m->router_logits, FJ_F32, m->route_weights, FJ_F32, m->route_experts, rows, c.experts, K, true);
      if (m->uniform_routing) {
        route_uniform_kernel<<<(rows + 255) / 256, 256, 0, be->stream>>>(m->route_experts, m->route_weights, rows, K, c.experts, l);
        ctx.launches++;
      }
      if (m->captured_experts) {
        const size_t at = static_cast<size_t>(l) * c.max_rows * K;
        cudaMemcpyAsync(m->captured_experts + at, m->route_experts, static_cast<size_t>(rows) * K * 4, cudaMemcpyDeviceToDevice, be->stream);
        cudaMemcpyAsync(m->captured_weights + at, m->route_weights, static_cast<size_t>(rows) * K * 4, cudaMemcpyDeviceToDevice, be->stream);
      }
    }
    // Few routes: one GEMV-style pass per route. More: bucket by expert; while the average expert has few rows the
    // 16-row tiles stream each active expert's nibbles (int8 tensor cores; measured faster up to 64 rows per expert),
    // beyond that 128-row tile GEMMs on tcgen05 (weights rounded to bf16) take over.
    const unsigned kGroupedRoutes = c.grouped_min_routes ? c.grouped_min_routes : 64;
    const unsigned kStreamRows = c.stream_rows_per_expert ? c.stream_rows_per_expert : 72;
    // `live`: how many of the n_routes ids are expected to be valid (a padded exchange carries whole slabs)
    auto bucketed_on = [&](fj::Ctx& ctx, void* plan, const void* x, unsigned src_div, const unsigned* ids, unsigned n_routes, unsigned live, unsigned n_experts, void* act, void* down_out,
                           bool down_bf16, const unsigned* slab_counts, unsigned slab_cap, unsigned slab_offset, unsigned slab_limit) -> bool {
      if (live < kGroupedRoutes || G != 64) return false;
      const bool stream = live < static_cast<uint64_t>(kStreamRows) * n_experts &&
                          fj::expert_stream_supported(H, I, 4, G, n_experts, x, L.gate.packed, L.gate.scales, L.gate.biases) &&
                          fj::expert_stream_supported(H, I, 4, G, n_experts, x, L.up.packed, L.up.scales, L.up.biases) &&
                          fj::expert_stream_supported(I, H, 4, G, n_experts, act, L.down.packed, L.down.scales, L.down.biases);
      if (stream) {
        fj::launch_route_plan(ctx, ids, n_routes, n_experts, plan, nullptr, 16, slab_counts, slab_cap, slab_offset, slab_limit);
        if (!fj::launch_expert_stream_pair(ctx, x, L.gate.packed, L.gate.scales, L.gate.biases, L.up.packed, L.up.scales, L.up.biases, plan, n_routes, n_experts, src_div, act, H,
                                           I, live) ||
            !fj::launch_expert_stream_single(ctx, act, L.down.packed, L.down.scales, L.down.biases, plan, n_routes, n_experts, 1, down_out, down_bf16, I, H, live))
          status = FJ_DEVICE_EXECUTION_FAILED;
        return true;
      }
      if (!fj::grouped_q4_supported(H, I, 4, G, n_experts, x, L.gate.packed) || !fj::grouped_q4_supported(I, H, 4, G, n_experts, act, L.down.packed)) return false;
      const unsigned tile_rows = fj::grouped_tile_rows(live, n_experts);
      fj::launch_route_plan(ctx, ids, n_routes, n_experts, plan, nullptr, tile_rows, slab_counts, slab_cap, slab_offset, slab_limit);
      fj::launch_grouped_q4_pair(ctx, x, L.gate.packed, L.gate.scales, L.gate.biases, L.up.packed, L.up.scales, L.up.biases, plan, n_routes, n_experts, src_div, act, H, I,
                                 tile_rows);
      fj::launch_grouped_q4_single(ctx, act, L.down.packed, L.down.scales, L.down.biases, plan, n_routes, n_experts, 1, down_out, down_bf16, I, H, tile_rows);
      return true;
    };
    auto bucketed = [&](const void* x, unsigned src_div, const unsigned* ids, unsigned n_routes, unsigned live, unsigned n_experts, void* act, void* down_out, bool down_bf16) -> bool {
      return bucketed_on(ctx, m->route_plan, x, src_div, ids, n_routes, live, n_experts, act, down_out, down_bf16, nullptr, 0, 0, 0);
    };
    mark(1);
    if (m->world == 1) {
      const unsigned routes = rows * K;
      mark(2);
      if (bucketed(m->normed, K, m->route_experts, routes, routes, c.experts, m->act, m->down_routes, false)) {
        mark(3);
        fj::launch_routes_combine(ctx, m->down_routes, FJ_F32, nullptr, m->route_experts, c.experts, m->route_weights, FJ_F32, hidden, dt, other, dt, rows, K, H);
      } else {
        fj::launch_gather_quant_matmul(ctx, m->normed, dt, L.gate.packed, L.gate.scales, L.gate.biases, dt, L.up.packed, L.up.scales, L.up.biases, m->route_experts, m->act, dt, rows, H,
                                       c.experts, I, K, 4, G, 1, nullptr);
        fj::launch_gather_quant_weighted_sum(ctx, m->act, dt, L.down.packed, L.down.scales, L.down.biases, dt, m->route_experts, m->route_weights, FJ_F32, hidden, dt, other, dt, rows, K,
                                             I, c.experts, H, 4, G, 2, nullptr);
      }
    } else if (m->ep_direct) {
      // Direct exchange: peer stores and flags instead of NCCL, no host round trip (kernels above). The layer's rows go in
      // `chunks` pieces, each on a stream of its own and one step behind the previous one: a chunk starts its dispatch when the
      // previous chunk's dispatch has left, and its experts when the previous chunk's experts are done, so transfers over
      // NVLink run under the other chunks' expert projections.
      const unsigned cap = m->capacity, W = m->world, rank = m->ep->rank, chunks = m->ep_chunks, cap_c = m->ep_chunk_capacity;
      const bool ret_bf16 = c.ep_return_bf16 != 0;
      const int ret_dt = ret_bf16 ? FJ_BF16 : FJ_F32;
      const unsigned exchange = ++m->ep_exchange;
      void** t = m->ep_tables;
      const EpPeers peers{reinterpret_cast<unsigned short* const*>(t), reinterpret_cast<unsigned* const*>(t + W), reinterpret_cast<unsigned long long* const*>(t + 2 * W),
                          reinterpret_cast<const unsigned char* const*>(t + 3 * W), reinterpret_cast<unsigned char* const*>(t + 4 * W)};
      unsigned* wait_err = m->ep_state;
      const bool push_back = m->ep_return_mode == 2;
      const unsigned sms = static_cast<unsigned>(ctx.sm_count > 0 ? ctx.sm_count : 148);
      const unsigned rows_c = (rows + chunks - 1) / chunks;
      if (chunks > 1) cudaEventRecord(m->ep_events[0], be->stream);
      for (unsigned ch = 0; ch < chunks; ++ch) {
        cudaStream_t st = ch == 0 ? be->stream : m->ep_streams[ch - 1];
        fj::Ctx cx = ctx;
        cx.stream = st;
        cx.launches = 0;
        const unsigned row0 = std::min(rows, ch * rows_c), row1 = std::min(rows, row0 + rows_c), n_rows = row1 - row0, routes = n_rows * K;
        const unsigned fbase = ch * 2 * W;
        unsigned *send_counts = m->ep_counts + fbase, *recv_counts = send_counts + W, *ticket = m->ep_state + 1 + ch, *ticket_back = m->ep_state + 1 + chunks + ch, *stale = m->ep_state + 1 + 2 * chunks + ch * W;
        if (ch > 0) {
          cudaStreamWaitEvent(st, m->ep_events[0], 0);                  // the routing of this layer
          cudaStreamWaitEvent(st, m->ep_events[1 + 3 * (ch - 1)], 0);  // the previous chunk's rows have left
        }
        ep_push_dispatch_kernel<<<std::max(1u, std::min((routes + 7) / 8, 4u * sms)), 256, 0, st>>>(static_cast<const unsigned short*>(m->normed), m->route_experts, row0 * K, row1 * K, K, H, cap,
                                                                                                  ch * cap_c, cap_c, rank, W, m->experts_local, peers, m->route_slot, send_counts, ticket,
                                                                                                  fbase, exchange);
        if (chunks > 1) cudaEventRecord(m->ep_events[1 + 3 * ch], st);
        ep_wait_kernel<<<1, 128, 0, st>>>(m->ep_flags + fbase, W, exchange, cap_c, recv_counts, stale, m->recv_experts + ch * cap_c, m->ep_live_dev + static_cast<size_t>(l) * chunks + ch,
                                          wait_err, m->ep_max_polls, nullptr, 0, cap);
        cx.launches += 2;
        if (ch == 0) mark(2);
        if (ch > 0) cudaStreamWaitEvent(st, m->ep_events[1 + 3 * (ch - 1) + 1], 0);  // the previous chunk's experts
        // how many rows arrive is known on the device only; the kernels are chosen from what this chunk received in the previous step
        const unsigned seen_before = m->ep_live_host[static_cast<size_t>(l) * chunks + ch];
        unsigned live = seen_before ? seen_before : std::max(routes, 1u);
        if (c.grouped_min_routes == 0) live = std::max(live, kGroupedRoutes);  // slabs are mostly empty: the bucketed kernels skip what the per-route ones would visit
        if (!bucketed_on(cx, m->ep_plans[ch], m->recv_rows, 1, m->recv_experts, W * cap, live, m->experts_local, m->act_ep, m->down_ep, ret_bf16, recv_counts, cap, ch * cap_c, cap_c)) {
          // per-route kernels over this chunk's share of every slab (ids past the live count are invalid and skipped); only models built for tiny steps get here
          for (unsigned src = 0; src < W; ++src) {
            const size_t off = static_cast<size_t>(src) * cap + static_cast<size_t>(ch) * cap_c;
            const unsigned short* x = m->recv_rows + off * H;
            unsigned short* act = m->act_ep + off * I;
            void* down = reinterpret_cast<unsigned char*>(m->down_ep) + off * H * (ret_bf16 ? 2 : 4);
            fj::launch_gather_quant_matmul(cx, x, dt, L.gate.packed, L.gate.scales, L.gate.biases, dt, L.up.packed, L.up.scales, L.up.biases, m->recv_experts + off, act, dt, cap_c, H,
                                           m->experts_local, I, 1, 4, G, 1, nullptr);
            fj::launch_gather_quant_matmul(cx, act, dt, L.down.packed, L.down.scales, L.down.biases, dt, nullptr, nullptr, nullptr, m->recv_experts + off, down, ret_dt, cap_c, I,
                                           m->experts_local, H, 1, 4, G, 0, nullptr);
          }
        }
        if (chunks > 1) cudaEventRecord(m->ep_events[1 + 3 * ch + 1], st);
        if (ch == 0) mark(3);
        const size_t at = static_cast<size_t>(row0) * H * 2;  // activations are bf16
        if (push_back) {
          // the owner writes every result row into its origin's memory, then the origin combines from there
          ep_push_return_kernel<<<8 * sms, 256, 0, st>>>(reinterpret_cast<const unsigned char*>(m->down_ep), static_cast<unsigned>(H * (ret_bf16 ? 2 : 4)), cap, ch * cap_c, cap_c, rank, W,
                                                        recv_counts, peers, ticket_back, fbase + W, exchange);
          ep_wait_kernel<<<1, 128, 0, st>>>(m->ep_flags + fbase + W, W, exchange, cap_c, nullptr, nullptr, nullptr, nullptr, wait_err, m->ep_max_polls);
          cx.launches += 2;
          if (n_rows)
            fj::launch_routes_combine(cx, m->returned, ret_dt, m->route_slot + static_cast<size_t>(row0) * K, nullptr, 0, m->route_weights + static_cast<size_t>(row0) * K, FJ_F32,
                                      static_cast<const unsigned char*>(hidden) + at, dt, static_cast<unsigned char*>(other) + at, dt, n_rows, K, H);
          if (ch > 0) cudaEventRecord(m->ep_events[1 + 3 * ch + 2], st);
          ctx.launches += cx.launches;
          continue;
        }
        // "my results of this chunk are ready" to every peer, then wait for theirs; the combine reads the rows where they are
        ep_wait_kernel<<<1, 128, 0, st>>>(m->ep_flags + fbase + W, W, exchange, cap_c, nullptr, nullptr, nullptr, nullptr, wait_err, m->ep_max_polls, peers.flags, fbase + W + rank);
        cx.launches++;
        if (n_rows) {
          const unsigned grid = std::min(n_rows, 16u * sms);
          const unsigned char* res = static_cast<const unsigned char*>(hidden) + at;
          unsigned char* out = static_cast<unsigned char*>(other) + at;
          if (ret_bf16)
            ep_pull_combine_kernel<true><<<grid, 256, 0, st>>>(peers.results, m->route_slot + static_cast<size_t>(row0) * K, m->route_weights + static_cast<size_t>(row0) * K, res, dt, out, dt,
                                                               n_rows, K, H, cap, rank);
          else
            ep_pull_combine_kernel<false><<<grid, 256, 0, st>>>(peers.results, m->route_slot + static_cast<size_t>(row0) * K, m->route_weights + static_cast<size_t>(row0) * K, res, dt, out, dt,
                                                                n_rows, K, H, cap, rank);
          cx.launches++;
        }
        if (ch > 0) cudaEventRecord(m->ep_events[1 + 3 * ch + 2], st);
        ctx.launches += cx.launches;
      }
      for (unsigned ch = 1; ch < chunks; ++ch) cudaStreamWaitEvent(be->stream, m->ep_events[1 + 3 * ch + 2], 0);
      if (status != FJ_OK) break;
    } else {
      const unsigned cap = m->capacity, routes = rows * K, W = m->world;
      // rows come back from the experts' owners as f32 (bit-identical to one GPU) or, on request, rounded to bf16 (half the bytes)
      const bool ret_bf16 = c.ep_return_bf16 != 0;
      const int ret_dt = ret_bf16 ? FJ_BF16 : FJ_F32;
      // Small steps (decode): whole slabs of `cap` slots travel, padded with an out-of-range expert id, and
      // nothing has to come back to the host. Large steps: the row counts are exchanged and read back first
      // so that only live rows travel. The choice depends on the model's capacity only, so all ranks agree.
      const bool padded = cap <= 1024;
      cudaMemsetAsync(m->ep_counts, 0, 2 * W * 4, be->stream);
      if (padded) cudaMemsetAsync(m->send_experts, 0xFF, static_cast<size_t>(W) * cap * 4, be->stream);
      if (routes) {
        ep_plan_kernel<<<std::min((routes + 255) / 256, 256u), 256, 0, be->stream>>>(m->route_experts, routes, m->experts_local, W, cap, m->send_experts, m->route_slot, m->ep_counts);
        ep_scatter_rows_kernel<<<std::min(routes, 4096u), 128, 0, be->stream>>>(static_cast<const unsigned short*>(m->normed), m->route_slot, routes, K, H, m->send_rows);
        ctx.launches += 2;
      }
      std::vector<unsigned> slab_at(W), packed_at(W), slab_counts(W, cap);
      const unsigned *send_counts = slab_counts.data(), *recv_counts = slab_counts.data();
      unsigned received = 0;
      if (padded) {
        for (unsigned p = 0; p < W; ++p) { slab_at[p] = p * cap; packed_at[p] = p * cap; }
        received = W * cap;
      } else {
        // how many rows every peer will send here: one 4-byte exchange, then both count vectors go to the host
        status = ep_all_to_all(m->ep, m->ep_counts, m->ep_counts + W, 4);
        if (status != FJ_OK) break;
        cudaMemcpyAsync(m->ep_counts_host, m->ep_counts, 2 * W * 4, cudaMemcpyDeviceToHost, be->stream);
        status = ep_wait_stream(m->ep);  // bounded: a rank that never joins must not hang the others' hosts
        if (status != FJ_OK) break;
        send_counts = m->ep_counts_host;
        recv_counts = m->ep_counts_host + W;
        for (unsigned p = 0; p < W; ++p) { slab_at[p] = p * cap; packed_at[p] = received; received += recv_counts[p]; }
        if (received > W * cap) { status = FJ_EXECUTION_FAILED; break; }
      }
      status = ep_all_to_all_rows(m->ep, m->send_rows, slab_at.data(), send_counts, m->recv_rows, packed_at.data(), recv_counts, static_cast<size_t>(H) * 2, m->send_experts,
                                  m->recv_experts, 4);
      if (status != FJ_OK) break;
      mark(2);
      if (received) {
        // rows received for this rank's experts, densely packed by source: one route each
        if (!bucketed(m->recv_rows, 1, m->recv_experts, received, padded ? cap : received, m->experts_local, m->act_ep, m->down_ep, ret_bf16)) {
          fj::launch_gather_quant_matmul(ctx, m->recv_rows, dt, L.gate.packed, L.gate.scales, L.gate.biases, dt, L.up.packed, L.up.scales, L.up.biases, m->recv_experts, m->act_ep, dt,
                                         received, H, m->experts_local, I, 1, 4, G, 1, nullptr);
          fj::launch_gather_quant_matmul(ctx, m->act_ep, dt, L.down.packed, L.down.scales, L.down.biases, dt, nullptr, nullptr, nullptr, m->recv_experts, m->down_ep, ret_dt, received, I,
                                         m->experts_local, H, 1, 4, G, 0, nullptr);
        }
      }
      if (status != FJ_OK) break;
      mark(3);
      status = ep_all_to_all_rows(m->ep, m->down_ep, packed_at.data(), recv_counts, m->returned, slab_at.data(), send_counts, static_cast<size_t>(H) * (ret_bf16 ? 2 : 4));
      if (status != FJ_OK) break;
      if (rows) {
        fj::launch_routes_combine(ctx, m->returned, ret_dt, m->route_slot, nullptr, 0, m->route_weights, FJ_F32, hidden, dt, other, dt, rows, K, H);
      }
    }
    mark(4);
    std::swap(hidden, other);
    if (rows != 0) {
      const void* next_norm = l + 1 < c.layers ? m->layers[l + 1].input_norm : m->final_norm;
      fj::launch_rms_norm(ctx, dense_view(hidden, dt, rows, H, H), weight_view(next_norm, dt, rows, H), dense_view(m->normed, dt, rows, H, H), rows, H, c.eps);
    }
  }
  if (status != FJ_OK) { cudaStreamSynchronize(be->stream); return status; }
  if (rows != 0) {
    // the final norm ran on every row; the greedy token comes from each lane's last row
    launch_gather_last_rows(ctx, m->normed, dt, pool->pack.cu_seqlens, m->last_normed, lanes, H);
    void* logits = m->logits;
    if (logits_out) {
      fj_buffer_rec* r = find_buffer(be, logits_out);
      if (!r || r->readonly || r->bytes < static_cast<uint64_t>(lanes) * c.vocab * 2) return FJ_INVALID_INPUT;
      logits = r->ptr;
    }
    q4(m->last_normed, m->lm_head, logits, dt, lanes, H, c.vocab, 4);
    fj::launch_argmax(ctx, logits, dt, c.vocab, m->tokens_out, lanes, c.vocab, m->argmax_scratch);
  }
  m->last_kernels = ctx.launches - launches_before;
  m->last_work_items = n_work;
  if (cudaGetLastError() != cudaSuccess) return FJ_DEVICE_EXECUTION_FAILED;
  if (m->ep_direct) cudaMemcpyAsync(m->ep_live_host + static_cast<size_t>(c.layers) * m->ep_chunks, m->ep_state, 4, cudaMemcpyDeviceToHost, be->stream);
  if (out_tokens && rows != 0) {
    cudaMemcpyAsync(out_tokens, m->tokens_out, static_cast<size_t>(lanes) * 4, cudaMemcpyDeviceToHost, be->stream);
    if (m->ep) {
      const int32_t waited = ep_wait_stream(m->ep);  // the step's exchanges are still in flight: wait for them with the group's deadline
      if (waited == FJ_OK && m->ep_direct && m->ep_live_host[static_cast<size_t>(c.layers) * m->ep_chunks] != 0) return FJ_TIMEOUT;  // a device-side wait of the direct exchange ran out
      return waited;
    }
    return cuda_status(cudaStreamSynchronize(be->stream));
  }
  return FJ_OK;
}
