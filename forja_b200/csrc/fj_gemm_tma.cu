// Dense 16-bit GEMM on the 5th-generation tensor cores, fed by the tensor memory accelerator:
// C[M,N] = A[M,K] * W[N,K]^T ("NT", both operands K-major), f32 accumulation in tensor memory, one rounding on
// store (reference operator: Op::Matmul, crates/forja-cpu/src/lib.rs:815-848; here: prefill and decode projections,
// the lm_head, the expanded-slab path of Op::QuantMatmul).
//
// One CTA owns a 128 x BN output tile (BN 32 ... 256) and is split into three roles that never meet at a CTA barrier
// inside the main loop:
//   warp 0, one thread   producer: per 64-wide k step one cp.async.bulk.tensor.2d (TMA) for the A tile (128 rows x 128
//                        bytes) and one for the W tile (BN rows x 128 bytes) into the next free stage; the tensor maps
//                        carry the 128-byte swizzle, so the tiles land in the K-major layout the tensor core reads,
//                        rows past M or N are filled with zeros by the hardware, and the bytes are counted on the
//                        stage's "full" mbarrier (expect_tx).
//   warp 1, one thread   issues four tcgen05.mma.cta_group::1.kind::f16 (M 128, N BN, K 16) per stage into a
//                        128-lane x BN-column f32 accumulator in TMEM; tcgen05.commit arrives on the stage's "empty"
//                        mbarrier when the tensor core has read the stage, and on "done" after the last step.
//   warps 2-5            epilogue: wait for "done", read their 32 TMEM lanes (= rows) with tcgen05.ld, 32 columns at a
//                        time, round and store rows of 64 bytes.
// Stages: as many as fit in 200 KB (4 at BN 256 ... 8 at BN 32/64), so a CTA alone keeps 100-190 KB of loads in flight -
// what a decode-sized grid (one CTA per SM or fewer) needs to pull its weight stream at HBM speed.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the role gives up, the give-up is counted in a device
// counter, the tile is left unwritten, tensor memory is freed and the kernel returns.
//
// The tensor maps cover memory of this GPU only and every load is a plain (non-multicast) one-CTA load.
#include "fj_kernels.h"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace fj {

namespace {

constexpr int TM_BM = 128, TM_BK = 64, TM_THREADS = 192;
constexpr int TM_A_BYTES = TM_BM * 128;  // 128 rows x 128 bytes
constexpr unsigned kSpinLimit = 1u << 24;

template <int BN> constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);
template <int BN> constexpr int kStageBytes = TM_A_BYTES + BN * 128;
template <int BN> constexpr int kSmemBytes = kStages<BN> * kStageBytes<BN> + 1024;  // + slack to align the base to 1024 bytes

__device__ unsigned g_tma_giveups = 0;

__device__ inline void mbar_init(unsigned addr, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count) : "memory"); }
__device__ inline void mbar_expect_tx(unsigned addr, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(addr), "r"(bytes) : "memory");
}
// Polls until the phase with the given parity has completed; false when the limit ran out.
__device__ inline bool mbar_wait(unsigned addr, unsigned parity) {
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// One tile of a 2-d tensor map into shared memory; x = element coordinate along K (a multiple of 64, so x * 2 bytes is
// 16-byte aligned), y = row. Completion is counted in bytes on `mbar`.
__device__ inline void tma_load_2d(unsigned smem_dst, const CUtensorMap* map, int x, int y, unsigned mbar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_dst),
               "l"(reinterpret_cast<unsigned long long>(map)), "r"(mbar), "r"(x), "r"(y)
               : "memory");
}
// K-major operand tile in the 128-byte swizzle: start address, 8-row group stride 1024 bytes, descriptor version 1,
// layout type 2 (SWIZZLE_128B).
__device__ inline unsigned long long smem_desc(unsigned smem_addr) {
  unsigned long long d = 0;
  d |= static_cast<unsigned long long>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<unsigned long long>(1) << 16;
  d |= static_cast<unsigned long long>(1024 >> 4) << 32;
  d |= static_cast<unsigned long long>(1) << 46;
  d |= static_cast<unsigned long long>(2) << 61;
  return d;
}
// kind::f16 instruction descriptor: D f32, A and B of the given 16-bit format, both K-major, N = bn, M = 128.
__device__ inline unsigned instr_desc(bool bf16, unsigned bn) {
  const unsigned fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((bn >> 3) << 17) | (static_cast<unsigned>(TM_BM >> 4) << 24);
}

struct TmaGemmParams {
  void* c; int c_dt; size_t ldc;
  unsigned m, n, k;
  int bf16;
  unsigned splits, k_per_split;  // the CTAs of a cluster (blockIdx.z = rank in the cluster) share a tile along K; k_per_split is a multiple of 64
};

// 32 consecutive accumulator columns of this thread's TMEM lane, as f32 bit patterns.
__device__ inline void tmem_load_32(unsigned taddr, unsigned (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
        "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
// All threads of all CTAs of the cluster meet; writes to shared memory before it are visible to cluster-wide reads after it.
__device__ inline void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// 32 consecutive columns of one output row, from their f32 bit patterns: rounded once, 64-byte rows when aligned.
__device__ inline void store_row_chunk(const TmaGemmParams& p, unsigned row, unsigned c_first, const unsigned (&v)[32]) {
  const size_t base = static_cast<size_t>(row) * p.ldc + c_first;
  if (p.c_dt != F32 && c_first + 32 <= p.n && base % 8 == 0 && reinterpret_cast<size_t>(p.c) % 16 == 0) {
    unsigned short* dst = static_cast<unsigned short*>(p.c) + base;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      unsigned packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(v[q * 8 + 2 * j]), hi = __uint_as_float(v[q * 8 + 2 * j + 1]);
        if (p.c_dt == BF16) {
          __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
          packed[j] = *reinterpret_cast<unsigned*>(&t);
        } else {
          __half2 t = __floats2half2_rn(lo, hi);
          packed[j] = *reinterpret_cast<unsigned*>(&t);
        }
      }
      *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (c_first + j < p.n) store_from_f32(p.c, p.c_dt, base + j, __uint_as_float(v[j]));
  }
}

template <int BN>
__global__ void __launch_bounds__(TM_THREADS, 1) gemm_nt_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, TmaGemmParams p) {
  constexpr int STAGES = kStages<BN>;
  constexpr int STAGE_BYTES = kStageBytes<BN>;
  constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ unsigned char tma_smem_raw[];
  __shared__ __align__(8) unsigned long long s_full[STAGES], s_empty[STAGES], s_done;
  __shared__ unsigned s_tmem;
  __shared__ int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned row0 = blockIdx.y * TM_BM, col0 = blockIdx.x * BN;
  const unsigned k_begin = blockIdx.z * p.k_per_split;
  const unsigned k_iters = (min(p.k, k_begin + p.k_per_split) - k_begin) / TM_BK;
  const unsigned raw = static_cast<unsigned>(__cvta_generic_to_shared(tma_smem_raw));
  const unsigned smem_base = (raw + 1023u) & ~1023u;
  const unsigned full_base = static_cast<unsigned>(__cvta_generic_to_shared(&s_full[0]));
  const unsigned empty_base = static_cast<unsigned>(__cvta_generic_to_shared(&s_empty[0]));
  const unsigned done_bar = static_cast<unsigned>(__cvta_generic_to_shared(&s_done));

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(full_base + 8 * i, 1); mbar_init(empty_base + 8 * i, 1); }
    mbar_init(done_bar, 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(&s_tmem));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem = s_tmem;
  pdl_sync();  // barriers and tensor memory are set up while the previous kernel drains; its results are read from here on

  if (warp == 0) {
    if (lane == 0) {
      for (unsigned it = 0; it < k_iters; ++it) {
        const unsigned stage = it % STAGES;
        if (it >= STAGES && !mbar_wait(empty_base + 8 * stage, ((it / STAGES) - 1) & 1u)) { s_failed = 1; break; }
        const unsigned dst = smem_base + stage * STAGE_BYTES;
        mbar_expect_tx(full_base + 8 * stage, STAGE_BYTES);
        tma_load_2d(dst, &map_a, static_cast<int>(k_begin + it * TM_BK), static_cast<int>(row0), full_base + 8 * stage);
        tma_load_2d(dst + TM_A_BYTES, &map_w, static_cast<int>(k_begin + it * TM_BK), static_cast<int>(col0), full_base + 8 * stage);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc = instr_desc(p.bf16 != 0, BN);
      for (unsigned it = 0; it < k_iters; ++it) {
        const unsigned stage = it % STAGES;
        if (!mbar_wait(full_base + 8 * stage, (it / STAGES) & 1u)) { s_failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned at = smem_base + stage * STAGE_BYTES;
        const unsigned long long a_desc = smem_desc(at), b_desc = smem_desc(at + TM_A_BYTES);
#pragma unroll
        for (int ks = 0; ks < TM_BK / 16; ++ks) {
          // 16 k = 32 bytes further along the swizzled row: +2 in the descriptor's 16-byte address units
          const unsigned accumulate = (it != 0 || ks != 0) ? 1u : 0u;
          asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem), "l"(a_desc + 2ull * ks),
                       "l"(b_desc + 2ull * ks), "r"(idesc), "r"(accumulate)
                       : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(empty_base + 8 * stage) : "memory");
        if (it + 1 == k_iters) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(done_bar) : "memory");
      }
    }
  } else {
    // epilogue warps 2..5; a warp reads the TMEM lanes 32 * (warp % 4) .. + 31
    const unsigned quarter = static_cast<unsigned>(warp) & 3u;
    const bool ready = mbar_wait(done_bar, 0);
    if (!ready) s_failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned row = row0 + quarter * 32 + lane;
    const unsigned tile_row = quarter * 32 + lane;
    // Split K inside a cluster: ranks above 0 park their f32 partial tile in their own shared memory (the pipeline stages
    // are free by now; 16-byte pieces of a row are XOR-ed with the row number so that a warp's stores spread over the banks),
    // rank 0 adds them in rank order to its own accumulator through distributed shared memory and writes the tile.
    if (ready && blockIdx.z != 0) {
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the stages were last touched through the async proxy (TMA writes, tensor-core reads)
#pragma unroll 1
      for (int cb = 0; cb < (BN + 31) / 32; ++cb) {
        unsigned v[32];
        tmem_load_32(tmem + ((quarter * 32u) << 16) + cb * 32, v);
        const unsigned row_base = smem_base + tile_row * (BN * 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const unsigned piece = static_cast<unsigned>(cb * 8 + j) ^ (tile_row & 7u);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(row_base + piece * 16), "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3]) : "memory");
        }
      }
    }
    if (p.splits > 1) cluster_sync();  // partials are in place
    if (ready && blockIdx.z == 0) {
#pragma unroll 1
      for (int cb = 0; cb < (BN + 31) / 32; ++cb) {
        unsigned v[32];
        tmem_load_32(tmem + ((quarter * 32u) << 16) + cb * 32, v);
        for (unsigned rank = 1; rank < p.splits; ++rank) {
          const unsigned local = smem_base + tile_row * (BN * 4);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const unsigned piece = static_cast<unsigned>(cb * 8 + j) ^ (tile_row & 7u);
            unsigned remote, t0, t1, t2, t3;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local + piece * 16), "r"(rank));
            asm volatile("ld.shared::cluster.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(t0), "=r"(t1), "=r"(t2), "=r"(t3) : "r"(remote) : "memory");
            v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + __uint_as_float(t0));
            v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + __uint_as_float(t1));
            v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + __uint_as_float(t2));
            v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + __uint_as_float(t3));
          }
        }
        if (row < p.m) store_row_chunk(p, row, col0 + cb * 32, v);
      }
    }
  }
  // every thread of every CTA of the cluster: nobody leaves (and frees its shared memory) while rank 0 may still read it
  if (p.splits > 1) {
    if (warp < 2) cluster_sync();  // the two main-loop warps take part in the first meeting as well
    cluster_sync();
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) atomicAdd(&g_tma_giveups, 1u);
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ---- tensor maps -----------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_entry() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &entry, 12000, cudaEnableDefault, &result) != cudaSuccess || result != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(entry);
  }();
  return fn;
}

struct MapKey {
  const void* base; unsigned rows, k, box_rows; size_t ld; int bf16;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && k == o.k && box_rows == o.box_rows && ld == o.ld && bf16 == o.bf16; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& key) const {
    size_t h = reinterpret_cast<size_t>(key.base) * 0x9E3779B97F4A7C15ull;
    h ^= (static_cast<size_t>(key.rows) << 32 | key.k) * 0xC2B2AE3D27D4EB4Full;
    h ^= (key.ld * 31 + key.box_rows * 7 + static_cast<size_t>(key.bf16)) * 0x165667B19E3779F9ull;
    return h;
  }
};

// A [rows, k] row-major matrix of 16-bit elements with row stride `ld` as a 2-d tensor map with boxes of 64 elements
// (128 bytes, swizzled) x box_rows rows. Maps are cached: the step's operands are the same few buffers launch after launch.
bool tensor_map_2d(const void* base, unsigned rows, unsigned k, size_t ld, unsigned box_rows, bool bf16, CUtensorMap* out) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, k, box_rows, ld, bf16 ? 1 : 0};
  std::lock_guard<std::mutex> lock(mutex);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn encode = encode_tiled_entry();
  if (!encode) return false;
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {TM_BK, box_rows};
  const cuuint32_t element_strides[2] = {1, 1};
  CUtensorMap map;
  const CUresult status = encode(&map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, map);
  *out = map;
  return true;
}

template <int BN>
bool run_tma(Ctx& ctx, const CUtensorMap& map_a, const CUtensorMap& map_w, const TmaGemmParams& p) {
  static SmemOptIn opted;
  if (!opt_in_smem(opted, gemm_nt_tma_kernel<BN>, kSmemBytes<BN>)) { cudaGetLastError(); return false; }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((p.n + BN - 1) / BN, (p.m + TM_BM - 1) / TM_BM, p.splits);
  config.blockDim = dim3(TM_THREADS);
  config.dynamicSmemBytes = kSmemBytes<BN>;
  config.stream = ctx.stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = 1;
  if (p.splits > 1) {  // the CTAs that share a tile along K form a cluster
    attributes[1].id = cudaLaunchAttributeClusterDimension;
    attributes[1].val.clusterDim.x = 1;
    attributes[1].val.clusterDim.y = 1;
    attributes[1].val.clusterDim.z = p.splits;
    config.numAttrs = 2;
  }
  if (cudaLaunchKernelEx(&config, gemm_nt_tma_kernel<BN>, map_a, map_w, p) != cudaSuccess) return false;  // the error stays pending for the submission
  ctx.launches++;
  return true;
}

}  // namespace

bool gemm_nt_tma_supported(int a_dt, int w_dt, unsigned m, unsigned n, unsigned k, size_t lda, size_t ldw, const void* a, const void* w) {
  return (a_dt == BF16 || a_dt == F16) && a_dt == w_dt && m >= 1 && n >= 16 && k >= TM_BK && k % TM_BK == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
         (reinterpret_cast<size_t>(a) | reinterpret_cast<size_t>(w)) % 16 == 0 && encode_tiled_entry() != nullptr;
}

// Tile width and K split. Width: the widest tile that still gives every SM a CTA; grids that cannot fill the GPU take 64
// columns, the narrowest outputs 32. Such grids with 2048 k or more are also split along K, 2 or 4 ways, while the grid stays
// within one wave and every split keeps at least eight k steps: the CTAs of a split form a thread-block cluster and meet
// through distributed shared memory (no partials in global memory, no atomics). What the split buys is less operand traffic
// per SM: every CTA of an unsplit 128-row tile pulls the whole 128 x K activation block through its SM's L2 port. Measured on
// the 128-row decode projections: 2048 x 1024 in 9.2 us instead of 11.5, 3072 x 1024 in 10.7 instead of 15.8; 1024 x 4096 is
// faster unsplit (7.9 against 9.2 us).
void gemm_nt_tma_plan(unsigned m, unsigned n, unsigned k, int sm_count, unsigned* tile_n, unsigned* splits, unsigned* k_per_split) {
  const unsigned row_blocks = (m + TM_BM - 1) / TM_BM;
  const unsigned sms = static_cast<unsigned>(sm_count > 0 ? sm_count : 148);
  unsigned bn = row_blocks * ((n + 63) / 64) >= sms / 4 ? 64 : 32;
  for (unsigned candidate : {256u, 128u, 64u}) {
    if (row_blocks * ((n + candidate - 1) / candidate) >= sms) { bn = candidate; break; }
  }
  const unsigned tiles = row_blocks * ((n + bn - 1) / bn), k_iters = k / TM_BK;
  unsigned parts = 1;
  if (k_iters >= 32) {  // a cluster launch costs about 1.5 us more than a plain one: below 2048 k the shorter main loop does not pay for it
    while (parts < 4 && tiles * parts * 2 <= sms && k_iters / (parts * 2) >= 8) parts *= 2;
  }
  const unsigned iters_per = (k_iters + parts - 1) / parts;
  *tile_n = bn;
  *k_per_split = iters_per * TM_BK;
  *splits = (k_iters + iters_per - 1) / iters_per;
}

bool launch_gemm_nt_tma(Ctx& ctx, const void* a, int a_dt, size_t lda, const void* w, size_t ldw, void* c, int c_dt, size_t ldc, unsigned m, unsigned n, unsigned k) {
  unsigned bn = 64, splits = 1, k_per_split = k;
  gemm_nt_tma_plan(m, n, k, ctx.sm_count, &bn, &splits, &k_per_split);
  CUtensorMap map_a, map_w;
  if (!tensor_map_2d(a, m, k, lda, TM_BM, a_dt == BF16, &map_a) || !tensor_map_2d(w, n, k, ldw, bn, a_dt == BF16, &map_w)) return false;
  TmaGemmParams p{c, c_dt, ldc, m, n, k, a_dt == BF16 ? 1 : 0, splits, k_per_split};
  switch (bn) {
    case 256: return run_tma<256>(ctx, map_a, map_w, p);
    case 128: return run_tma<128>(ctx, map_a, map_w, p);
    case 64: return run_tma<64>(ctx, map_a, map_w, p);
    default: return run_tma<32>(ctx, map_a, map_w, p);
  }
}

unsigned gemm_tma_giveups() {
  unsigned value = 0;
  cudaMemcpyFromSymbol(&value, g_tma_giveups, sizeof(value));
  return value;
}

}  // namespace fj
