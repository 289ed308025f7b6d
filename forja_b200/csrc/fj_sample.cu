// Op::Sample / Op::SampleMasked: temperature, top-k and top-p truncation followed by counter-based
// Gumbel-max selection (reference: crates/forja-cpu/src/lib.rs:1553-1575 parameter words,
// :1597-1638 sample_allowed, :1640-1653 allow-mask validation, :1655-1680 truncate_top_p,
// :1682-1700 splitmix64 / sampled_score).
//
// One CTA per row. The reference sorts the allowed indices by (value descending under IEEE total
// order, then index descending), keeps the first top_k, cuts that list where the running sum of
// exp((v - v_max) / T) / total reaches top_p, and takes the arg-max of v / T - ln(-ln(u)) over what
// is left (ties: highest index). Here the order is never materialised for the whole row:
//  * 64-bit keys (order key of the value, index) are unique, so "the first n of the sorted list"
//    is "every key >= the key of rank n"; that key comes from an 8-pass radix select;
//  * the two sums of truncate_top_p are sequential f32 sums in sorted order, which are reproduced
//    exactly by sorting only the prefix whose weights are >= 2^-26: every later term is smaller
//    than half an ulp of both running sums (total >= 1 and cumulative >= 1 / total) and leaves them
//    unchanged. The prefix is sorted in shared memory, 4096 keys at a time, and one thread adds it
//    up in order. A NaN or an infinite maximum makes the reference's total non-finite, which keeps
//    one candidate; that case is detected up front;
//  * the final arg-max runs over every allowed element whose key is >= the cut key.
// Differences to the CPU reference can only come from expf/logf (device results may differ from the
// host library in the last place) and only flip a choice at an exact near-tie.
#include "fj_kernels.h"

namespace fj {

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr unsigned SAMPLE_CHUNK = 4096;

struct SampleArgs {
  const void* x;
  int x_dt;
  size_t row_stride;
  const unsigned* params;  // temperature bits, top_k, top_p bits, seed lo, seed hi
  const unsigned* allow;   // bit i of word i / 32 set = index i permitted; nullptr = all
  unsigned* out;
  unsigned width, position;
  ErrorRecord* err;
};

struct SampleShared {
  unsigned long long reduce_key[32];
  unsigned reduce_count[32];
  unsigned hist[256];
  unsigned long long prefix;
  unsigned rank;
  unsigned gathered;
  unsigned long long keep_key;
  float total;
  float cumulative;
  int found;
  int flag;
};

__device__ inline unsigned long long splitmix64(unsigned long long value) {
  value += 0x9e3779b97f4a7c15ULL;
  value = (value ^ (value >> 30)) * 0xbf58476d1ce4e5b9ULL;
  value = (value ^ (value >> 27)) * 0x94d049bb133111ebULL;
  return value ^ (value >> 31);
}

// Bits of the sampled score; non-finite logits keep their own bits (no temperature, no noise).
__device__ inline unsigned sampled_score_bits(unsigned logit_bits, float temperature, unsigned long long seed, unsigned position, unsigned index) {
  if ((logit_bits & 0x7F800000u) == 0x7F800000u) return logit_bits;
  const unsigned long long counter = seed ^ (static_cast<unsigned long long>(position) << 32) ^ static_cast<unsigned long long>(index);
  const unsigned mantissa = static_cast<unsigned>(splitmix64(counter) >> 40);
  const float uniform = __fmul_rn(__fadd_rn(static_cast<float>(mantissa), 0.5f), 1.0f / 16777216.0f);
  return __float_as_uint(__fsub_rn(__fdiv_rn(__uint_as_float(logit_bits), temperature), logf(-logf(uniform))));
}

__device__ inline bool sample_allowed(const SampleArgs& a, unsigned i) { return a.allow == nullptr || ((a.allow[i >> 5] >> (i & 31)) & 1u) != 0; }

__device__ inline unsigned long long sample_key(const SampleArgs& a, size_t row_offset, unsigned i) {
  return (static_cast<unsigned long long>(total_order_key_bits(load_f32_bits(a.x, a.x_dt, row_offset + i))) << 32) | i;
}

__device__ inline unsigned long long block_max_u64(unsigned long long v, SampleShared& s) {
  v = warp_max_u64(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.reduce_key[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long r = s.reduce_key[0];
  for (int w = 1; w < SAMPLE_THREADS / 32; ++w) r = r > s.reduce_key[w] ? r : s.reduce_key[w];
  return r;
}
__device__ inline unsigned block_sum_u32(unsigned v, SampleShared& s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.reduce_count[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned r = 0;
  for (int w = 0; w < SAMPLE_THREADS / 32; ++w) r += s.reduce_count[w];
  return r;
}

// Key of rank `rank` (1-based, descending) among the allowed elements of the row; rank <= number allowed.
__device__ unsigned long long select_rank(const SampleArgs& a, size_t row_offset, unsigned rank, SampleShared& s) {
  __syncthreads();
  if (threadIdx.x == 0) { s.prefix = 0; s.rank = rank; }
  for (int shift = 56; shift >= 0; shift -= 8) {
    for (unsigned b = threadIdx.x; b < 256; b += SAMPLE_THREADS) s.hist[b] = 0;
    __syncthreads();
    const unsigned long long prefix = s.prefix;
    // eight rounds at a time: the loads of a batch are independent of each other, so they are in flight together
    constexpr int kBatch = 8;
    for (unsigned base = threadIdx.x; base < a.width; base += SAMPLE_THREADS * kBatch) {
      unsigned long long keys[kBatch];
      bool live[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const unsigned i = base + u * SAMPLE_THREADS;
        live[u] = i < a.width && sample_allowed(a, i);
        keys[u] = live[u] ? sample_key(a, row_offset, i) : 0ULL;
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (live[u] && (shift == 56 || (keys[u] >> (shift + 8)) == (prefix >> (shift + 8)))) atomicAdd(&s.hist[(keys[u] >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned above = 0, want = s.rank;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (above + s.hist[bin] >= want) break;
        above += s.hist[bin];
      }
      s.prefix = prefix | (static_cast<unsigned long long>(bin) << shift);
      s.rank = want - above;
    }
    __syncthreads();
  }
  return s.prefix;
}

// Descending bitonic sort of n (a power of two) keys in shared memory.
__device__ void sort_desc(unsigned long long* keys, unsigned n) {
  for (unsigned size = 2; size <= n; size <<= 1) {
    for (unsigned stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (unsigned t = threadIdx.x; t < n / 2; t += SAMPLE_THREADS) {
        const unsigned lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
        const bool descending = (lo & size) == 0;
        const unsigned long long x = keys[lo], y = keys[hi];
        if ((x < y) == descending) { keys[lo] = y; keys[hi] = x; }
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(SampleArgs a) {
  extern __shared__ __align__(16) unsigned char sample_smem[];
  unsigned long long* buf = reinterpret_cast<unsigned long long*>(sample_smem);          // [SAMPLE_CHUNK]
  float* wbuf = reinterpret_cast<float*>(sample_smem + SAMPLE_CHUNK * sizeof(unsigned long long));  // [SAMPLE_CHUNK]
  __shared__ SampleShared s;
  pdl_sync();
  const unsigned row = blockIdx.x;
  const size_t row_offset = static_cast<size_t>(row) * a.row_stride;

  // parameters (SamplingParameters::from_words) and the allow mask (validate_allow_mask)
  const float temperature = __uint_as_float(a.params[0]), top_p = __uint_as_float(a.params[2]);
  const unsigned top_k = a.params[1];
  const unsigned long long seed = static_cast<unsigned long long>(a.params[3]) | (static_cast<unsigned long long>(a.params[4]) << 32);
  bool valid = isfinite(temperature) && temperature >= 0.0f && isfinite(top_p) && top_p > 0.0f && top_p <= 1.0f;
  if (a.allow != nullptr) {
    const unsigned words = (a.width + 31) / 32, remainder = a.width % 32;
    unsigned any = 0;
    for (unsigned w = threadIdx.x; w < words; w += SAMPLE_THREADS) any |= a.allow[w];
    const unsigned total_any = block_sum_u32(any != 0 ? 1u : 0u, s);
    if (total_any == 0 || (remainder != 0 && (a.allow[words - 1] & ~((1u << remainder) - 1u)) != 0)) valid = false;
  }
  if (!valid) {
    if (threadIdx.x == 0) { report_error(a.err, ERR_INVALID, row); a.out[row] = 0; }
    return;
  }

  // allowed count and the greatest sort key (value, then highest index), which is also the greedy choice
  unsigned n_allowed = 0;
  unsigned long long best_key = 0;
  for (unsigned i = threadIdx.x; i < a.width; i += SAMPLE_THREADS) {
    if (!sample_allowed(a, i)) continue;
    ++n_allowed;
    const unsigned long long key = sample_key(a, row_offset, i);
    best_key = key > best_key ? key : best_key;
  }
  n_allowed = block_sum_u32(n_allowed, s);
  best_key = block_max_u64(best_key, s);
  if (temperature == 0.0f || top_k == 1) {
    if (threadIdx.x == 0) a.out[row] = static_cast<unsigned>(best_key & 0xFFFFFFFFu);
    return;
  }

  const unsigned cap = top_k == 0 ? n_allowed : min(top_k, n_allowed);
  const unsigned long long cap_key = cap == n_allowed ? 0ULL : select_rank(a, row_offset, cap, s);
  unsigned long long cut_key = cap_key;

  if (top_p < 1.0f) {
    const unsigned max_bits = key_to_bits(static_cast<unsigned>(best_key >> 32));
    const float v_max = __uint_as_float(max_bits);
    // weights that can move the running sums, and values that make the total non-finite
    unsigned significant = 0, poison = (max_bits & 0x7F800000u) == 0x7F800000u ? 1u : 0u;
    for (unsigned i = threadIdx.x; i < a.width; i += SAMPLE_THREADS) {
      if (!sample_allowed(a, i)) continue;
      const unsigned long long key = sample_key(a, row_offset, i);
      if (key < cap_key) continue;
      const unsigned bits = key_to_bits(static_cast<unsigned>(key >> 32));
      if ((bits & 0x7FFFFFFFu) > 0x7F800000u) poison = 1;
      else if (expf(__fdiv_rn(__fsub_rn(__uint_as_float(bits), v_max), temperature)) >= 1.4901161193847656e-08f) ++significant;  // 2^-26
    }
    significant = block_sum_u32(significant, s);
    poison = block_sum_u32(poison, s);
    if (poison != 0 || significant == 0) {
      cut_key = best_key;  // keeps the first candidate only
    } else {
      const unsigned chunks = (significant + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
      __syncthreads();
      if (threadIdx.x == 0) { s.total = 0.0f; s.cumulative = 0.0f; s.found = 0; }
      for (int phase = 0; phase < 2; ++phase) {
        unsigned long long previous = 0;
        for (unsigned c = 0; c < chunks; ++c) {
          const unsigned first = c * SAMPLE_CHUNK, last = min(first + SAMPLE_CHUNK, significant), count = last - first;
          if (!(chunks == 1 && phase == 1)) {
            const unsigned long long low_key = last == n_allowed ? 0ULL : (last == cap ? cap_key : select_rank(a, row_offset, last, s));  // rank cap is known already
            unsigned padded = 1;
            while (padded < count) padded <<= 1;
            __syncthreads();
            if (threadIdx.x == 0) s.gathered = 0;
            for (unsigned j = threadIdx.x; j < padded; j += SAMPLE_THREADS) buf[j] = 0;
            __syncthreads();
            for (unsigned i = threadIdx.x; i < a.width; i += SAMPLE_THREADS) {
              if (!sample_allowed(a, i)) continue;
              const unsigned long long key = sample_key(a, row_offset, i);
              if (key >= low_key && (c == 0 || key < previous)) {
                const unsigned at = atomicAdd(&s.gathered, 1u);
                if (at < SAMPLE_CHUNK) buf[at] = key;
              }
            }
            sort_desc(buf, padded);
            for (unsigned j = threadIdx.x; j < count; j += SAMPLE_THREADS)
              wbuf[j] = expf(__fdiv_rn(__fsub_rn(__uint_as_float(key_to_bits(static_cast<unsigned>(buf[j] >> 32))), v_max), temperature));
            previous = low_key;
            __syncthreads();
          }
          if (threadIdx.x == 0) {
            if (phase == 0) {
              float total = s.total;
              for (unsigned j = 0; j < count; ++j) total = __fadd_rn(total, wbuf[j]);
              s.total = total;
            } else {
              float cumulative = s.cumulative;
              const float total = s.total;
              for (unsigned j = 0; j < count; ++j) {
                cumulative = __fadd_rn(cumulative, __fdiv_rn(wbuf[j], total));
                if (cumulative >= top_p) { s.keep_key = buf[j]; s.found = 1; break; }
              }
              s.cumulative = cumulative;
            }
          }
          __syncthreads();
          if (s.found) break;
        }
      }
      if (s.found) cut_key = s.keep_key;
    }
  }

  // Gumbel-max over the kept candidates; equal scores: highest index
  unsigned long long best = 0;
  for (unsigned i = threadIdx.x; i < a.width; i += SAMPLE_THREADS) {
    if (!sample_allowed(a, i)) continue;
    const unsigned bits = load_f32_bits(a.x, a.x_dt, row_offset + i);
    const unsigned long long key = (static_cast<unsigned long long>(total_order_key_bits(bits)) << 32) | i;
    if (key < cut_key) continue;
    const unsigned long long scored = (static_cast<unsigned long long>(total_order_key_bits(sampled_score_bits(bits, temperature, seed, a.position, i))) << 32) | i;
    best = scored > best ? scored : best;
  }
  best = block_max_u64(best, s);
  if (threadIdx.x == 0) a.out[row] = static_cast<unsigned>(best & 0xFFFFFFFFu);
}

}  // namespace

void launch_sample(Ctx& ctx, const void* x, int x_dt, size_t row_stride, const unsigned* params, const unsigned* allow, unsigned* out, unsigned rows, unsigned width,
                   unsigned position, ErrorRecord* err) {
  if (rows == 0 || width == 0) return;
  const size_t smem = SAMPLE_CHUNK * (sizeof(unsigned long long) + sizeof(float));
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    configured[device] = true;
  }
  SampleArgs a{x, x_dt, row_stride, params, allow, out, width, position, err};
  launch_pdl(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), smem, ctx.stream, a);
  ctx.launches++;
}

}  // namespace fj
