// C ABI of the backend: buffer registry, program recognition, submission of validated dispatches.
// Mirrors forja_core::Backend / Submission (crates/forja-core/src/backend.rs:609-984) and the
// per-op execution of the reference CPU backend (crates/forja-cpu/src/lib.rs:1419-1516); every op
// runs as hand-written sm_100a kernels, there is no host fallback.
#include "fj_backend.h"

#include <math.h>
#include <string.h>

#include <algorithm>
#include <chrono>
#include <functional>
#include <thread>

using fj::View;

namespace fjb {

int32_t cuda_status(cudaError_t e) {
  if (e == cudaSuccess) return FJ_OK;
  if (e == cudaErrorMemoryAllocation) return FJ_ALLOCATION_FAILED;
  return FJ_DEVICE_EXECUTION_FAILED;
}

fj_buffer_rec* find_buffer(fj_backend* be, uint64_t id) {
  auto it = be->buffers.find(id);
  return it == be->buffers.end() ? nullptr : &it->second;
}

int32_t alloc_buffer(fj_backend* be, uint64_t bytes, uint64_t* id) {
  uint64_t total = 0;
  if (__builtin_add_overflow(be->used_bytes, bytes, &total)) return FJ_QUOTA_EXCEEDED;
  if (be->limit_bytes != 0 && total > be->limit_bytes) return FJ_QUOTA_EXCEEDED;
  void* ptr = nullptr;
  uint64_t alloc_bytes = bytes == 0 ? 16 : bytes;
  if (cudaMalloc(&ptr, alloc_bytes) != cudaSuccess) { cudaGetLastError(); return FJ_ALLOCATION_FAILED; }
  if (cudaMemsetAsync(ptr, 0, alloc_bytes, be->stream) != cudaSuccess) { cudaFree(ptr); return FJ_ALLOCATION_FAILED; }
  fj_buffer_rec rec;
  rec.ptr = ptr; rec.bytes = bytes; rec.readonly = false;
  *id = be->next_buffer++;
  be->buffers[*id] = rec;
  be->used_bytes += bytes;
  return FJ_OK;
}

uint64_t element_count(const fj_tensor& t) {
  uint64_t n = 1;
  for (uint32_t a = 0; a < t.rank; ++a) n *= t.shape[a];
  return n;
}

bool is_contiguous(const fj_tensor& t) {
  uint64_t expect = 1;
  for (int a = static_cast<int>(t.rank) - 1; a >= 0; --a) {
    if (t.shape[a] != 1 && t.strides[a] != expect) return false;
    expect *= t.shape[a];
  }
  return true;
}

// Byte range [lo, hi) a view can touch, with every product and sum overflow-checked like the
// reference's layout arithmetic (crates/forja-core/src/layout.rs uses checked_mul / checked_add
// throughout). An empty view spans [lo, lo). False: rank or dtype out of range, or the arithmetic
// wraps 64 bits - such a view addresses nothing valid.
bool tensor_byte_span(const fj_tensor& t, uint64_t* lo, uint64_t* hi) {
  if (t.rank > 8 || t.dtype > FJ_U32) return false;
  const uint64_t esz = fj::dtype_size(static_cast<int>(t.dtype));
  if (__builtin_mul_overflow(t.offset, esz, lo)) return false;
  bool empty = false;
  for (uint32_t a = 0; a < t.rank; ++a) empty = empty || t.shape[a] == 0;
  if (empty) { *hi = *lo; return true; }
  uint64_t last = t.offset;
  for (uint32_t a = 0; a < t.rank; ++a) {
    uint64_t step = 0;
    if (__builtin_mul_overflow(static_cast<uint64_t>(t.shape[a] - 1), t.strides[a], &step)) return false;
    if (__builtin_add_overflow(last, step, &last)) return false;
  }
  uint64_t count = 0;
  if (__builtin_add_overflow(last, static_cast<uint64_t>(1), &count)) return false;
  return !__builtin_mul_overflow(count, esz, hi);
}

void* tensor_ptr(fj_backend* be, const fj_tensor& t, bool for_write) {
  fj_buffer_rec* rec = find_buffer(be, t.buffer);
  if (rec == nullptr) return nullptr;
  if (for_write && rec->readonly) return nullptr;
  uint64_t lo = 0, hi = 0;
  if (!tensor_byte_span(t, &lo, &hi)) return nullptr;
  if (lo > rec->bytes || hi > rec->bytes) return nullptr;  // an empty view is never dereferenced but must still start inside
  return static_cast<char*>(rec->ptr) + lo;
}

bool make_view(fj_backend* be, const fj_tensor& t, bool for_write, View* out) {
  void* p = tensor_ptr(be, t, for_write);
  if (p == nullptr) return false;
  out->base = p;
  out->dtype = static_cast<int>(t.dtype);
  out->rank = static_cast<int>(t.rank);
  for (int a = 0; a < 8; ++a) { out->shape[a] = a < static_cast<int>(t.rank) ? t.shape[a] : 1; out->strides[a] = a < static_cast<int>(t.rank) ? t.strides[a] : 0; }
  if (t.rank == 0) { out->rank = 1; out->shape[0] = 1; out->strides[0] = 0; }
  return true;
}

const float* freq_table(fj_backend* be, float theta, float scale, unsigned count, bool reciprocal) {
  char key[96];
  uint32_t tb, sb;
  memcpy(&tb, &theta, 4); memcpy(&sb, &scale, 4);
  snprintf(key, sizeof(key), "%08x:%08x:%u:%d", tb, sb, count, reciprocal ? 1 : 0);
  auto it = be->freq_tables.find(key);
  if (it != be->freq_tables.end()) return it->second;
  std::vector<float> host(count);
  for (unsigned i = 0; i < count; ++i) {
    if (reciprocal) {
      // Op::Rope: theta.powf(2 * i / width).recip()  (crates/forja-cpu/src/lib.rs:694-696)
      float width = static_cast<float>(count * 2);
      host[i] = 1.0f / powf(theta, 2.0f * static_cast<float>(i) / width);
    } else {
      // guest programs: theta.powf(index as f32 * (-2 / head_dim))  (crates/forja-sdk/src/nn/blocks.rs:435-436)
      host[i] = powf(theta, static_cast<float>(i) * scale);
    }
  }
  float* dev = nullptr;
  if (cudaMalloc(&dev, std::max<size_t>(count, 1) * sizeof(float)) != cudaSuccess) return nullptr;
  cudaMemcpyAsync(dev, host.data(), count * sizeof(float), cudaMemcpyHostToDevice, be->stream);
  cudaStreamSynchronize(be->stream);
  be->freq_tables[key] = dev;
  return dev;
}

static bool ensure_scratch(fj_backend* be, void** ptr, size_t* have, size_t bytes) {
  if (*have >= bytes) return true;
  cudaStreamSynchronize(be->stream);  // nothing in flight may still use the old area
  if (*ptr) cudaFree(*ptr);
  *ptr = nullptr; *have = 0;
  size_t want = std::max<size_t>(bytes, 1 << 20);
  if (cudaMalloc(ptr, want) != cudaSuccess) { cudaGetLastError(); return false; }
  cudaMemsetAsync(*ptr, 0, want, be->stream);
  *have = want;
  return true;
}
bool ensure_gemm_scratch(fj_backend* be, size_t bytes) { return ensure_scratch(be, &be->gemm_scratch, &be->gemm_scratch_bytes, bytes); }
bool ensure_attn_scratch(fj_backend* be, size_t bytes) { return ensure_scratch(be, &be->attn_scratch, &be->attn_scratch_bytes, bytes); }

}  // namespace fjb

using namespace fjb;

// ---------------------------------------------------------------------------------------------
// program recognition: structural match on the expression DAG with constants folded
// ---------------------------------------------------------------------------------------------
namespace {

enum { T_INPUT = 0, T_CONST = 1, T_INDEX = 2, T_EXTENT = 3, T_UNARY = 4, T_BINARY = 5, T_SELECT = 6, T_CAST = 7, T_REDUCE = 8 };
enum { U_NEG, U_ABS, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_SIN, U_COS, U_TANH, U_SIGMOID, U_RECIP, U_FLOOR, U_LOG1P, U_EXPROUNDED };
enum { B_ADD, B_SUB, B_MUL, B_DIV, B_MIN, B_MAX, B_POW };
enum { R_SUM = 0 };

struct Prog {
  const uint32_t* insts; uint32_t n;
  const uint32_t* at(uint32_t i) const { return insts + 4 * i; }
  // constant folding of Const/arith subtrees (f32, same operations as the interpreter)
  bool constant(uint32_t i, float* v) const {
    const uint32_t* in = at(i);
    switch (in[0]) {
      case T_CONST: memcpy(v, &in[1], 4); return true;
      case T_UNARY: { float x; if (!constant(in[2], &x)) return false; if (in[1] == U_NEG) { *v = -x; return true; } if (in[1] == U_RECIP) { *v = 1.0f / x; return true; } return false; }
      case T_BINARY: {
        float a, b;
        if (!constant(in[2], &a) || !constant(in[3], &b)) return false;
        switch (in[1]) { case B_ADD: *v = a + b; return true; case B_SUB: *v = a - b; return true; case B_MUL: *v = a * b; return true; case B_DIV: *v = a / b; return true; default: return false; }
      }
      default: return false;
    }
  }
  bool is_input(uint32_t i, uint32_t slot) const { return at(i)[0] == T_INPUT && at(i)[1] == slot; }
  bool unary(uint32_t i, uint32_t op, uint32_t* x) const { if (at(i)[0] != T_UNARY || at(i)[1] != op) return false; *x = at(i)[2]; return true; }
  bool binary(uint32_t i, uint32_t op, uint32_t* l, uint32_t* r) const { if (at(i)[0] != T_BINARY || at(i)[1] != op) return false; *l = at(i)[2]; *r = at(i)[3]; return true; }
  // commutative binary where one side satisfies `first`; the other side is returned
  bool binary_with(uint32_t i, uint32_t op, const std::function<bool(uint32_t)>& first, uint32_t* other) const {
    uint32_t l, r;
    if (!binary(i, op, &l, &r)) return false;
    if (first(l)) { *other = r; return true; }
    if (first(r)) { *other = l; return true; }
    return false;
  }
  // same expression (structural equality)
  bool same(uint32_t a, uint32_t b) const {
    if (a == b) return true;
    const uint32_t *x = at(a), *y = at(b);
    if (x[0] != y[0]) return false;
    switch (x[0]) {
      case T_INPUT: case T_CONST: case T_INDEX: case T_EXTENT: return x[1] == y[1];
      case T_UNARY: case T_CAST: case T_REDUCE: return x[1] == y[1] && same(x[2], y[2]);
      case T_BINARY: return x[1] == y[1] && ((same(x[2], y[2]) && same(x[3], y[3])) || ((x[1] == B_ADD || x[1] == B_MUL) && same(x[2], y[3]) && same(x[3], y[2])));
      default: return false;
    }
  }
  // square(i, &x): i == x * x
  bool square(uint32_t i, uint32_t* x) const { uint32_t l, r; if (!binary(i, B_MUL, &l, &r) || !same(l, r)) return false; *x = l; return true; }
  // inverse RMS: rsqrt(sum / width + eps) with width a constant or cast(extent); returns the reduced expression
  bool inverse_rms(uint32_t i, uint32_t* reduced, float* eps, float* width /*0 = extent*/) const {
    uint32_t arg, mean = 0, l, r;
    if (!unary(i, U_RSQRT, &arg)) return false;
    float e;
    if (!binary(arg, B_ADD, &l, &r)) return false;
    if (constant(r, &e)) mean = l; else if (constant(l, &e)) mean = r; else return false;
    *eps = e;
    uint32_t sum, den;
    if (!binary(mean, B_DIV, &sum, &den)) return false;
    float w;
    if (constant(den, &w)) *width = w;
    else if (at(den)[0] == T_CAST && at(den)[1] == 0 && at(at(den)[2])[0] == T_EXTENT) *width = 0.0f;
    else return false;
    if (at(sum)[0] != T_REDUCE || at(sum)[1] != R_SUM) return false;
    *reduced = at(sum)[2];
    return true;
  }
};

// normalized(i, x_is, w_slot): i == (x * inv) * Input(w_slot); returns inv
bool match_scaled(const Prog& p, uint32_t i, const std::function<bool(uint32_t)>& is_x, uint32_t w_slot, uint32_t* inv) {
  uint32_t inner;
  if (!p.binary_with(i, B_MUL, [&](uint32_t n) { return p.is_input(n, w_slot); }, &inner)) return false;
  return p.binary_with(inner, B_MUL, is_x, inv);
}

bool recognise(uint32_t kind, const uint32_t* insts, uint32_t n, const uint32_t* outs, uint32_t n_out, fj_program_rec* rec) {
  Prog p{insts, n};
  for (uint32_t i = 0; i < n; ++i) {  // operands must point backward
    const uint32_t* in = p.at(i);
    if (in[0] > T_REDUCE) return false;
    if ((in[0] == T_UNARY || in[0] == T_CAST || in[0] == T_REDUCE) && in[2] >= i) return false;
    if (in[0] == T_BINARY && (in[2] >= i || in[3] >= i)) return false;
    if (in[0] == T_SELECT && (in[1] >= i || in[2] >= i || in[3] >= i)) return false;
  }
  auto out_of = [&](uint32_t slot, uint32_t* inst) { for (uint32_t o = 0; o < n_out; ++o) if (outs[2 * o] == slot && outs[2 * o + 1] < n) { *inst = outs[2 * o + 1]; return true; } return false; };
  uint32_t o0, o1, l, r;
  if (!out_of(0, &o0)) return false;
  if (kind == 0 && n_out == 1) {
    // add: Input0 + Input1
    if (p.binary(o0, B_ADD, &l, &r) && ((p.is_input(l, 0) && p.is_input(r, 1)) || (p.is_input(l, 1) && p.is_input(r, 0)))) { rec->kernel = 1; return true; }
    // silu_mul: (gate * sigmoid(gate)) * up
    uint32_t inner, sig, x;
    if (p.binary_with(o0, B_MUL, [&](uint32_t q) { return p.is_input(q, 1); }, &inner) &&
        p.binary_with(inner, B_MUL, [&](uint32_t q) { return p.is_input(q, 0); }, &sig) && p.unary(sig, U_SIGMOID, &x) && p.is_input(x, 0)) { rec->kernel = 2; return true; }
    // gated up, the matmul epilogue of engines/smollm2/src/optimized.rs:249-252: (gate * sigmoid(gate)) * up with up = Input0 (the accumulator), gate = Input1
    if (p.binary_with(o0, B_MUL, [&](uint32_t q) { return p.is_input(q, 0); }, &inner) &&
        p.binary_with(inner, B_MUL, [&](uint32_t q) { return p.is_input(q, 1); }, &sig) && p.unary(sig, U_SIGMOID, &x) && p.is_input(x, 1)) { rec->kernel = 7; return true; }
    return false;
  }
  if (kind == 1 && n_out == 1) {
    // rms_norm: (x * rsqrt(mean(x*x) + eps)) * w
    uint32_t inv, red, sq;
    float eps, width;
    if (match_scaled(p, o0, [&](uint32_t q) { return p.is_input(q, 0); }, 1, &inv) && p.inverse_rms(inv, &red, &eps, &width) && width == 0.0f &&
        p.square(red, &sq) && p.is_input(sq, 0)) { rec->kernel = 3; rec->eps = eps; return true; }
    return false;
  }
  if (!out_of(1, &o1)) return false;
  if (kind == 1 && n_out == 2) {
    // residual_norm: value = r + u; out0 = value; out1 = (value * inv) * w
    if (p.binary(o0, B_ADD, &l, &r) && ((p.is_input(l, 0) && p.is_input(r, 1)) || (p.is_input(l, 1) && p.is_input(r, 0)))) {
      uint32_t inv, red, sq;
      float eps, width;
      if (match_scaled(p, o1, [&](uint32_t q) { return p.same(q, o0); }, 2, &inv) && p.inverse_rms(inv, &red, &eps, &width) && width == 0.0f &&
          p.square(red, &sq) && p.same(sq, o0)) { rec->kernel = 4; rec->eps = eps; return true; }
      return false;
    }
    // qk_norm_rope: out0 = nlo*cos - nhi*sin; out1 = nhi*cos + nlo*sin
    uint32_t a, b, c, d;
    if (!p.binary(o0, B_SUB, &a, &b) || !p.binary(o1, B_ADD, &c, &d)) return false;
    // a = nlo * cos, b = nhi * sin
    uint32_t al, ar, bl, br;
    if (!p.binary(a, B_MUL, &al, &ar) || !p.binary(b, B_MUL, &bl, &br)) return false;
    uint32_t cosn, sinn, nlo, nhi, ang;
    if (p.unary(ar, U_COS, &ang)) { cosn = ar; nlo = al; } else if (p.unary(al, U_COS, &ang)) { cosn = al; nlo = ar; } else return false;
    uint32_t ang2;
    if (p.unary(br, U_SIN, &ang2)) { sinn = br; nhi = bl; } else if (p.unary(bl, U_SIN, &ang2)) { sinn = bl; nhi = br; } else return false;
    if (!p.same(ang, ang2)) return false;
    // out1 = nhi*cos + nlo*sin (either order)
    auto is_prod = [&](uint32_t q, uint32_t x, uint32_t y) { uint32_t ql, qr; return p.binary(q, B_MUL, &ql, &qr) && ((p.same(ql, x) && p.same(qr, y)) || (p.same(ql, y) && p.same(qr, x))); };
    if (!((is_prod(c, nhi, cosn) && is_prod(d, nlo, sinn)) || (is_prod(d, nhi, cosn) && is_prod(c, nlo, sinn)))) return false;
    // angle = pos(Input 4) * pow(theta, cast(index) * scale)
    uint32_t freq;
    if (!p.binary_with(ang, B_MUL, [&](uint32_t q) { return p.is_input(q, 4); }, &freq)) return false;
    uint32_t base, expo;
    float theta, scale;
    if (!p.binary(freq, B_POW, &base, &expo) || !p.constant(base, &theta)) return false;
    uint32_t idx;
    if (!p.binary_with(expo, B_MUL, [&](uint32_t q) { float t; return p.constant(q, &t); }, &idx)) return false;
    {
      uint32_t el, er;
      p.binary(expo, B_MUL, &el, &er);
      if (!p.constant(el == idx ? er : el, &scale)) return false;
    }
    if (p.at(idx)[0] != T_CAST || p.at(idx)[1] != 0 || p.at(p.at(idx)[2])[0] != T_INDEX) return false;
    // nlo = (Input0 * inv) * Input2 ; nhi = (Input1 * inv) * Input3 ; inv = rsqrt(sum(lo*lo + hi*hi)/head_dim + eps)
    uint32_t inv_lo, inv_hi, red;
    float eps, width;
    if (!match_scaled(p, nlo, [&](uint32_t q) { return p.is_input(q, 0); }, 2, &inv_lo)) return false;
    if (!match_scaled(p, nhi, [&](uint32_t q) { return p.is_input(q, 1); }, 3, &inv_hi) || !p.same(inv_lo, inv_hi)) return false;
    if (!p.inverse_rms(inv_lo, &red, &eps, &width) || width <= 0.0f) return false;
    uint32_t s0, s1, x0, x1;
    if (!p.binary(red, B_ADD, &s0, &s1) || !p.square(s0, &x0) || !p.square(s1, &x1)) return false;
    if (!((p.is_input(x0, 0) && p.is_input(x1, 1)) || (p.is_input(x0, 1) && p.is_input(x1, 0)))) return false;
    rec->kernel = 5; rec->eps = eps; rec->theta = theta; rec->head_dim = width; rec->exponent_scale = scale;
    return true;
  }
  if (kind == 0 && n_out == 2) {
    // rope_pairs: out0 = first*cos - second*sin ; out1 = second*cos + first*sin ; angle = Input2 * pow(theta, cast(index)*scale)
    uint32_t a, b, c, d, al, ar, bl, br, ang, ang2, cosn, sinn, fst, snd;
    if (!p.binary(o0, B_SUB, &a, &b) || !p.binary(o1, B_ADD, &c, &d)) return false;
    if (!p.binary(a, B_MUL, &al, &ar) || !p.binary(b, B_MUL, &bl, &br)) return false;
    if (p.unary(ar, U_COS, &ang)) { cosn = ar; fst = al; } else if (p.unary(al, U_COS, &ang)) { cosn = al; fst = ar; } else return false;
    if (p.unary(br, U_SIN, &ang2)) { sinn = br; snd = bl; } else if (p.unary(bl, U_SIN, &ang2)) { sinn = bl; snd = br; } else return false;
    if (!p.same(ang, ang2) || !p.is_input(fst, 0) || !p.is_input(snd, 1)) return false;
    auto is_prod = [&](uint32_t q, uint32_t x, uint32_t y) { uint32_t ql, qr; return p.binary(q, B_MUL, &ql, &qr) && ((p.same(ql, x) && p.same(qr, y)) || (p.same(ql, y) && p.same(qr, x))); };
    if (!((is_prod(c, snd, cosn) && is_prod(d, fst, sinn)) || (is_prod(d, snd, cosn) && is_prod(c, fst, sinn)))) return false;
    uint32_t freq, base, expo, idx;
    float theta, scale;
    if (!p.binary_with(ang, B_MUL, [&](uint32_t q) { return p.is_input(q, 2); }, &freq)) return false;
    if (!p.binary(freq, B_POW, &base, &expo) || !p.constant(base, &theta)) return false;
    if (!p.binary_with(expo, B_MUL, [&](uint32_t q) { float t; return p.constant(q, &t); }, &idx)) return false;
    {
      uint32_t el, er;
      p.binary(expo, B_MUL, &el, &er);
      if (!p.constant(el == idx ? er : el, &scale)) return false;
    }
    if (p.at(idx)[0] != T_CAST || p.at(idx)[1] != 0 || p.at(p.at(idx)[2])[0] != T_INDEX) return false;
    rec->kernel = 6; rec->theta = theta; rec->exponent_scale = scale;
    return true;
  }
  return false;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// submission
// ---------------------------------------------------------------------------------------------

struct fj_submission {
  fj_backend* be = nullptr;
  uint64_t serial = 0;
  cudaEvent_t start = nullptr, stop = nullptr;
  uint32_t count = 0;
  std::vector<uint32_t> ops;
  std::vector<uint32_t> kernels;
  std::vector<cudaEvent_t> marks;  // count + 1 events when profiled
  std::vector<uint64_t> costs;     // {read bytes, write bytes, flops} per dispatch when profiled
  fj::ErrorRecord* host_err = nullptr;  // pinned, count entries (recycled through the backend)
  size_t host_err_capacity = 0;
  bool done = false;
  int32_t result = FJ_OK;
  fj_device_error error{};
  uint64_t launches = 0;
};

namespace {

struct Exec {
  fj_backend* be;
  std::vector<void*> temps;            // stream-ordered temporaries, freed at the end of submit
  std::vector<std::function<void()>> finals;  // scatter-backs of materialised outputs for the current dispatch
  fj::ErrorRecord* dev_err = nullptr;

  void* temp(size_t bytes) {
    void* p = nullptr;
    if (cudaMallocAsync(&p, std::max<size_t>(bytes, 16), be->stream) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    temps.push_back(p);
    return p;
  }
  template <typename T> T* upload(const std::vector<T>& host) {
    T* dev = static_cast<T*>(temp(host.size() * sizeof(T)));
    if (dev && !host.empty()) cudaMemcpyAsync(dev, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice, be->stream);
    return dev;
  }
  // contiguous logical image of an input tensor (the tensor itself when already contiguous)
  const void* input(const fj_tensor& t) {
    void* p = tensor_ptr(be, t, false);
    if (p == nullptr) return nullptr;
    if (is_contiguous(t)) return p;
    uint64_t n = element_count(t);
    void* tmp = temp(n * fj::dtype_size(t.dtype));
    if (!tmp) return nullptr;
    View in, out;
    make_view(be, t, false, &in);
    out = in; out.base = tmp;
    uint64_t stride = 1;
    for (int a = static_cast<int>(t.rank) - 1; a >= 0; --a) { out.strides[a] = stride; stride *= t.shape[a]; }
    fj::launch_copy(be->ctx, in, out, n);
    return tmp;
  }
  // contiguous destination for an output tensor; scattered back by finish() when it was a temp
  void* output(const fj_tensor& t) {
    void* p = tensor_ptr(be, t, true);
    if (p == nullptr) return nullptr;
    if (is_contiguous(t)) return p;
    uint64_t n = element_count(t);
    void* tmp = temp(n * fj::dtype_size(t.dtype));
    if (!tmp) return nullptr;
    fj_tensor copy = t;
    finals.push_back([this, copy, tmp, n]() {
      View out, in;
      make_view(be, copy, true, &out);
      in = out; in.base = tmp;
      uint64_t stride = 1;
      for (int a = static_cast<int>(copy.rank) - 1; a >= 0; --a) { in.strides[a] = stride; stride *= copy.shape[a]; }
      fj::launch_copy(be->ctx, in, out, n);
    });
    return tmp;
  }
  void finish() { for (auto& f : finals) f(); finals.clear(); }
};

bool same_shape(const fj_tensor& a, const fj_tensor& b) {
  if (a.rank != b.rank) return false;
  for (uint32_t i = 0; i < a.rank; ++i) if (a.shape[i] != b.shape[i]) return false;
  return true;
}
bool is_float(uint32_t dt) { return dt <= FJ_BF16; }

// ---- per-op execution; each returns an fj_status ---------------------------------------------

int32_t exec_copy(Exec& x, const fj_dispatch& d) {
  if (d.n_inputs != 1 || d.n_outputs != 1 || !same_shape(d.inputs[0], d.outputs[0])) return FJ_INVALID_INPUT;
  View in, out;
  if (!make_view(x.be, d.inputs[0], false, &in) || !make_view(x.be, d.outputs[0], true, &out)) return FJ_INVALID_INPUT;
  const bool in_int = !is_float(in.dtype), out_int = !is_float(out.dtype);
  if (in_int != out_int) return FJ_INVALID_INPUT;
  fj::launch_copy(x.be->ctx, in, out, element_count(d.inputs[0]));
  return FJ_OK;
}

// view of `w` broadcast over the leading axes of `like` (w indexes the last axis)
bool broadcast_last(fj_backend* be, const fj_tensor& w, const fj_tensor& like, View* out) {
  if (w.rank != 1 || like.rank == 0 || w.shape[0] != like.shape[like.rank - 1]) return false;
  fj_tensor b = w;
  b.rank = like.rank;
  for (uint32_t a = 0; a < like.rank; ++a) { b.shape[a] = like.shape[a]; b.strides[a] = 0; }
  b.strides[like.rank - 1] = w.strides[0];
  // bounds are those of the 1-d weight itself
  if (tensor_ptr(be, w, false) == nullptr) return false;
  out->base = tensor_ptr(be, w, false);
  out->dtype = w.dtype; out->rank = like.rank;
  for (int a = 0; a < 8; ++a) { out->shape[a] = a < static_cast<int>(like.rank) ? b.shape[a] : 1; out->strides[a] = a < static_cast<int>(like.rank) ? b.strides[a] : 0; }
  return true;
}

int32_t exec_rms_norm(Exec& x, const fj_dispatch& d) {
  if (d.n_inputs != 2 || d.n_outputs != 1 || !same_shape(d.inputs[0], d.outputs[0]) || d.inputs[0].rank == 0) return FJ_INVALID_INPUT;
  View in, w, out;
  if (!make_view(x.be, d.inputs[0], false, &in) || !make_view(x.be, d.outputs[0], true, &out) || !broadcast_last(x.be, d.inputs[1], d.inputs[0], &w)) return FJ_INVALID_INPUT;
  const unsigned width = d.inputs[0].shape[d.inputs[0].rank - 1];
  if (width == 0) return FJ_OK;
  fj::launch_rms_norm(x.be->ctx, in, w, out, element_count(d.inputs[0]) / width, width, d.f0);
  return FJ_OK;
}

int32_t exec_argmax(Exec& x, const fj_dispatch& d) {
  if (d.n_inputs != 1 || d.n_outputs != 1 || d.inputs[0].rank == 0 || !is_float(d.inputs[0].dtype) || d.outputs[0].dtype != FJ_U32) return FJ_INVALID_INPUT;
  const unsigned width = d.inputs[0].shape[d.inputs[0].rank - 1];
  if (width == 0) return FJ_EXECUTION_FAILED;
  const uint64_t rows = element_count(d.inputs[0]) / width;
  if (element_count(d.outputs[0]) != rows) return FJ_INVALID_INPUT;
  const void* in = x.input(d.inputs[0]);
  unsigned* out = static_cast<unsigned*>(x.output(d.outputs[0]));
  void* scratch = x.temp(fj::argmax_scratch_bytes(static_cast<unsigned>(rows), width));
  if (!in || !out || !scratch) return FJ_INVALID_INPUT;
  fj::launch_argmax(x.be->ctx, in, d.inputs[0].dtype, width, out, static_cast<unsigned>(rows), width, scratch);
  return FJ_OK;
}

// Op::Sample (2 inputs) and Op::SampleMasked (3 inputs), crates/forja-core/src/ops.rs:1546-1592.
int32_t exec_sample(Exec& x, const fj_dispatch& d, fj::ErrorRecord* err) {
  if ((d.n_inputs != 2 && d.n_inputs != 3) || d.n_outputs != 1 || d.inputs[0].rank == 0 || !is_float(d.inputs[0].dtype) || d.outputs[0].dtype != FJ_U32) return FJ_INVALID_INPUT;
  if (d.inputs[1].dtype != FJ_U32 || d.inputs[1].rank != 1 || d.inputs[1].shape[0] != 5) return FJ_INVALID_INPUT;
  const unsigned width = d.inputs[0].shape[d.inputs[0].rank - 1];
  if (width == 0) return FJ_EXECUTION_FAILED;
  const uint64_t rows = element_count(d.inputs[0]) / width;
  if (element_count(d.outputs[0]) != rows || rows > 0x7FFFFFFFu) return FJ_INVALID_INPUT;
  const bool masked = d.n_inputs == 3;
  if (masked && (d.inputs[2].dtype != FJ_U32 || d.inputs[2].rank != 1 || d.inputs[2].shape[0] != (width + 31) / 32 || !is_contiguous(d.inputs[2]))) return FJ_INVALID_INPUT;
  const void* in = x.input(d.inputs[0]);
  const void* params = x.input(d.inputs[1]);
  const void* allow = masked ? x.input(d.inputs[2]) : nullptr;
  unsigned* out = static_cast<unsigned*>(x.output(d.outputs[0]));
  if (!in || !params || !out || (masked && !allow)) return FJ_INVALID_INPUT;
  fj::launch_sample(x.be->ctx, in, d.inputs[0].dtype, width, static_cast<const unsigned*>(params), static_cast<const unsigned*>(allow), out, static_cast<unsigned>(rows), width, d.u0, err);
  return FJ_OK;
}

int32_t exec_top_k(Exec& x, const fj_dispatch& d) {
  if (d.n_inputs != 1 || d.n_outputs != 2 || d.inputs[0].rank == 0 || !is_float(d.inputs[0].dtype) || d.outputs[1].dtype != FJ_U32) return FJ_INVALID_INPUT;
  const unsigned width = d.inputs[0].shape[d.inputs[0].rank - 1], k = d.u0;
  if (k == 0 || k > width) return FJ_INVALID_INPUT;
  if (width > 24000 || (d.u1 && k > 64)) return FJ_UNSUPPORTED_OPERATION;
  const uint64_t rows = element_count(d.inputs[0]) / width;
  if (element_count(d.outputs[0]) != rows * k || element_count(d.outputs[1]) != rows * k) return FJ_INVALID_INPUT;
  const void* in = x.input(d.inputs[0]);
  void* values = x.output(d.outputs[0]);
  unsigned* indices = static_cast<unsigned*>(x.output(d.outputs[1]));
  if (!in || !values || !indices) return FJ_INVALID_INPUT;
  fj::launch_top_k(x.be->ctx, in, d.inputs[0].dtype, values, d.outputs[0].dtype, indices, static_cast<unsigned>(rows), width, k, d.u1 != 0);
  return FJ_OK;
}

// halves of a [.., width] tensor as views over [.., width/2]
bool half_views(fj_backend* be, const fj_tensor& t, bool for_write, View* lo, View* hi) {
  if (t.rank == 0 || t.shape[t.rank - 1] % 2 != 0) return false;
  if (!make_view(be, t, for_write, lo)) return false;
  const unsigned half = t.shape[t.rank - 1] / 2;
  lo->shape[t.rank - 1] = half;
  *hi = *lo;
  hi->base = static_cast<char*>(lo->base) + static_cast<size_t>(half) * t.strides[t.rank - 1] * fj::dtype_size(t.dtype);
  return true;
}

int32_t exec_rope(Exec& x, const fj_dispatch& d) {
  if (d.n_inputs != 2 || d.n_outputs != 1 || d.inputs[0].rank != 3 || !same_shape(d.inputs[0], d.outputs[0])) return FJ_INVALID_INPUT;
  if (d.inputs[1].rank != 1 || d.inputs[1].dtype != FJ_U32 || d.inputs[1].shape[0] != d.inputs[0].shape[0]) return FJ_INVALID_INPUT;
  View lo, hi, olo, ohi, pos;
  if (!half_views(x.be, d.inputs[0], false, &lo, &hi) || !half_views(x.be, d.outputs[0], true, &olo, &ohi)) return FJ_INVALID_INPUT;
  if (!make_view(x.be, d.inputs[1], false, &pos)) return FJ_INVALID_INPUT;
  pos.rank = 3;
  pos.strides[0] = d.inputs[1].strides[0]; pos.strides[1] = 0; pos.strides[2] = 0;
  for (int a = 0; a < 3; ++a) pos.shape[a] = lo.shape[a];
  const unsigned half = lo.shape[2];
  const float* table = freq_table(x.be, d.f0, 0.0f, half, true);
  if (!table) return FJ_ALLOCATION_FAILED;
  fj::launch_rope_pairs(x.be->ctx, lo, hi, pos, olo, ohi, element_count(d.inputs[0]) / 2, half, table);
  return FJ_OK;
}

int32_t exec_embed(Exec& x, const fj_dispatch& d, fj::ErrorRecord* err) {
  if (d.n_inputs != 2 || d.n_outputs != 1 || d.inputs[0].rank != 2 || d.inputs[1].dtype != FJ_U32) return FJ_INVALID_INPUT;
  const unsigned vocab = d.inputs[0].shape[0], width = d.inputs[0].shape[1];
  const uint64_t count = element_count(d.inputs[1]);
  if (element_count(d.outputs[0]) != count * width) return FJ_INVALID_INPUT;
  const void* table = x.input(d.inputs[0]);
  const unsigned* ids = static_cast<const unsigned*>(x.input(d.inputs[1]));
  void* out = x.output(d.outputs[0]);
  if (!table || !ids || !out) return FJ_INVALID_INPUT;
  fj::launch_embed(x.be->ctx, table, d.inputs[0].dtype, ids, out, d.outputs[0].dtype, vocab, width, static_cast<unsigned>(count), err);
  return FJ_OK;
}

bool quant_params_ok(unsigned bits, unsigned group) { return (bits == 4 || bits == 8) && (group == 32 || group == 64 || group == 128); }

int32_t exec_quant_embed(Exec& x, const fj_dispatch& d, fj::ErrorRecord* err) {
  if (d.n_inputs != 4 || d.n_outputs != 1 || d.inputs[0].rank != 2 || !quant_params_ok(d.u0, d.u1)) return FJ_INVALID_INPUT;
  const unsigned vocab = d.inputs[0].shape[0], packed_width = d.inputs[0].shape[1];
  const uint64_t count = element_count(d.inputs[3]);
  const unsigned width = packed_width * (32 / d.u0);
  if (width % d.u1 != 0 || element_count(d.outputs[0]) != count * width || d.inputs[1].dtype != d.inputs[2].dtype) return FJ_INVALID_INPUT;
  const void *packed = x.input(d.inputs[0]), *scales = x.input(d.inputs[1]), *biases = x.input(d.inputs[2]), *ids = x.input(d.inputs[3]);
  void* out = x.output(d.outputs[0]);
  if (!packed || !scales || !biases || !ids || !out) return FJ_INVALID_INPUT;
  fj::launch_quant_embed(x.be->ctx, static_cast<const unsigned*>(packed), scales, biases, d.inputs[1].dtype, static_cast<const unsigned*>(ids), out,
                         d.outputs[0].dtype, vocab, packed_width, static_cast<unsigned>(count), d.u0, d.u1, err);
  return FJ_OK;
}

// Scalar epilogue of a matrix product (apply_epilogue_accumulators, crates/forja-cpu/src/lib.rs:443-493): the Map program sees the
// f32 accumulator as input 0 and the extra operands after it; its output is rounded once to the output dtype. Recognised
// forms: accumulator + extra (bias or residual add), silu(extra) * accumulator (gated up), silu(accumulator) * extra.
// Runs the product into an f32 temporary via `product(temp tensor)`, then one element-wise pass.
template <typename Product>
int32_t with_epilogue(Exec& x, const fj_dispatch& d, uint32_t primitive_inputs, Product product) {
  if (d.program == 0 || d.program > x.be->programs.size()) return FJ_INVALID_INPUT;
  const uint32_t kernel = x.be->programs[d.program - 1].kernel;
  if (kernel != 1 && kernel != 2 && kernel != 7) return FJ_UNSUPPORTED_OPERATION;
  if (d.n_inputs != primitive_inputs + 1 || d.n_outputs != 1) return FJ_INVALID_INPUT;
  const fj_tensor &extra = d.inputs[primitive_inputs], &out = d.outputs[0];
  if (!same_shape(extra, out) || !is_float(extra.dtype) || !is_float(out.dtype) || out.rank != 2) return FJ_INVALID_INPUT;
  const uint64_t elements = element_count(out);
  float* acc = static_cast<float*>(x.temp(std::max<uint64_t>(elements, 1) * sizeof(float)));
  if (!acc) return FJ_ALLOCATION_FAILED;
  const int32_t status = product(acc);
  if (status != FJ_OK || elements == 0) return status;
  View ve, vo;
  if (!make_view(x.be, extra, false, &ve) || !make_view(x.be, out, true, &vo)) return FJ_INVALID_INPUT;
  View va = dense_view(acc, FJ_F32, out.shape[0], out.shape[1], out.shape[1]);
  if (kernel == 1) fj::launch_add(x.be->ctx, va, ve, vo, elements);
  else if (kernel == 7) fj::launch_silu_mul(x.be->ctx, ve, va, vo, elements);  // gate = extra, up = accumulator
  else fj::launch_silu_mul(x.be->ctx, va, ve, vo, elements);                    // gate = accumulator, up = extra
  return FJ_OK;
}

int32_t exec_matmul_plain(Exec& x, const fj_dispatch& d, float* acc_out);

int32_t exec_matmul(Exec& x, const fj_dispatch& d) {
  if (d.program != 0) {
    if (d.n_inputs < 2 || d.inputs[0].rank != 2) return FJ_UNSUPPORTED_OPERATION;  // epilogues are used on rank-2 products
    return with_epilogue(x, d, 2, [&](float* acc) { return exec_matmul_plain(x, d, acc); });
  }
  return exec_matmul_plain(x, d, nullptr);
}

// acc_out != nullptr: the product goes to that contiguous f32 [m, n] area instead of the dispatch's output.
int32_t exec_matmul_plain(Exec& x, const fj_dispatch& d, float* acc_out) {
  if (d.n_inputs < 2 || d.n_outputs != 1 || (acc_out == nullptr && d.n_inputs != 2)) return FJ_INVALID_INPUT;
  const fj_tensor &a = d.inputs[0], &b = d.inputs[1];
  fj_tensor c = d.outputs[0];
  if (acc_out != nullptr) { c.dtype = FJ_F32; c.strides[0] = c.shape[1]; c.strides[1] = 1; }
  if (a.rank != b.rank || a.rank != c.rank || (a.rank != 2 && a.rank != 3)) return FJ_INVALID_INPUT;
  const uint32_t r = a.rank;
  const unsigned m = a.shape[r - 2], k = a.shape[r - 1], n = b.shape[r - 1];
  const unsigned batch = r == 3 ? a.shape[0] : 1;
  if (b.shape[r - 2] != k || c.shape[r - 2] != m || c.shape[r - 1] != n || (r == 3 && (b.shape[0] != batch || c.shape[0] != batch))) return FJ_INVALID_INPUT;
  if (m == 0 || n == 0) return FJ_OK;
  // fast path: rank 2, rows contiguous, weight stored [n, k] and viewed transposed, same float dtype
  const bool nt = r == 2 && a.strides[1] == 1 && b.strides[0] == 1 && c.strides[1] == 1 && a.dtype == b.dtype && is_float(a.dtype) && is_float(c.dtype) && k > 0;
  if (nt) {
    const void* ap = tensor_ptr(x.be, a, false);
    const void* bp = tensor_ptr(x.be, b, false);
    void* cp = acc_out != nullptr ? static_cast<void*>(acc_out) : tensor_ptr(x.be, c, true);
    if (!ap || !bp || !cp) return FJ_INVALID_INPUT;
    size_t need = fj::gemm_scratch_bytes(m, n, k);
    void* scratch = nullptr; size_t scratch_bytes = 0;
    if (a.dtype != FJ_F32 && m > 16 && need <= (size_t(1) << 30) && ensure_gemm_scratch(x.be, need)) { scratch = x.be->gemm_scratch; scratch_bytes = x.be->gemm_scratch_bytes; }
    fj::launch_gemm_nt(x.be->ctx, ap, a.dtype, a.strides[0], bp, b.dtype, b.strides[1], cp, c.dtype, c.strides[0], m, n, k, scratch, scratch_bytes);
    return FJ_OK;
  }
  View va, vb, vc;
  if (!make_view(x.be, a, false, &va) || !make_view(x.be, b, false, &vb)) return FJ_INVALID_INPUT;
  if (acc_out != nullptr) vc = dense_view(acc_out, FJ_F32, m, n, n);
  else if (!make_view(x.be, c, true, &vc)) return FJ_INVALID_INPUT;
  fj::launch_matmul_generic(x.be->ctx, va, vb, vc, batch, m, n, k);
  return FJ_OK;
}

// Op::Sdpa, crates/forja-core/src/ops.rs:270 (check :2180-2234): q [hq, T, d], k [kvh, L, d], v [kvh, L, dv] -> out [hq, T, dv];
// f0 = scale, u0 = causal, u1 = q_start. Views may be strided (a cache sliced to its live length).
int32_t exec_sdpa(Exec& x, const fj_dispatch& d) {
  if (d.n_inputs != 3 || d.n_outputs != 1) return FJ_INVALID_INPUT;
  const fj_tensor &q = d.inputs[0], &k = d.inputs[1], &v = d.inputs[2], &o = d.outputs[0];
  if (q.rank != 3 || k.rank != 3 || v.rank != 3 || o.rank != 3 || !is_float(q.dtype) || !is_float(k.dtype) || !is_float(v.dtype) || !is_float(o.dtype)) return FJ_INVALID_INPUT;
  if (k.shape[0] == 0 || q.shape[0] % k.shape[0] != 0 || v.shape[0] != k.shape[0] || v.shape[1] != k.shape[1] || k.shape[2] != q.shape[2]) return FJ_INVALID_INPUT;
  if (o.shape[0] != q.shape[0] || o.shape[1] != q.shape[1] || o.shape[2] != v.shape[2]) return FJ_INVALID_INPUT;
  // causal rows attend q_start + row + 1 keys: the last row must not reach past the cache (ops.rs check_sdpa)
  if (d.u0 && static_cast<uint64_t>(d.u1) + q.shape[1] > k.shape[1]) return FJ_INVALID_INPUT;
  View vq, vk, vv, vo;
  if (!make_view(x.be, q, false, &vq) || !make_view(x.be, k, false, &vk) || !make_view(x.be, v, false, &vv) || !make_view(x.be, o, true, &vo)) return FJ_INVALID_INPUT;
  return fj::launch_sdpa(x.be->ctx, vq, vk, vv, vo, d.f0, d.u0 != 0, d.u1) ? FJ_OK : FJ_UNSUPPORTED_OPERATION;
}

// Op::GatherMatmul, crates/forja-core/src/ops.rs:254 (check :1749-1796): x [rows, inner], weights [experts, inner, cols],
// indices u32 [rows, routes] -> out [rows, routes, cols] in the activation dtype.
int32_t exec_gather_matmul(Exec& x, const fj_dispatch& d, fj::ErrorRecord* err) {
  if (d.n_inputs != 3 || d.n_outputs != 1) return FJ_INVALID_INPUT;
  const fj_tensor &a = d.inputs[0], &w = d.inputs[1], &idx = d.inputs[2], &o = d.outputs[0];
  if (a.rank != 2 || w.rank != 3 || idx.rank != 2 || o.rank != 3 || !is_float(a.dtype) || !is_float(w.dtype) || idx.dtype != FJ_U32 || o.dtype != a.dtype) return FJ_INVALID_INPUT;
  if (w.shape[1] != a.shape[1] || idx.shape[0] != a.shape[0] || o.shape[0] != a.shape[0] || o.shape[1] != idx.shape[1] || o.shape[2] != w.shape[2]) return FJ_INVALID_INPUT;
  View va, vw, vi, vo;
  if (!make_view(x.be, a, false, &va) || !make_view(x.be, w, false, &vw) || !make_view(x.be, idx, false, &vi) || !make_view(x.be, o, true, &vo)) return FJ_INVALID_INPUT;
  return fj::launch_gather_matmul(x.be->ctx, va, vw, vi, vo, err) ? FJ_OK : FJ_UNSUPPORTED_OPERATION;
}

int32_t exec_quant_matmul_plain(Exec& x, const fj_dispatch& d, float* acc_out);

int32_t exec_quant_matmul(Exec& x, const fj_dispatch& d) {
  if (d.program != 0) return with_epilogue(x, d, 4, [&](float* acc) { return exec_quant_matmul_plain(x, d, acc); });
  return exec_quant_matmul_plain(x, d, nullptr);
}

// acc_out != nullptr: the product goes to that contiguous f32 [m, n] area instead of the dispatch's output.
int32_t exec_quant_matmul_plain(Exec& x, const fj_dispatch& d, float* acc_out) {
  if (d.n_inputs < 4 || d.n_outputs != 1 || (acc_out == nullptr && d.n_inputs != 4) || !quant_params_ok(d.u0, d.u1)) return FJ_INVALID_INPUT;
  const fj_tensor &xt = d.inputs[0], &pk = d.inputs[1];
  if (xt.rank != 2 || pk.rank != 2 || pk.dtype != FJ_U32 || d.inputs[2].dtype != d.inputs[3].dtype || !is_float(xt.dtype)) return FJ_INVALID_INPUT;
  const unsigned m = xt.shape[0], k = xt.shape[1], n = pk.shape[0];
  if (pk.shape[1] != k * d.u0 / 32 || k % d.u1 != 0 || element_count(d.inputs[2]) != static_cast<uint64_t>(n) * (k / d.u1) || element_count(d.outputs[0]) != static_cast<uint64_t>(m) * n) return FJ_INVALID_INPUT;
  const void *xp = x.input(xt), *pp = x.input(pk), *sp = x.input(d.inputs[2]), *bp = x.input(d.inputs[3]);
  void* out = acc_out != nullptr ? static_cast<void*>(acc_out) : x.output(d.outputs[0]);
  const uint32_t out_dtype = acc_out != nullptr ? static_cast<uint32_t>(FJ_F32) : d.outputs[0].dtype;
  if (!xp || !pp || !sp || !bp || !out) return FJ_INVALID_INPUT;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  void* gemm_scratch = nullptr;
  size_t gemm_scratch_bytes = 0;
  if (m > 16 && xt.dtype != FJ_F32) {
    // slab of dequantised weights for the tensor-core path (at most 64 MiB) + split-K scratch
    workspace_bytes = std::min<size_t>(static_cast<size_t>(n) * k * 2, size_t(64) << 20);
    workspace_bytes = std::max<size_t>(workspace_bytes, static_cast<size_t>(k) * 64 * 2);
    workspace = x.temp(workspace_bytes);
    if (!workspace) return FJ_ALLOCATION_FAILED;
    const unsigned slab_cols = static_cast<unsigned>(std::min<size_t>(n, workspace_bytes / (static_cast<size_t>(k) * 2)));
    size_t need = fj::gemm_scratch_bytes(m, slab_cols, k);
    if (need <= (size_t(1) << 30) && ensure_gemm_scratch(x.be, need)) { gemm_scratch = x.be->gemm_scratch; gemm_scratch_bytes = x.be->gemm_scratch_bytes; }
  }
  fj::launch_quant_matmul(x.be->ctx, xp, xt.dtype, static_cast<const unsigned*>(pp), sp, bp, d.inputs[2].dtype, out, out_dtype, m, k, n, d.u0, d.u1, workspace,
                          workspace_bytes, gemm_scratch, gemm_scratch_bytes);
  return FJ_OK;
}

// From this many routes on, GatherQuantMatmul buckets the routes by expert: 16-row tiles that stream each active
// expert once while the average expert has fewer than kStreamRowsPerExpert rows, tile GEMMs (128 rows on tcgen05, weights
// rounded to bf16) beyond that.
constexpr uint64_t kGroupedRoutes = 64;
constexpr uint64_t kStreamRowsPerExpert = 72;

int32_t exec_gather_quant(Exec& x, const fj_dispatch& d, fj::ErrorRecord* err) {
  if (d.n_outputs != 1 || !quant_params_ok(d.u0, d.u1)) return FJ_INVALID_INPUT;
  int epilogue = 0;
  if (d.program != 0) {
    if (d.program > x.be->programs.size()) return FJ_INVALID_INPUT;
    const uint32_t kernel = x.be->programs[d.program - 1].kernel;
    if (kernel == 2) epilogue = 1; else if (kernel == 1) epilogue = 2; else return FJ_UNSUPPORTED_OPERATION;
  }
  const bool weighted = d.inputs[0].rank == 3 && (d.n_inputs == 6 || d.n_inputs == 7);
  if (weighted) {
    const fj_tensor &act = d.inputs[0], &pk = d.inputs[1], &idx = d.inputs[4], &wt = d.inputs[5];
    if (pk.rank != 3 || idx.dtype != FJ_U32 || pk.dtype != FJ_U32) return FJ_INVALID_INPUT;
    const unsigned rows = act.shape[0], routes = act.shape[1], k = act.shape[2], experts = pk.shape[0], n = pk.shape[1];
    if (pk.shape[2] != k * d.u0 / 32 || k % d.u1 != 0 || element_count(idx) != static_cast<uint64_t>(rows) * routes || element_count(wt) != element_count(idx) ||
        element_count(d.outputs[0]) != static_cast<uint64_t>(rows) * n) return FJ_INVALID_INPUT;
    if ((epilogue == 2) != (d.n_inputs == 7) || epilogue == 1) return FJ_INVALID_INPUT;
    const void *ap = x.input(act), *pp = x.input(pk), *sp = x.input(d.inputs[2]), *bp = x.input(d.inputs[3]), *ip = x.input(idx), *wp = x.input(wt);
    const void* ex = epilogue == 2 ? x.input(d.inputs[6]) : nullptr;
    void* out = x.output(d.outputs[0]);
    if (!ap || !pp || !sp || !bp || !ip || !wp || !out || (epilogue == 2 && !ex)) return FJ_INVALID_INPUT;
    if (epilogue == 2 && element_count(d.inputs[6]) != element_count(d.outputs[0])) return FJ_INVALID_INPUT;
    // many routes: bucket by expert, tile GEMMs into per-route f32 rows, then the ordered weighted sum
    const uint64_t total = static_cast<uint64_t>(rows) * routes;
    const bool bucket_ok = total >= kGroupedRoutes && total < (1u << 30) && act.dtype == FJ_BF16 && d.inputs[2].dtype == FJ_BF16;
    const bool stream = bucket_ok && total < kStreamRowsPerExpert * experts && fj::expert_stream_supported(k, n, d.u0, d.u1, experts, ap, pp, sp, bp);
    if (stream || (bucket_ok && fj::grouped_q4_supported(k, n, d.u0, d.u1, experts, ap, pp))) {
      void* plan = x.temp(fj::route_plan_bytes(static_cast<unsigned>(total), experts));
      float* per_route = static_cast<float*>(x.temp(total * n * sizeof(float)));
      if (!plan || !per_route) return FJ_ALLOCATION_FAILED;
      const unsigned tile_rows = stream ? 16 : fj::grouped_tile_rows(static_cast<unsigned>(total), experts);
      fj::launch_route_plan(x.be->ctx, static_cast<const unsigned*>(ip), static_cast<unsigned>(total), experts, plan, err, tile_rows);
      if (stream) {
        if (!fj::launch_expert_stream_single(x.be->ctx, ap, static_cast<const unsigned*>(pp), sp, bp, plan, static_cast<unsigned>(total), experts, 1, per_route, false, k, n))
          return FJ_DEVICE_EXECUTION_FAILED;
      } else fj::launch_grouped_q4_single(x.be->ctx, ap, static_cast<const unsigned*>(pp), sp, bp, plan, static_cast<unsigned>(total), experts, 1, per_route, false, k, n, tile_rows);
      fj::launch_routes_combine(x.be->ctx, per_route, FJ_F32, nullptr, static_cast<const unsigned*>(ip), experts, wp, wt.dtype, ex, epilogue == 2 ? d.inputs[6].dtype : 0, out,
                                d.outputs[0].dtype, rows, routes, n);
      return FJ_OK;
    }
    fj::launch_gather_quant_weighted_sum(x.be->ctx, ap, act.dtype, static_cast<const unsigned*>(pp), sp, bp, d.inputs[2].dtype, static_cast<const unsigned*>(ip), wp,
                                         wt.dtype, ex, epilogue == 2 ? d.inputs[6].dtype : 0, out, d.outputs[0].dtype, rows, routes, k, experts, n, d.u0, d.u1, epilogue, err);
    return FJ_OK;
  }
  if (d.n_inputs != 5 && d.n_inputs != 8) return FJ_INVALID_INPUT;
  const bool paired = d.n_inputs == 8;
  const fj_tensor &xt = d.inputs[0], &pk = d.inputs[1], &idx = d.inputs[paired ? 7 : 4];
  if (xt.rank != 2 || pk.rank != 3 || idx.rank != 2 || idx.dtype != FJ_U32) return FJ_INVALID_INPUT;
  const unsigned rows = xt.shape[0], k = xt.shape[1], experts = pk.shape[0], n = pk.shape[1], routes = idx.shape[1];
  if (pk.shape[2] != k * d.u0 / 32 || k % d.u1 != 0 || idx.shape[0] != rows || element_count(d.outputs[0]) != static_cast<uint64_t>(rows) * routes * n) return FJ_INVALID_INPUT;
  if ((paired && epilogue != 1) || (!paired && epilogue != 0)) return paired ? FJ_UNSUPPORTED_OPERATION : FJ_INVALID_INPUT;
  const void *xp = x.input(xt), *pp = x.input(pk), *sp = x.input(d.inputs[2]), *bp = x.input(d.inputs[3]), *ip = x.input(idx);
  const void *pp2 = nullptr, *sp2 = nullptr, *bp2 = nullptr;
  if (paired) { pp2 = x.input(d.inputs[4]); sp2 = x.input(d.inputs[5]); bp2 = x.input(d.inputs[6]); if (!pp2 || !sp2 || !bp2) return FJ_INVALID_INPUT; }
  void* out = x.output(d.outputs[0]);
  if (!xp || !pp || !sp || !bp || !ip || !out) return FJ_INVALID_INPUT;
  const uint64_t total = static_cast<uint64_t>(rows) * routes;
  const bool bucket_ok = total >= kGroupedRoutes && total < (1u << 30) && xt.dtype == FJ_BF16 && d.outputs[0].dtype == FJ_BF16 && d.inputs[2].dtype == FJ_BF16 &&
                         (!paired || d.inputs[5].dtype == FJ_BF16);
  const bool stream = bucket_ok && total < kStreamRowsPerExpert * experts && fj::expert_stream_supported(k, n, d.u0, d.u1, experts, xp, pp, sp, bp) &&
                      (!paired || fj::expert_stream_supported(k, n, d.u0, d.u1, experts, xp, pp2, sp2, bp2));
  if (stream || (bucket_ok && fj::grouped_q4_supported(k, n, d.u0, d.u1, experts, xp, pp) && (!paired || reinterpret_cast<size_t>(pp2) % 16 == 0))) {
    // routes with an out-of-range expert id belong to no bucket: their rows stay zero and the lowest id is reported
    void* plan = x.temp(fj::route_plan_bytes(static_cast<unsigned>(total), experts));
    if (!plan) return FJ_ALLOCATION_FAILED;
    cudaMemsetAsync(out, 0, total * n * 2, x.be->stream);
    const unsigned tile_rows = stream ? 16 : fj::grouped_tile_rows(static_cast<unsigned>(total), experts);
    fj::launch_route_plan(x.be->ctx, static_cast<const unsigned*>(ip), static_cast<unsigned>(total), experts, plan, err, tile_rows);
    if (stream) {
      const bool ok = paired ? fj::launch_expert_stream_pair(x.be->ctx, xp, static_cast<const unsigned*>(pp), sp, bp, static_cast<const unsigned*>(pp2), sp2, bp2, plan,
                                                             static_cast<unsigned>(total), experts, routes, out, k, n)
                             : fj::launch_expert_stream_single(x.be->ctx, xp, static_cast<const unsigned*>(pp), sp, bp, plan, static_cast<unsigned>(total), experts, routes, out, true, k, n);
      if (!ok) return FJ_DEVICE_EXECUTION_FAILED;
    } else if (paired)
      fj::launch_grouped_q4_pair(x.be->ctx, xp, static_cast<const unsigned*>(pp), sp, bp, static_cast<const unsigned*>(pp2), sp2, bp2, plan, static_cast<unsigned>(total), experts, routes,
                                 out, k, n, tile_rows);
    else
      fj::launch_grouped_q4_single(x.be->ctx, xp, static_cast<const unsigned*>(pp), sp, bp, plan, static_cast<unsigned>(total), experts, routes, out, true, k, n, tile_rows);
    return FJ_OK;
  }
  fj::launch_gather_quant_matmul(x.be->ctx, xp, xt.dtype, static_cast<const unsigned*>(pp), sp, bp, d.inputs[2].dtype, static_cast<const unsigned*>(pp2), sp2, bp2,
                                 static_cast<const unsigned*>(ip), out, d.outputs[0].dtype, rows, k, experts, n, routes, d.u0, d.u1, epilogue, err);
  return FJ_OK;
}

int32_t exec_paged_copy(Exec& x, const fj_dispatch& d, fj::ErrorRecord* err) {
  if ((d.n_inputs != 3 && d.n_inputs != 4) || d.n_outputs != 1) return FJ_INVALID_INPUT;
  const bool into = d.u0 == 0;
  const fj_tensor& pool = into ? d.outputs[0] : d.inputs[0];
  const fj_tensor& ordinary = into ? d.inputs[0] : d.outputs[0];
  const fj_tensor &table = d.inputs[1], &gens = d.inputs[2];
  if (pool.rank != 3 || !is_contiguous(pool) || table.dtype != FJ_U32 || gens.dtype != FJ_U32 || !is_contiguous(table) || !is_contiguous(gens)) return FJ_INVALID_INPUT;
  const unsigned page_tokens = d.u2, physical = pool.shape[0], elements = pool.shape[2];
  if (page_tokens == 0 || pool.shape[1] != page_tokens || ordinary.rank == 0) return FJ_INVALID_INPUT;
  const unsigned tokens = ordinary.shape[0];
  if (element_count(ordinary) != static_cast<uint64_t>(tokens) * elements || element_count(gens) != physical || element_count(table) % 2 != 0) return FJ_INVALID_INPUT;
  if (static_cast<uint64_t>(d.u1) + tokens > 0xFFFFFFFFull) return FJ_INVALID_INPUT;
  void* pp = tensor_ptr(x.be, pool, into);
  const unsigned* tp = static_cast<const unsigned*>(tensor_ptr(x.be, table, false));
  const unsigned* gp = static_cast<const unsigned*>(tensor_ptr(x.be, gens, false));
  const unsigned* act = d.n_inputs == 4 ? static_cast<const unsigned*>(tensor_ptr(x.be, d.inputs[3], false)) : nullptr;
  void* op = into ? const_cast<void*>(x.input(ordinary)) : x.output(ordinary);
  if (!pp || !tp || !gp || !op || (d.n_inputs == 4 && !act)) return FJ_INVALID_INPUT;
  fj::launch_paged_copy(x.be->ctx, into, op, ordinary.dtype, elements, pp, pool.dtype, tp, static_cast<unsigned>(element_count(table) / 2), gp, physical, d.u1, tokens,
                        page_tokens, elements, act, err);
  return FJ_OK;
}

bool ranges_overlap(fj_backend* be, const fj_tensor& a, const fj_tensor& b) {
  if (a.buffer != b.buffer) return false;
  uint64_t al, ah, bl, bh;
  // a view whose span cannot be computed is refused by tensor_ptr before anything runs; calling it
  // a hazard here only keeps it out of a coalesced run
  if (!tensor_byte_span(a, &al, &ah) || !tensor_byte_span(b, &bl, &bh)) return true;
  (void)be;
  return al < bh && bl < ah;
}

// Executes a run [first, first + count) of PagedSdpa / PagedSdpaAppend dispatches that share
// planes and geometry as ONE ragged attention launch (after per-lane appends for the Append op).
int32_t exec_paged_attention_run(Exec& x, const fj_dispatch* ds, uint32_t count, fj::ErrorRecord* err) {
  const fj_dispatch& d0 = ds[0];
  const bool append = d0.op == FJ_OP_PAGED_SDPA_APPEND;
  const fj_tensor& kpool = append ? d0.outputs[1] : d0.inputs[1];
  const fj_tensor& vpool = append ? d0.outputs[2] : d0.inputs[2];
  if (kpool.rank != 4 || vpool.rank != 4 || !is_contiguous(kpool) || !is_contiguous(vpool)) return FJ_INVALID_INPUT;
  fj::AttnGeometry g;
  g.kv_heads = kpool.shape[2]; g.head_dim = kpool.shape[3]; g.value_dim = vpool.shape[3]; g.page_tokens = d0.u3; g.physical_pages = kpool.shape[0];
  g.q_heads = d0.inputs[0].shape[0]; g.q_dtype = d0.inputs[0].dtype; g.kv_dtype = kpool.dtype; g.out_dtype = d0.outputs[0].dtype; g.scale = d0.f0;
  if (g.page_tokens == 0 || kpool.shape[1] != g.page_tokens || vpool.shape[1] != g.page_tokens || vpool.shape[0] != g.physical_pages || vpool.shape[2] != g.kv_heads ||
      vpool.dtype != kpool.dtype || g.kv_heads == 0 || g.q_heads % g.kv_heads != 0 || !isfinite(g.scale) || g.head_dim > 256 || g.value_dim > 256) return FJ_INVALID_INPUT;
  void* kp = tensor_ptr(x.be, kpool, append);
  void* vp = tensor_ptr(x.be, vpool, append);
  if (!kp || !vp) return FJ_INVALID_INPUT;
  const fj_tensor& gens0 = d0.inputs[4];
  const unsigned* gp = static_cast<const unsigned*>(tensor_ptr(x.be, gens0, false));
  if (!gp || gens0.dtype != FJ_U32 || element_count(gens0) != g.physical_pages || !is_contiguous(gens0)) return FJ_INVALID_INPUT;

  std::vector<fj::AttnSeq> seqs(count);
  std::vector<fj::AppendLane> appends(append ? count : 0);
  unsigned max_q_len = 0;
  for (uint32_t i = 0; i < count; ++i) {
    const fj_dispatch& d = ds[i];
    const fj_tensor &q = d.inputs[0], &table = d.inputs[3], &out = d.outputs[0];
    if (q.rank != 3 || out.rank != 3 || q.shape[0] != g.q_heads || q.shape[2] != g.head_dim || out.shape[0] != g.q_heads || out.shape[1] != q.shape[1] || out.shape[2] != g.value_dim)
      return FJ_INVALID_INPUT;
    if (q.strides[2] != 1 || out.strides[2] != 1 || table.dtype != FJ_U32 || !is_contiguous(table) || element_count(table) % 2 != 0) return FJ_INVALID_INPUT;
    const bool has_activity = d.n_inputs == 6;
    fj::AttnSeq& s = seqs[i];
    s.q = tensor_ptr(x.be, q, false);
    s.out = tensor_ptr(x.be, out, true);
    s.table = static_cast<const unsigned*>(tensor_ptr(x.be, table, false));
    s.activity = has_activity ? static_cast<const unsigned*>(tensor_ptr(x.be, d.inputs[5], false)) : nullptr;
    if (!s.q || !s.out || !s.table || (has_activity && !s.activity)) return FJ_INVALID_INPUT;
    s.q_len = q.shape[1];
    s.q_start = d.u1;
    s.table_pages = static_cast<unsigned>(element_count(table) / 2);
    s.causal = append ? 1 : (d.u0 ? 1 : 0);
    if (append) {
      if (d.u1 == 0xFFFFFFFFu || s.q_len != 1) return FJ_INVALID_INPUT;
      s.key_length = d.u1 + 1;
    } else {
      s.key_length = d.u2;
    }
    s.q_tok_stride = q.strides[1]; s.q_head_stride = q.strides[0]; s.o_tok_stride = out.strides[1]; s.o_head_stride = out.strides[0];
    s.err_index = i;  // every lane reports to the record of its own dispatch
    max_q_len = std::max(max_q_len, s.q_len);
    if (append) {
      // PagedCopy of the new K and V rows at q_start (crates/forja-cpu/src/lib.rs:272-290)
      const fj_tensor &kn = d.inputs[1], &vn = d.inputs[2];
      const void* knp = x.input(kn);
      const void* vnp = x.input(vn);
      if (!knp || !vnp || element_count(kn) != static_cast<uint64_t>(g.kv_heads) * g.head_dim || element_count(vn) != static_cast<uint64_t>(g.kv_heads) * g.value_dim) return FJ_INVALID_INPUT;
      if (!is_float(kn.dtype) || !is_float(vn.dtype)) return FJ_INVALID_INPUT;
      appends[i] = fj::AppendLane{knp, vnp, s.table, s.activity, s.table_pages, d.u1, i, static_cast<int>(kn.dtype), static_cast<int>(vn.dtype)};
    }
  }
  if (append) {
    // the new K and V rows of every lane go into their pages in one launch (one validate + copy pair per lane before)
    fj::AppendLane* dev_appends = x.upload(appends);
    if (!dev_appends) return FJ_ALLOCATION_FAILED;
    fj::launch_paged_append_batch(x.be->ctx, dev_appends, count, kp, vp, kpool.dtype, gp, g.physical_pages, g.page_tokens, g.kv_heads * g.head_dim, g.kv_heads * g.value_dim, err);
  }
  fj::AttnSeq* dev_seqs = x.upload(seqs);
  if (!dev_seqs) return FJ_ALLOCATION_FAILED;

  bool mma = fj::attn_decode_mma_supported(g, max_q_len);
  if (mma) {
    for (auto& s : seqs) {
      if ((reinterpret_cast<size_t>(s.q) & 3) || (s.q_tok_stride & 1) || (s.q_head_stride & 1)) mma = false;
    }
  }
  if (!mma) {
    // longer query runs (prefill chunks): 128-row tensor-core blocks when the shape allows, else the f32 kernel
    bool blocks = fj::attn_prefill_mma_supported(g);
    for (auto& s : seqs) {
      if ((reinterpret_cast<size_t>(s.q) & 3) || (s.q_tok_stride & 1) || (s.q_head_stride & 1)) blocks = false;
    }
    if (blocks) {
      const unsigned per_block = fj::attn_prefill_tokens_per_block(g);
      std::vector<uint2> items;
      for (uint32_t i = 0; i < count; ++i)
        for (unsigned t = 0; t < seqs[i].q_len; t += per_block) items.push_back(make_uint2(i, t));
      uint2* dev_items = x.upload(items);
      if (!dev_items) return FJ_ALLOCATION_FAILED;
      fj::launch_attn_prefill_mma(x.be->ctx, g, dev_seqs, dev_items, static_cast<unsigned>(items.size()), kp, vp, gp, err);
      return FJ_OK;
    }
    fj::launch_attn_generic(x.be->ctx, g, dev_seqs, count, max_q_len, kp, vp, gp, err);
    return FJ_OK;
  }
  // split-K work list: chunks of `chunk` tokens per (lane, kv head), sized to fill the GPU
  uint64_t total_tokens = 0;
  for (auto& s : seqs) total_tokens += s.key_length;
  const uint64_t target_items = static_cast<uint64_t>(x.be->ctx.sm_count) * 2 * 4;
  uint64_t chunk = (total_tokens * g.kv_heads + target_items - 1) / std::max<uint64_t>(target_items, 1);
  chunk = std::min<uint64_t>(std::max<uint64_t>((chunk + 63) / 64 * 64, 64), 1024);
  // the work list itself is built on the device from the lane descriptors; the host only needs its length
  uint64_t n_work = 0;
  for (uint32_t i = 0; i < count; ++i) {
    const unsigned len = seqs[i].key_length;
    n_work += (len == 0 ? 1 : (len + chunk - 1) / chunk) * g.kv_heads;
  }
  if (n_work > (1u << 24)) return FJ_QUOTA_EXCEEDED;
  const unsigned groups = count * g.kv_heads;
  const size_t o_bytes = fj::attn_part_o_bytes(static_cast<unsigned>(n_work), g.head_dim), ml_bytes = fj::attn_part_ml_bytes(static_cast<unsigned>(n_work));
  const size_t counter_bytes = (static_cast<size_t>(groups) * sizeof(unsigned) + 255) / 256 * 256;
  if (!ensure_attn_scratch(x.be, counter_bytes + o_bytes + ml_bytes)) return FJ_ALLOCATION_FAILED;
  fj::AttnScratch scratch;
  scratch.counters = static_cast<unsigned*>(x.be->attn_scratch);
  scratch.part_o = reinterpret_cast<float*>(static_cast<char*>(x.be->attn_scratch) + counter_bytes);
  scratch.part_ml = reinterpret_cast<float*>(static_cast<char*>(x.be->attn_scratch) + counter_bytes + o_bytes);
  fj::AttnWork* dev_work = static_cast<fj::AttnWork*>(x.temp(static_cast<size_t>(n_work) * sizeof(fj::AttnWork)));
  if (!dev_work) return FJ_ALLOCATION_FAILED;
  fj::launch_build_work_from_seqs(x.be->ctx, dev_seqs, count, g.kv_heads, static_cast<unsigned>(chunk), dev_work, static_cast<unsigned>(n_work));
  fj::launch_attn_decode_mma(x.be->ctx, g, dev_seqs, dev_work, static_cast<unsigned>(n_work), kp, vp, gp, scratch, err);
  return FJ_OK;
}

bool paged_run_compatible(fj_backend* be, const fj_dispatch& a, const fj_dispatch& b) {
  if (a.op != b.op || a.n_inputs != b.n_inputs || a.n_outputs != b.n_outputs) return false;
  const bool append = a.op == FJ_OP_PAGED_SDPA_APPEND;
  const fj_tensor &ka = append ? a.outputs[1] : a.inputs[1], &kb = append ? b.outputs[1] : b.inputs[1];
  const fj_tensor &va = append ? a.outputs[2] : a.inputs[2], &vb = append ? b.outputs[2] : b.inputs[2];
  if (ka.buffer != kb.buffer || ka.offset != kb.offset || va.buffer != vb.buffer || va.offset != vb.offset) return false;
  if (a.inputs[4].buffer != b.inputs[4].buffer || a.inputs[4].offset != b.inputs[4].offset) return false;
  if (memcmp(&a.f0, &b.f0, 4) != 0 || a.u3 != b.u3) return false;
  if (a.inputs[0].rank != 3 || b.inputs[0].rank != 3 || a.inputs[0].shape[0] != b.inputs[0].shape[0] || a.inputs[0].shape[2] != b.inputs[0].shape[2]) return false;
  if (a.inputs[0].dtype != b.inputs[0].dtype || a.outputs[0].dtype != b.outputs[0].dtype) return false;
  (void)be;
  return true;
}

int32_t exec_program(Exec& x, const fj_dispatch& d) {
  if (d.program == 0 || d.program > x.be->programs.size()) return FJ_INVALID_INPUT;
  const fj_program_rec& rec = x.be->programs[d.program - 1];
  if (d.n_outputs == 0) return FJ_INVALID_INPUT;
  const fj_tensor& shape_of = d.outputs[0];
  for (uint32_t i = 0; i < d.n_inputs; ++i) if (!same_shape(d.inputs[i], shape_of)) return FJ_INVALID_INPUT;
  for (uint32_t i = 0; i < d.n_outputs; ++i) if (!same_shape(d.outputs[i], shape_of)) return FJ_INVALID_INPUT;
  const uint64_t n = element_count(shape_of);
  if (n == 0) return FJ_OK;
  const unsigned width = shape_of.rank ? shape_of.shape[shape_of.rank - 1] : 1;
  View in[5], out[2];
  for (uint32_t i = 0; i < d.n_inputs && i < 5; ++i) if (!make_view(x.be, d.inputs[i], false, &in[i])) return FJ_INVALID_INPUT;
  for (uint32_t i = 0; i < d.n_outputs && i < 2; ++i) if (!make_view(x.be, d.outputs[i], true, &out[i])) return FJ_INVALID_INPUT;
  switch (rec.kernel) {
    case 1: if (d.n_inputs != 2 || d.n_outputs != 1) return FJ_INVALID_INPUT; fj::launch_add(x.be->ctx, in[0], in[1], out[0], n); return FJ_OK;
    case 2: if (d.n_inputs != 2 || d.n_outputs != 1) return FJ_INVALID_INPUT; fj::launch_silu_mul(x.be->ctx, in[0], in[1], out[0], n); return FJ_OK;
    case 3: if (d.n_inputs != 2 || d.n_outputs != 1) return FJ_INVALID_INPUT; fj::launch_rms_norm(x.be->ctx, in[0], in[1], out[0], n / width, width, rec.eps); return FJ_OK;
    case 4: if (d.n_inputs != 3 || d.n_outputs != 2) return FJ_INVALID_INPUT; fj::launch_residual_norm(x.be->ctx, in[0], in[1], in[2], out[0], out[1], n / width, width, rec.eps); return FJ_OK;
    case 5: {
      if (d.n_inputs != 5 || d.n_outputs != 2) return FJ_INVALID_INPUT;
      const float* table = freq_table(x.be, rec.theta, rec.exponent_scale, width, false);
      if (!table) return FJ_ALLOCATION_FAILED;
      fj::launch_qk_norm_rope(x.be->ctx, in[0], in[1], in[2], in[3], in[4], out[0], out[1], n / width, width, rec.head_dim, rec.eps, table);
      return FJ_OK;
    }
    case 6: {
      if (d.n_inputs != 3 || d.n_outputs != 2) return FJ_INVALID_INPUT;
      const float* table = freq_table(x.be, rec.theta, rec.exponent_scale, width, false);
      if (!table) return FJ_ALLOCATION_FAILED;
      fj::launch_rope_pairs(x.be->ctx, in[0], in[1], in[2], out[0], out[1], n, width, table);
      return FJ_OK;
    }
    default: return FJ_UNSUPPORTED_OPERATION;
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------

extern "C" {

int32_t fj_backend_create(int32_t device, uint64_t memory_limit, fj_backend** out) {
  if (out == nullptr) return FJ_INVALID_INPUT;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) { cudaGetLastError(); return FJ_ALLOCATION_FAILED; }
  if (cudaSetDevice(device) != cudaSuccess) return FJ_ALLOCATION_FAILED;
  auto* be = new fj_backend();
  be->device = device;
  be->limit_bytes = memory_limit;
  if (cudaGetDeviceProperties(&be->prop, device) != cudaSuccess || cudaStreamCreateWithFlags(&be->stream, cudaStreamNonBlocking) != cudaSuccess) { delete be; return FJ_ALLOCATION_FAILED; }
  be->ctx.stream = be->stream;
  be->ctx.launches = 0;
  be->ctx.sm_count = be->prop.multiProcessorCount;
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
    uint64_t threshold = ~0ull;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold);
  }
  *out = be;
  return FJ_OK;
}

void fj_backend_destroy(fj_backend* be) {
  if (!be) return;
  cudaSetDevice(be->device);
  cudaStreamSynchronize(be->stream);
  for (auto& kv : be->buffers) cudaFree(kv.second.ptr);
  for (auto& kv : be->freq_tables) cudaFree(kv.second);
  for (auto e : be->timers) cudaEventDestroy(e);
  for (auto& block : be->pinned_pool) cudaFreeHost(block.first);
  if (be->gemm_scratch) cudaFree(be->gemm_scratch);
  if (be->attn_scratch) cudaFree(be->attn_scratch);
  cudaStreamDestroy(be->stream);
  delete be;
}

int32_t fj_device_info(fj_backend* be, fj_device_info_t* out) {
  if (!be || !out) return FJ_INVALID_INPUT;
  memset(out, 0, sizeof(*out));
  strncpy(out->name, be->prop.name, sizeof(out->name) - 1);
  out->sm_count = be->prop.multiProcessorCount;
  out->cc_major = be->prop.major; out->cc_minor = be->prop.minor;
  out->total_memory = be->prop.totalGlobalMem;
  out->l2_bytes = be->prop.l2CacheSize;
  out->max_smem_per_block = static_cast<uint32_t>(be->prop.sharedMemPerBlockOptin);
  return FJ_OK;
}

int32_t fj_set_memory_limit(fj_backend* be, uint64_t bytes) {
  if (!be) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  if (bytes != 0 && bytes < be->used_bytes) return FJ_QUOTA_EXCEEDED;
  be->limit_bytes = bytes;
  return FJ_OK;
}
int32_t fj_memory_usage(fj_backend* be, uint64_t* used, uint64_t* limit) {
  if (!be) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  if (used) *used = be->used_bytes;
  if (limit) *limit = be->limit_bytes;
  return FJ_OK;
}

int32_t fj_alloc(fj_backend* be, uint64_t bytes, uint64_t* buffer) {
  if (!be || !buffer) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  return alloc_buffer(be, bytes, buffer);
}

int32_t fj_import_readonly(fj_backend* be, const void* host, uint64_t bytes, uint64_t* buffer) {
  if (!be || !buffer || (bytes && !host)) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  int32_t st = alloc_buffer(be, bytes, buffer);
  if (st != FJ_OK) return st;
  fj_buffer_rec* rec = find_buffer(be, *buffer);
  if (bytes && cudaMemcpyAsync(rec->ptr, host, bytes, cudaMemcpyHostToDevice, be->stream) != cudaSuccess) return FJ_EXECUTION_FAILED;
  if (cudaStreamSynchronize(be->stream) != cudaSuccess) return FJ_EXECUTION_FAILED;
  rec->readonly = true;
  return FJ_OK;
}

int32_t fj_release(fj_backend* be, uint64_t buffer) {
  if (!be) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  fj_buffer_rec* rec = find_buffer(be, buffer);
  if (!rec) return FJ_INVALID_INPUT;
  cudaSetDevice(be->device);
  cudaStreamSynchronize(be->stream);  // submitted work may still read the allocation
  cudaFree(rec->ptr);
  be->used_bytes -= rec->bytes;
  be->buffers.erase(buffer);
  return FJ_OK;
}

int32_t fj_write(fj_backend* be, uint64_t buffer, uint64_t byte_offset, const void* src, uint64_t len) {
  if (!be || (len && !src)) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  fj_buffer_rec* rec = find_buffer(be, buffer);
  if (!rec || rec->readonly || byte_offset > rec->bytes || len > rec->bytes - byte_offset) return FJ_INVALID_INPUT;
  if (len == 0) return FJ_OK;
  cudaSetDevice(be->device);
  if (cudaMemcpyAsync(static_cast<char*>(rec->ptr) + byte_offset, src, len, cudaMemcpyHostToDevice, be->stream) != cudaSuccess) return FJ_EXECUTION_FAILED;
  return cuda_status(cudaStreamSynchronize(be->stream));
}

int32_t fj_read(fj_backend* be, uint64_t buffer, uint64_t byte_offset, void* dst, uint64_t len) {
  if (!be || (len && !dst)) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  fj_buffer_rec* rec = find_buffer(be, buffer);
  if (!rec || byte_offset > rec->bytes || len > rec->bytes - byte_offset) return FJ_INVALID_INPUT;
  if (len == 0) return FJ_OK;
  cudaSetDevice(be->device);
  if (cudaMemcpyAsync(dst, static_cast<char*>(rec->ptr) + byte_offset, len, cudaMemcpyDeviceToHost, be->stream) != cudaSuccess) return FJ_EXECUTION_FAILED;
  return cuda_status(cudaStreamSynchronize(be->stream));
}

int32_t fj_read_strided(fj_backend* be, const fj_tensor* view, void* dst) {
  if (!be || !view || !dst) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  const uint64_t n = element_count(*view);
  if (n == 0) return FJ_OK;
  Exec x{be};
  const void* p = x.input(*view);
  if (!p) return FJ_INVALID_INPUT;
  cudaError_t e = cudaMemcpyAsync(dst, p, n * fj::dtype_size(view->dtype), cudaMemcpyDeviceToHost, be->stream);
  for (void* t : x.temps) cudaFreeAsync(t, be->stream);
  if (e != cudaSuccess) return FJ_EXECUTION_FAILED;
  return cuda_status(cudaStreamSynchronize(be->stream));
}

int32_t fj_buffer_device_ptr(fj_backend* be, uint64_t buffer, void** ptr, uint64_t* bytes) {
  if (!be || !ptr) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  fj_buffer_rec* rec = find_buffer(be, buffer);
  if (!rec) return FJ_INVALID_INPUT;
  *ptr = rec->ptr;
  if (bytes) *bytes = rec->bytes;
  return FJ_OK;
}

int32_t fj_program_prepare(fj_backend* be, uint32_t kind, const uint32_t* insts, uint32_t n_insts, const uint32_t* outputs, uint32_t n_outputs, uint64_t* handle) {
  if (!be || !insts || !outputs || !handle || kind > 1) return FJ_INVALID_INPUT;
  if (n_insts == 0 || n_insts > 256 || n_outputs == 0 || n_outputs > 4) return FJ_INVALID_INPUT;  // program.rs:25-31
  fj_program_rec rec;
  if (!recognise(kind, insts, n_insts, outputs, n_outputs, &rec)) return FJ_UNSUPPORTED_OPERATION;
  std::lock_guard<std::mutex> lock(be->mutex);
  be->programs.push_back(rec);
  *handle = be->programs.size();
  return FJ_OK;
}

int32_t fj_tensor_byte_span(const fj_tensor* view, uint64_t* lo, uint64_t* hi) {
  if (view == nullptr || lo == nullptr || hi == nullptr) return FJ_INVALID_INPUT;
  return tensor_byte_span(*view, lo, hi) ? FJ_OK : FJ_INVALID_INPUT;
}

int32_t fj_program_classify(uint32_t kind, const uint32_t* insts, uint32_t n_insts, const uint32_t* outputs, uint32_t n_outputs, uint32_t* kernel, float consts[4]) {
  if (!insts || !outputs || kind > 1 || n_insts == 0 || n_insts > 256 || n_outputs == 0 || n_outputs > 4) return FJ_INVALID_INPUT;
  fj_program_rec r;
  if (!recognise(kind, insts, n_insts, outputs, n_outputs, &r)) return FJ_UNSUPPORTED_OPERATION;
  if (kernel) *kernel = r.kernel;
  if (consts) { consts[0] = r.eps; consts[1] = r.theta; consts[2] = r.head_dim; consts[3] = r.exponent_scale; }
  return FJ_OK;
}

int32_t fj_program_info(fj_backend* be, uint64_t handle, uint32_t* kernel, float consts[4]) {
  if (!be) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  if (handle == 0 || handle > be->programs.size()) return FJ_INVALID_INPUT;
  const fj_program_rec& r = be->programs[handle - 1];
  if (kernel) *kernel = r.kernel;
  if (consts) { consts[0] = r.eps; consts[1] = r.theta; consts[2] = r.head_dim; consts[3] = r.exponent_scale; }
  return FJ_OK;
}

// Algorithmic traffic and arithmetic of one dispatch, the reference's KernelCost (crates/forja-core/src/cost.rs:109-153:
// logical operand bytes read and written, 2 flops per multiply-add; attention per cost/attention.rs:38-137: the K/V rows
// actually attended, 12 bytes of table and generation per page touched, the causal triangle of (query, key) pairs;
// paged copies per :96-121). Saturates instead of overflowing.
static void dispatch_cost(const fj_dispatch& d, uint64_t* read_bytes, uint64_t* write_bytes, uint64_t* flops) {
  auto sat_mul = [](uint64_t a, uint64_t b) { uint64_t r; return __builtin_mul_overflow(a, b, &r) ? ~0ull : r; };
  auto sat_add = [](uint64_t a, uint64_t b) { uint64_t r; return __builtin_add_overflow(a, b, &r) ? ~0ull : r; };
  auto tensor_bytes = [&](const fj_tensor& t) { uint64_t n = 1; for (uint32_t a = 0; a < t.rank && a < 8; ++a) n = sat_mul(n, t.shape[a]); return sat_mul(n, fj::dtype_size(static_cast<int>(t.dtype > FJ_U32 ? FJ_U32 : t.dtype))); };
  uint64_t rd = 0, wr = 0, fl = 0;
  for (uint32_t i = 0; i < d.n_inputs; ++i) rd = sat_add(rd, tensor_bytes(d.inputs[i]));
  for (uint32_t i = 0; i < d.n_outputs; ++i) wr = sat_add(wr, tensor_bytes(d.outputs[i]));
  const auto pages_touched = [&](uint64_t start, uint64_t tokens, uint64_t page) { return tokens == 0 || page == 0 ? 0ull : (start + tokens - 1) / page - start / page + 1; };
  switch (d.op) {
    case FJ_OP_MATMUL:
      if (d.n_inputs == 2 && d.inputs[0].rank >= 2 && d.inputs[1].rank == d.inputs[0].rank) {
        const fj_tensor &a = d.inputs[0], &b = d.inputs[1];
        uint64_t batch = a.rank == 3 ? a.shape[0] : 1;
        fl = sat_mul(sat_mul(2 * batch, a.shape[a.rank - 2]), sat_mul(a.shape[a.rank - 1], b.shape[b.rank - 1]));
      }
      break;
    case FJ_OP_QUANT_MATMUL:
      if (d.n_inputs == 4 && d.inputs[0].rank == 2 && d.inputs[1].rank == 2) fl = sat_mul(sat_mul(2ull * d.inputs[0].shape[0], d.inputs[0].shape[1]), d.inputs[1].shape[0]);
      break;
    case FJ_OP_GATHER_MATMUL:
      if (d.n_inputs == 3 && d.inputs[0].rank == 2 && d.inputs[1].rank == 3 && d.inputs[2].rank == 2)
        fl = sat_mul(sat_mul(2ull * d.inputs[0].shape[0], d.inputs[2].shape[1]), sat_mul(d.inputs[1].shape[1], d.inputs[1].shape[2]));
      break;
    case FJ_OP_GATHER_QUANT_MATMUL:
      if (d.n_inputs >= 5 && d.n_outputs == 1 && d.inputs[1].rank == 3) {  // routes x (rows of one expert matrix x inner), per projection
        const fj_tensor& idx = d.inputs[d.n_inputs == 8 ? 7 : 4];
        const uint64_t routes = idx.rank == 2 ? static_cast<uint64_t>(idx.shape[0]) * idx.shape[1] : 0;
        const uint64_t inner = static_cast<uint64_t>(d.inputs[1].shape[2]) * 32 / (d.u0 ? d.u0 : 4);
        fl = sat_mul(sat_mul(2 * routes, d.inputs[1].shape[1]), inner) * (d.n_inputs == 8 ? 2 : 1);
      }
      break;
    case FJ_OP_PAGED_COPY:
      if (d.n_inputs >= 3 && d.n_outputs == 1) {
        const bool into = d.u0 == 0;
        const fj_tensor& ordinary = into ? d.inputs[0] : d.outputs[0];
        const fj_tensor& pool = into ? d.outputs[0] : d.inputs[0];
        uint64_t elements = 1;
        for (uint32_t a = 0; a < ordinary.rank && a < 8; ++a) elements = sat_mul(elements, ordinary.shape[a]);
        const uint64_t pool_bytes = sat_mul(elements, fj::dtype_size(static_cast<int>(pool.dtype)));
        rd = into ? tensor_bytes(ordinary) : pool_bytes;
        wr = into ? pool_bytes : tensor_bytes(ordinary);
        rd = sat_add(rd, 12 * pages_touched(d.u1, ordinary.rank ? ordinary.shape[0] : 0, d.u2) + (d.n_inputs == 4 ? 4 : 0));
      }
      break;
    case FJ_OP_SDPA:
    case FJ_OP_PAGED_SDPA:
    case FJ_OP_PAGED_SDPA_APPEND:
      if (d.n_inputs >= 3 && d.n_outputs >= 1 && d.inputs[0].rank == 3) {
        const bool paged = d.op != FJ_OP_SDPA, append = d.op == FJ_OP_PAGED_SDPA_APPEND;
        const fj_tensor& key = append ? d.outputs[1] : d.inputs[1];
        const fj_tensor& value = append ? d.outputs[2] : d.inputs[2];
        if ((paged && (key.rank != 4 || value.rank != 4)) || (!paged && (key.rank != 3 || value.rank != 3))) break;
        const uint64_t heads = d.inputs[0].shape[0], queries = d.inputs[0].shape[1], width = d.inputs[0].shape[2];
        const uint64_t value_width = value.shape[value.rank - 1], kv_heads = key.shape[paged ? 2 : 0];
        const uint64_t q_start = d.u1;
        const bool causal = append || d.u0 != 0;
        const uint64_t key_length = append ? q_start + 1 : (paged ? d.u2 : key.shape[1]);
        const uint64_t pairs = causal ? sat_add(sat_mul(queries, q_start + 1), queries ? queries * (queries - 1) / 2 : 0) : sat_mul(queries, key_length);
        fl = sat_mul(sat_mul(2 * heads, pairs), width + value_width);
        const uint64_t kv_bytes = sat_mul(sat_mul(kv_heads, key_length), sat_mul(width + value_width, fj::dtype_size(static_cast<int>(key.dtype))));
        rd = sat_add(tensor_bytes(d.inputs[0]), kv_bytes);
        wr = tensor_bytes(d.outputs[0]);
        if (paged) rd = sat_add(rd, 12 * pages_touched(0, key_length, d.u3) + (d.n_inputs == 6 ? 4 : 0));
        if (append) {
          rd = sat_add(rd, sat_add(tensor_bytes(d.inputs[1]), tensor_bytes(d.inputs[2])));
          for (int i = 1; i <= 2; ++i) {
            uint64_t elements = 1;
            for (uint32_t a = 0; a < d.inputs[i].rank && a < 8; ++a) elements = sat_mul(elements, d.inputs[i].shape[a]);
            wr = sat_add(wr, sat_mul(elements, fj::dtype_size(static_cast<int>(d.outputs[i].dtype))));
          }
        }
      }
      break;
    default: break;
  }
  *read_bytes = rd; *write_bytes = wr; *flops = fl;
}

int32_t fj_submit(fj_backend* be, const fj_dispatch* dispatches, uint32_t count, uint32_t profiled, fj_submission** out) {
  if (!be || !out || (count && !dispatches)) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  auto* sub = new fj_submission();
  sub->be = be;
  sub->serial = be->next_serial++;
  sub->count = count;
  sub->ops.resize(count);
  sub->kernels.assign(count, 0);
  cudaEventCreate(&sub->start);
  cudaEventCreate(&sub->stop);
  Exec x{be};
  const unsigned long long launches_before = be->ctx.launches;
  if (count) {
    {
      std::lock_guard<std::mutex> pinned(be->pinned_mutex);
      for (size_t i = 0; i < be->pinned_pool.size(); ++i) {
        if (be->pinned_pool[i].second >= count) {
          sub->host_err = static_cast<fj::ErrorRecord*>(be->pinned_pool[i].first);
          sub->host_err_capacity = be->pinned_pool[i].second;
          be->pinned_pool.erase(be->pinned_pool.begin() + i);
          break;
        }
      }
    }
    if (!sub->host_err) {
      sub->host_err_capacity = std::max<size_t>(count, 64);
      if (cudaMallocHost(reinterpret_cast<void**>(&sub->host_err), sub->host_err_capacity * sizeof(fj::ErrorRecord)) != cudaSuccess) { cudaGetLastError(); sub->host_err = nullptr; }
    }
    x.dev_err = static_cast<fj::ErrorRecord*>(x.temp(count * sizeof(fj::ErrorRecord)));
    if (!sub->host_err || !x.dev_err) { fj_sub_destroy(sub); return FJ_ALLOCATION_FAILED; }
    for (uint32_t i = 0; i < count; ++i) { sub->host_err[i].flag = 0; sub->host_err[i].value = 0xFFFFFFFFu; }
    cudaMemcpyAsync(x.dev_err, sub->host_err, count * sizeof(fj::ErrorRecord), cudaMemcpyHostToDevice, be->stream);
  }
  cudaEventRecord(sub->start, be->stream);
  int32_t status = FJ_OK;
  uint32_t i = 0;
  auto mark = [&]() {
    if (!profiled) return;
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, be->stream);
    sub->marks.push_back(e);
  };
  mark();
  while (i < count && status == FJ_OK) {
    const fj_dispatch& d = dispatches[i];
    sub->ops[i] = d.op;
    const unsigned long long before = be->ctx.launches;
    if (profiled && d.inputs && d.outputs) {
      if (sub->costs.empty()) sub->costs.assign(static_cast<size_t>(count) * 3, 0);
      dispatch_cost(d, &sub->costs[3 * i], &sub->costs[3 * i + 1], &sub->costs[3 * i + 2]);
    }
    fj::ErrorRecord* err = x.dev_err + i;
    uint32_t consumed = 1;
    if ((d.n_inputs && !d.inputs) || (d.n_outputs && !d.outputs)) status = FJ_INVALID_INPUT;
    else switch (d.op) {
      case FJ_OP_PROGRAM: status = exec_program(x, d); break;
      case FJ_OP_COPY: status = exec_copy(x, d); break;
      case FJ_OP_PAGED_COPY: status = exec_paged_copy(x, d, err); break;
      case FJ_OP_RMS_NORM: status = exec_rms_norm(x, d); break;
      case FJ_OP_ARGMAX: status = exec_argmax(x, d); break;
      case FJ_OP_TOP_K: status = exec_top_k(x, d); break;
      case FJ_OP_SAMPLE: status = exec_sample(x, d, err); break;
      case FJ_OP_ROPE: status = exec_rope(x, d); break;
      case FJ_OP_EMBED: status = exec_embed(x, d, err); break;
      case FJ_OP_QUANT_EMBED: status = exec_quant_embed(x, d, err); break;
      case FJ_OP_MATMUL: status = exec_matmul(x, d); break;
      case FJ_OP_QUANT_MATMUL: status = exec_quant_matmul(x, d); break;
      case FJ_OP_GATHER_QUANT_MATMUL: status = exec_gather_quant(x, d, err); break;
      case FJ_OP_SDPA: status = exec_sdpa(x, d); break;
      case FJ_OP_GATHER_MATMUL: status = exec_gather_matmul(x, d, err); break;
      case FJ_OP_PAGED_SDPA:
      case FJ_OP_PAGED_SDPA_APPEND: {
        const bool append = d.op == FJ_OP_PAGED_SDPA_APPEND;
        const uint32_t want_in = append ? 5 : 5, want_out = append ? 3 : 1;
        if ((d.n_inputs != want_in && d.n_inputs != want_in + 1) || d.n_outputs != want_out) { status = FJ_INVALID_INPUT; break; }
        // extend the run while the next dispatch shares planes/geometry and does not touch what the run writes. The bytes the
        // run has written so far are kept as one hull per buffer (conservative: a gap inside the hull counts as written), so
        // the test is one comparison per operand instead of one per earlier lane.
        uint32_t end = i + 1;
        struct Hull { uint64_t buffer, lo, hi; };
        std::vector<Hull> written;
        auto note_output = [&](const fj_tensor& t) {
          uint64_t lo = 0, hi = 0;
          if (!tensor_byte_span(t, &lo, &hi)) return false;
          for (Hull& h : written)
            if (h.buffer == t.buffer) { h.lo = std::min(h.lo, lo); h.hi = std::max(h.hi, hi); return true; }
          written.push_back(Hull{t.buffer, lo, hi});
          return true;
        };
        auto touches_written = [&](const fj_tensor& t) {
          uint64_t lo = 0, hi = 0;
          if (!tensor_byte_span(t, &lo, &hi)) return true;
          for (const Hull& h : written)
            if (h.buffer == t.buffer && lo < h.hi && h.lo < hi) return true;
          return false;
        };
        bool spans_ok = note_output(d.outputs[0]);
        while (spans_ok && end < count && (dispatches[end].n_inputs == d.n_inputs) && dispatches[end].inputs && dispatches[end].outputs && paged_run_compatible(be, d, dispatches[end])) {
          const fj_dispatch& next = dispatches[end];
          bool hazard = touches_written(next.inputs[0]) || touches_written(next.outputs[0]);
          if (append) hazard = hazard || touches_written(next.inputs[1]) || touches_written(next.inputs[2]);
          if (hazard || !note_output(next.outputs[0])) break;
          ++end;
        }
        consumed = end - i;
        for (uint32_t j = i; j < end; ++j) sub->ops[j] = dispatches[j].op;
        status = exec_paged_attention_run(x, dispatches + i, consumed, err);
        break;
      }
      default: status = FJ_UNSUPPORTED_OPERATION; break;
    }
    x.finish();
    sub->kernels[i] = static_cast<uint32_t>(be->ctx.launches - before);
    for (uint32_t j = 0; j < consumed; ++j) mark();
    i += consumed;
  }
  if (count) cudaMemcpyAsync(sub->host_err, x.dev_err, count * sizeof(fj::ErrorRecord), cudaMemcpyDeviceToHost, be->stream);
  cudaEventRecord(sub->stop, be->stream);
  for (void* t : x.temps) cudaFreeAsync(t, be->stream);
  sub->launches = be->ctx.launches - launches_before;
  if (status != FJ_OK) {
    // validation failures are synchronous errors of submit itself (the reference refuses to record the dispatch)
    cudaStreamSynchronize(be->stream);
    fj_sub_destroy(sub);
    return status;
  }
  cudaError_t launch_error = cudaGetLastError();
  if (launch_error != cudaSuccess) {
    sub->done = true;
    sub->result = FJ_DEVICE_EXECUTION_FAILED;
    sub->error.submission = sub->serial;
    sub->error.code = launch_error;
  }
  *out = sub;
  return FJ_OK;
}

// ---- graph templates: Backend::prepare_graph / replay, crates/forja-core/src/backend.rs:858-967 ----

struct fj_graph {
  fj_backend* be = nullptr;
  std::vector<fj_dispatch> dispatches;
  std::vector<std::vector<fj_tensor>> inputs, outputs;  // storage the dispatches point into
  std::vector<fj_graph_binding> bindings;
  uint32_t n_params = 0;
};

// Where a binding lands, or nullptr for a field code / operand index the template does not have.
// u32 fields come back through `narrow`, 64-bit tensor offsets through `wide`.
static bool graph_field(fj_graph* g, const fj_graph_binding& b, uint32_t** narrow, uint64_t** wide) {
  *narrow = nullptr; *wide = nullptr;
  if (b.dispatch >= g->dispatches.size()) return false;
  fj_dispatch& d = g->dispatches[b.dispatch];
  if (b.field <= FJ_GRAPH_FIELD_U3) { uint32_t* u[4] = {&d.u0, &d.u1, &d.u2, &d.u3}; *narrow = u[b.field]; return true; }
  const uint32_t kind = b.field & 0xF00u, operand = (b.field >> 4) & 0xFu, axis = b.field & 0xFu;
  const bool is_input = kind == FJ_GRAPH_FIELD_INPUT_OFFSET || kind == FJ_GRAPH_FIELD_INPUT_EXTENT;
  const bool is_output = kind == FJ_GRAPH_FIELD_OUTPUT_OFFSET || kind == FJ_GRAPH_FIELD_OUTPUT_EXTENT;
  if (!is_input && !is_output) return false;
  std::vector<fj_tensor>& tensors = is_input ? g->inputs[b.dispatch] : g->outputs[b.dispatch];
  if (operand >= tensors.size()) return false;
  fj_tensor& t = tensors[operand];
  if (kind == FJ_GRAPH_FIELD_INPUT_OFFSET || kind == FJ_GRAPH_FIELD_OUTPUT_OFFSET) { if (axis != 0) return false; *wide = &t.offset; return true; }
  if (axis >= t.rank) return false;
  *narrow = &t.shape[axis];
  return true;
}

int32_t fj_graph_prepare(fj_backend* be, const fj_dispatch* dispatches, uint32_t count, const fj_graph_binding* bindings, uint32_t n_bindings,
                         uint32_t n_params, fj_graph** out) {
  if (!be || !out || (count && !dispatches) || (n_bindings && !bindings) || n_params > 16) return FJ_INVALID_INPUT;  // ParamSpace holds at most 16 parameters
  auto* g = new fj_graph();
  g->be = be; g->n_params = n_params;
  g->dispatches.assign(dispatches, dispatches + count);
  g->inputs.resize(count); g->outputs.resize(count);
  for (uint32_t i = 0; i < count; ++i) {
    const fj_dispatch& d = dispatches[i];
    if ((d.n_inputs && !d.inputs) || (d.n_outputs && !d.outputs) || d.n_inputs > 16 || d.n_outputs > 16) { delete g; return FJ_INVALID_INPUT; }
    g->inputs[i].assign(d.inputs, d.inputs + d.n_inputs);
    g->outputs[i].assign(d.outputs, d.outputs + d.n_outputs);
  }
  for (uint32_t i = 0; i < count; ++i) { g->dispatches[i].inputs = g->inputs[i].data(); g->dispatches[i].outputs = g->outputs[i].data(); }
  g->bindings.assign(bindings, bindings + n_bindings);
  for (const fj_graph_binding& b : g->bindings) {
    uint32_t* narrow; uint64_t* wide;
    if (b.param >= n_params || !graph_field(g, b, &narrow, &wide)) { delete g; return FJ_INVALID_INPUT; }
  }
  *out = g;
  return FJ_OK;
}

// replay: every bound field becomes offset + scale * values[param], evaluated in checked 64-bit arithmetic and,
// for 32-bit fields, refused when it does not fit (Affine::evaluate, crates/forja-core/src/symbolic.rs:249-262);
// the instantiated commands then go through fj_submit, which validates them like any other submission.
int32_t fj_graph_replay(fj_graph* g, const uint32_t* values, uint32_t n_values, uint32_t profiled, fj_submission** out) {
  if (!g || !out || n_values != g->n_params || (n_values && !values)) return FJ_INVALID_INPUT;
  // instantiate into a private copy so that concurrent replays of one template do not see each other's values
  fj_graph copy;
  copy.be = g->be; copy.n_params = g->n_params;
  copy.dispatches = g->dispatches; copy.inputs = g->inputs; copy.outputs = g->outputs;
  for (size_t i = 0; i < copy.dispatches.size(); ++i) { copy.dispatches[i].inputs = copy.inputs[i].data(); copy.dispatches[i].outputs = copy.outputs[i].data(); }
  for (const fj_graph_binding& b : g->bindings) {
    uint32_t* narrow; uint64_t* wide;
    if (!graph_field(&copy, b, &narrow, &wide)) return FJ_INVALID_INPUT;
    uint64_t v = 0;
    if (__builtin_mul_overflow(static_cast<uint64_t>(b.scale), static_cast<uint64_t>(values[b.param]), &v) || __builtin_add_overflow(v, b.offset, &v)) return FJ_INVALID_INPUT;
    if (narrow) { if (v > 0xFFFFFFFFull) return FJ_INVALID_INPUT; *narrow = static_cast<uint32_t>(v); }
    else *wide = v;
  }
  return fj_submit(g->be, copy.dispatches.data(), static_cast<uint32_t>(copy.dispatches.size()), profiled, out);
}

void fj_graph_destroy(fj_graph* g) { delete g; }

int32_t fj_sub_wait(fj_submission* sub, uint64_t timeout_ns) {
  if (!sub) return FJ_INVALID_INPUT;
  if (sub->done) return sub->result;
  cudaSetDevice(sub->be->device);
  cudaError_t e;
  if (timeout_ns == 0) {
    e = cudaEventSynchronize(sub->stop);
  } else {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(timeout_ns);
    while ((e = cudaEventQuery(sub->stop)) == cudaErrorNotReady) {
      if (std::chrono::steady_clock::now() >= deadline) { cudaGetLastError(); return FJ_TIMEOUT; }
      std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
  }
  sub->done = true;
  if (e != cudaSuccess) {
    sub->result = FJ_DEVICE_EXECUTION_FAILED;
    sub->error.submission = sub->serial;
    sub->error.code = e;
    return sub->result;
  }
  for (uint32_t i = 0; i < sub->count; ++i) {
    if (sub->host_err[i].flag != 0) {
      sub->error.submission = sub->serial;
      sub->error.dispatch = i;
      sub->error.op = sub->ops[i];
      sub->error.flag = sub->host_err[i].flag;
      sub->error.value = sub->host_err[i].value;
      sub->result = sub->host_err[i].flag == fj::ERR_INDEX ? FJ_INDEX_OUT_OF_RANGE : sub->host_err[i].flag == fj::ERR_INVALID ? FJ_INVALID_INPUT : FJ_DEVICE_ERROR_FLAG;
      break;
    }
  }
  return sub->result;
}

int32_t fj_sub_gpu_time_ns(fj_submission* sub, uint64_t* ns) {
  if (!sub || !ns) return FJ_INVALID_INPUT;
  if (!sub->done) return FJ_INVALID_INPUT;
  float ms = 0.0f;
  if (cudaEventElapsedTime(&ms, sub->start, sub->stop) != cudaSuccess) { cudaGetLastError(); return FJ_EXECUTION_FAILED; }
  *ns = static_cast<uint64_t>(static_cast<double>(ms) * 1.0e6);
  return FJ_OK;
}
uint64_t fj_sub_completion_serial(fj_submission* sub) { return sub ? sub->serial : 0; }
int32_t fj_sub_error(fj_submission* sub, fj_device_error* out) {
  if (!sub || !out) return FJ_INVALID_INPUT;
  *out = sub->error;
  return FJ_OK;
}
uint32_t fj_sub_kernel_launches(fj_submission* sub) { return sub ? static_cast<uint32_t>(sub->launches) : 0; }
int32_t fj_sub_profile(fj_submission* sub, fj_dispatch_profile* out, uint32_t cap, uint32_t* count) {
  if (!sub || !count) return FJ_INVALID_INPUT;
  *count = sub->count;
  if (!out) return FJ_OK;
  for (uint32_t i = 0; i < sub->count && i < cap; ++i) {
    out[i].op = sub->ops[i];
    out[i].kernels = sub->kernels[i];
    out[i].ns = 0;
    const bool have_cost = sub->costs.size() == static_cast<size_t>(sub->count) * 3;
    out[i].read_bytes = have_cost ? sub->costs[3 * i] : 0;
    out[i].write_bytes = have_cost ? sub->costs[3 * i + 1] : 0;
    out[i].flops = have_cost ? sub->costs[3 * i + 2] : 0;
    if (sub->done && sub->marks.size() == static_cast<size_t>(sub->count) + 1) {
      float ms = 0.0f;
      if (cudaEventElapsedTime(&ms, sub->marks[i], sub->marks[i + 1]) == cudaSuccess) out[i].ns = static_cast<uint64_t>(static_cast<double>(ms) * 1.0e6);
      else cudaGetLastError();
    }
  }
  return FJ_OK;
}
void fj_sub_destroy(fj_submission* sub) {
  if (!sub) return;
  cudaSetDevice(sub->be->device);
  if (sub->stop) cudaEventSynchronize(sub->stop);  // physical completion before the pinned record goes away
  if (sub->start) cudaEventDestroy(sub->start);
  if (sub->stop) cudaEventDestroy(sub->stop);
  for (auto e : sub->marks) cudaEventDestroy(e);
  if (sub->host_err) {
    std::lock_guard<std::mutex> pinned(sub->be->pinned_mutex);
    if (sub->be->pinned_pool.size() < 64) sub->be->pinned_pool.emplace_back(sub->host_err, sub->host_err_capacity);
    else cudaFreeHost(sub->host_err);
  }
  delete sub;
}

int32_t fj_synchronize(fj_backend* be) {
  if (!be) return FJ_INVALID_INPUT;
  cudaSetDevice(be->device);
  return cuda_status(cudaStreamSynchronize(be->stream));
}
uint64_t fj_kernel_launch_count(fj_backend* be) { return be ? be->ctx.launches : 0; }

int32_t fj_timer_create(fj_backend* be, uint64_t* timer) {
  if (!be || !timer) return FJ_INVALID_INPUT;
  std::lock_guard<std::mutex> lock(be->mutex);
  cudaSetDevice(be->device);
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return FJ_ALLOCATION_FAILED;
  be->timers.push_back(e);
  *timer = be->timers.size();
  return FJ_OK;
}
int32_t fj_timer_record(fj_backend* be, uint64_t timer) {
  if (!be || timer == 0 || timer > be->timers.size()) return FJ_INVALID_INPUT;
  cudaSetDevice(be->device);
  return cuda_status(cudaEventRecord(be->timers[timer - 1], be->stream));
}
int32_t fj_timer_elapsed_ns(fj_backend* be, uint64_t start_timer, uint64_t stop_timer, uint64_t* ns) {
  if (!be || !ns || start_timer == 0 || stop_timer == 0 || start_timer > be->timers.size() || stop_timer > be->timers.size()) return FJ_INVALID_INPUT;
  cudaSetDevice(be->device);
  if (cudaEventSynchronize(be->timers[stop_timer - 1]) != cudaSuccess) return FJ_EXECUTION_FAILED;
  float ms = 0.0f;
  if (cudaEventElapsedTime(&ms, be->timers[start_timer - 1], be->timers[stop_timer - 1]) != cudaSuccess) return FJ_EXECUTION_FAILED;
  *ns = static_cast<uint64_t>(static_cast<double>(ms) * 1.0e6);
  return FJ_OK;
}

}  // extern "C"
