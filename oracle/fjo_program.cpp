// CPU oracle: scalar-program interpreter, restating crates/forja-cpu/src/interpreter.rs:38-396.
// Test infrastructure only; see fjo.h.
#include "fjo.h"
#include "fjo_convert.h"

#include <cmath>
#include <cstring>
#include <vector>

namespace fjo {
bool decode(const void* src, int dt, float* dst, size_t n);
bool encode(const float* src, void* dst, int dt, size_t n);

namespace {

enum Tag { T_INPUT = 0, T_CONST = 1, T_INDEX = 2, T_EXTENT = 3, T_UNARY = 4, T_BINARY = 5, T_SELECT = 6, T_CAST = 7, T_REDUCE = 8 };
enum Un { U_NEG, U_ABS, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_SIN, U_COS, U_TANH, U_SIGMOID, U_RECIP, U_FLOOR, U_LOG1P, U_EXPROUNDED };
enum Bin { B_ADD, B_SUB, B_MUL, B_DIV, B_MIN, B_MAX, B_POW, B_LT, B_LE, B_EQ, B_NE, B_GE, B_GT };
enum Red { R_SUM, R_MAX, R_MIN };
enum VT { V_F32 = 0, V_U32 = 1, V_BOOL = 2 };

struct Scalar { int type; float f; uint32_t u; bool b; };
inline Scalar sf(float v) { return {V_F32, v, 0, false}; }
inline Scalar su(uint32_t v) { return {V_U32, 0.0f, v, false}; }
inline Scalar sb(bool v) { return {V_BOOL, 0.0f, 0, v}; }

struct Input { bool is_u32; const float* f; const uint32_t* u; };

inline float propagating_min(float l, float r) { return (std::isnan(l) || std::isnan(r)) ? NAN : std::fmin(l, r); }
inline float propagating_max(float l, float r) { return (std::isnan(l) || std::isnan(r)) ? NAN : std::fmax(l, r); }

// Rust `as u32`: saturating, NaN -> 0 (interpreter.rs:370-373)
inline uint32_t f32_to_u32(float v) {
  if (std::isnan(v) || v <= 0.0f) return 0;
  if (v >= 4294967296.0f) return 0xFFFFFFFFu;
  return static_cast<uint32_t>(v);
}

bool unary(uint32_t op, const Scalar& x, Scalar* out) {
  if (x.type != V_F32) return false;
  float v = x.f, r;
  switch (op) {
    case U_NEG: r = -v; break;
    case U_ABS: r = std::fabs(v); break;
    case U_EXP: case U_EXPROUNDED: r = std::exp(v); break;
    case U_LOG: r = std::log(v); break;
    case U_LOG1P: r = std::log1p(v); break;
    case U_SQRT: r = std::sqrt(v); break;
    case U_RSQRT: r = 1.0f / std::sqrt(v); break;
    case U_SIN: r = std::sin(v); break;
    case U_COS: r = std::cos(v); break;
    case U_TANH: r = std::tanh(v); break;
    case U_SIGMOID: r = 1.0f / (1.0f + std::exp(-v)); break;
    case U_RECIP: r = 1.0f / v; break;
    case U_FLOOR: r = std::floor(v); break;
    default: return false;
  }
  *out = sf(r);
  return true;
}

bool binary(uint32_t op, const Scalar& l, const Scalar& r, Scalar* out) {
  if (l.type == V_F32 && r.type == V_F32) {
    float a = l.f, b = r.f;
    switch (op) {
      case B_ADD: *out = sf(a + b); return true;
      case B_SUB: *out = sf(a - b); return true;
      case B_MUL: *out = sf(a * b); return true;
      case B_DIV: *out = sf(a / b); return true;
      case B_MIN: *out = sf(propagating_min(a, b)); return true;
      case B_MAX: *out = sf(propagating_max(a, b)); return true;
      case B_POW: *out = sf(std::pow(a, b)); return true;
      case B_LT: *out = sb(a < b); return true;
      case B_LE: *out = sb(a <= b); return true;
      case B_EQ: *out = sb(a == b); return true;
      case B_NE: *out = sb(a != b); return true;
      case B_GE: *out = sb(a >= b); return true;
      case B_GT: *out = sb(a > b); return true;
      default: return false;
    }
  }
  if (l.type == V_U32 && r.type == V_U32) {
    uint32_t a = l.u, b = r.u;
    switch (op) {
      case B_ADD: *out = su(a + b); return true;
      case B_SUB: *out = su(a - b); return true;
      case B_MUL: *out = su(a * b); return true;
      case B_MIN: *out = su(a < b ? a : b); return true;
      case B_MAX: *out = su(a > b ? a : b); return true;
      case B_LT: *out = sb(a < b); return true;
      case B_LE: *out = sb(a <= b); return true;
      case B_EQ: *out = sb(a == b); return true;
      case B_NE: *out = sb(a != b); return true;
      case B_GE: *out = sb(a >= b); return true;
      case B_GT: *out = sb(a > b); return true;
      default: return false;  // Div, Pow refused on integers
    }
  }
  return false;
}

Scalar cast(uint32_t to, const Scalar& v) {
  switch (to) {
    case V_F32: return sf(v.type == V_F32 ? v.f : (v.type == V_U32 ? static_cast<float>(v.u) : (v.b ? 1.0f : 0.0f)));
    case V_U32: return su(v.type == V_F32 ? f32_to_u32(v.f) : (v.type == V_U32 ? v.u : (v.b ? 1u : 0u)));
    default: return sb(v.type == V_F32 ? v.f != 0.0f : (v.type == V_U32 ? v.u != 0 : v.b));
  }
}

void decode_coordinates(size_t linear, const uint32_t* shape, size_t rank, uint32_t* coords) {
  for (size_t a = rank; a-- > 0;) { coords[a] = static_cast<uint32_t>(linear % shape[a]); linear /= shape[a]; }
}

template <class Operand>
bool eval(const uint32_t* inst, const uint32_t* coords, const uint32_t* shape, size_t rank,
          const std::vector<Input>& inputs, size_t linear, Operand operand, Scalar* out) {
  switch (inst[0]) {
    case T_INPUT:
      if (inst[1] >= inputs.size()) return false;
      *out = inputs[inst[1]].is_u32 ? su(inputs[inst[1]].u[linear]) : sf(inputs[inst[1]].f[linear]);
      return true;
    case T_CONST: *out = sf(bits_f32(inst[1])); return true;
    case T_INDEX: if (inst[1] >= rank) return false; *out = su(coords[inst[1]]); return true;
    case T_EXTENT: if (inst[1] >= rank) return false; *out = su(shape[inst[1]]); return true;
    case T_UNARY: { Scalar x; return operand(inst[2], &x) && unary(inst[1], x, out); }
    case T_BINARY: { Scalar l, r; return operand(inst[2], &l) && operand(inst[3], &r) && binary(inst[1], l, r, out); }
    case T_SELECT: {
      Scalar c;
      if (!operand(inst[1], &c) || c.type != V_BOOL) return false;
      return operand(c.b ? inst[2] : inst[3], out);
    }
    case T_CAST: { Scalar x; if (!operand(inst[2], &x)) return false; *out = cast(inst[1], x); return true; }
    default: return false;  // Reduce is handled by the row driver
  }
}

}  // namespace
}  // namespace fjo

using namespace fjo;

extern "C" int fjo_program(int kind, const uint32_t* insts, size_t n_insts, const uint32_t* outputs,
                           size_t n_outputs, const uint32_t* shape, size_t rank,
                           const void* const* inputs_p, const int* input_dtypes, size_t n_inputs,
                           void* const* outs, const int* out_dtypes) {
  if (rank == 0 || rank > 8) return FJO_EXECUTION_FAILED;
  size_t elements = 1;
  for (size_t a = 0; a < rank; ++a) elements *= shape[a];
  std::vector<std::vector<float>> decoded(n_inputs);
  std::vector<Input> inputs(n_inputs);
  for (size_t i = 0; i < n_inputs; ++i) {
    if (input_dtypes[i] == FJO_U32) {
      inputs[i] = {true, nullptr, static_cast<const uint32_t*>(inputs_p[i])};
    } else {
      decoded[i].resize(elements);
      if (!decode(inputs_p[i], input_dtypes[i], decoded[i].data(), elements)) return FJO_EXECUTION_FAILED;
      inputs[i] = {false, decoded[i].data(), nullptr};
    }
  }
  size_t n_slots = 0;
  for (size_t o = 0; o < n_outputs; ++o) if (outputs[2 * o] + 1 > n_slots) n_slots = outputs[2 * o] + 1;
  std::vector<std::vector<float>> results(n_slots, std::vector<float>(elements));
  std::vector<uint32_t> coords(rank);

  if (kind == 0) {  // interpret_map, interpreter.rs:38-73
    std::vector<Scalar> values(n_insts);
    for (size_t linear = 0; linear < elements; ++linear) {
      decode_coordinates(linear, shape, rank, coords.data());
      for (size_t i = 0; i < n_insts; ++i) {
        auto operand = [&](uint32_t idx, Scalar* o) { if (idx >= i) return false; *o = values[idx]; return true; };
        if (!eval(&insts[4 * i], coords.data(), shape, rank, inputs, linear, operand, &values[i])) return FJO_EXECUTION_FAILED;
      }
      for (size_t o = 0; o < n_outputs; ++o) {
        const Scalar& v = values[outputs[2 * o + 1]];
        if (v.type != V_F32) return FJO_EXECUTION_FAILED;
        results[outputs[2 * o]][linear] = v.f;
      }
    }
  } else {  // interpret_row, interpreter.rs:86-150
    size_t row_width = shape[rank - 1];
    if (row_width == 0) return FJO_EXECUTION_FAILED;
    size_t row_count = elements / row_width;
    std::vector<std::vector<Scalar>> columns(n_insts, std::vector<Scalar>(row_width));
    for (size_t row = 0; row < row_count; ++row) {
      size_t row_start = row * row_width;
      for (size_t i = 0; i < n_insts; ++i) {
        const uint32_t* inst = &insts[4 * i];
        if (inst[0] == T_REDUCE) {  // reduce, interpreter.rs:260-279: sequential left to right
          if (inst[2] >= i) return FJO_EXECUTION_FAILED;
          const auto& operand = columns[inst[2]];
          if (operand[0].type != V_F32) return FJO_EXECUTION_FAILED;
          float acc;
          if (inst[1] == R_SUM) {
            acc = 0.0f;
            for (size_t l = 0; l < row_width; ++l) acc = acc + operand[l].f;
          } else {
            acc = operand[0].f;
            for (size_t l = 1; l < row_width; ++l)
              acc = inst[1] == R_MAX ? propagating_max(acc, operand[l].f) : propagating_min(acc, operand[l].f);
          }
          for (size_t l = 0; l < row_width; ++l) columns[i][l] = sf(acc);
        } else {
          for (size_t lane = 0; lane < row_width; ++lane) {
            size_t linear = row_start + lane;
            decode_coordinates(linear, shape, rank, coords.data());
            auto operand = [&](uint32_t idx, Scalar* o) { if (idx >= i) return false; *o = columns[idx][lane]; return true; };
            if (!eval(inst, coords.data(), shape, rank, inputs, linear, operand, &columns[i][lane])) return FJO_EXECUTION_FAILED;
          }
        }
      }
      for (size_t o = 0; o < n_outputs; ++o) {
        const auto& column = columns[outputs[2 * o + 1]];
        for (size_t l = 0; l < row_width; ++l) {
          if (column[l].type != V_F32) return FJO_EXECUTION_FAILED;
          results[outputs[2 * o]][row_start + l] = column[l].f;
        }
      }
    }
  }
  for (size_t s = 0; s < n_slots; ++s)
    if (!encode(results[s].data(), outs[s], out_dtypes[s], elements)) return FJO_EXECUTION_FAILED;
  return FJO_OK;
}
