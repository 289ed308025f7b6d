"""The scalar programs the reference engines submit, written in the reference's flat SSA IR
(support/forja-testing/src/representative.rs:7-126; source forms in
crates/forja-sdk/src/nn/blocks.rs:380-464 and engines/qwen3-coder/src/lib.rs:26-40).
Shared by the oracle tests and the GPU parity tests."""
from oracle import fjo


def rms_norm(eps, axis=1):
    p = fjo.Program(fjo.ROW)
    v, w = p.input(0), p.input(1)
    s = p.reduce(fjo.R_SUM, p.binary(fjo.B_MUL, v, v))
    mean = p.binary(fjo.B_DIV, s, p.cast(fjo.V_F32, p.extent(axis)))
    inv = p.unary(fjo.U_RSQRT, p.binary(fjo.B_ADD, mean, p.constant(eps)))
    p.output(0, p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, v, inv), w))
    return p


def residual_norm(eps, axis=1):
    p = fjo.Program(fjo.ROW)
    r, u, w = p.input(0), p.input(1), p.input(2)
    v = p.binary(fjo.B_ADD, r, u)
    s = p.reduce(fjo.R_SUM, p.binary(fjo.B_MUL, v, v))
    mean = p.binary(fjo.B_DIV, s, p.cast(fjo.V_F32, p.extent(axis)))
    inv = p.unary(fjo.U_RSQRT, p.binary(fjo.B_ADD, mean, p.constant(eps)))
    p.output(0, v)
    p.output(1, p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, v, inv), w))
    return p


def qk_norm_rope(eps, theta, head_dim, axis=2):
    p = fjo.Program(fjo.ROW)
    a, b, wa, wb, pos = (p.input(i) for i in range(5))
    sq = p.binary(fjo.B_ADD, p.binary(fjo.B_MUL, a, a), p.binary(fjo.B_MUL, b, b))
    s = p.reduce(fjo.R_SUM, sq)
    mean = p.binary(fjo.B_DIV, s, p.constant(head_dim))
    inv = p.unary(fjo.U_RSQRT, p.binary(fjo.B_ADD, mean, p.constant(eps)))
    a = p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, a, inv), wa)
    b = p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, b, inv), wb)
    freq = p.cast(fjo.V_F32, p.index(axis))
    expo = p.binary(fjo.B_MUL, freq, p.constant(-2.0 / head_dim))
    scale = p.binary(fjo.B_POW, p.constant(theta), expo)
    angle = p.binary(fjo.B_MUL, pos, scale)
    c, s_ = p.unary(fjo.U_COS, angle), p.unary(fjo.U_SIN, angle)
    p.output(0, p.binary(fjo.B_SUB, p.binary(fjo.B_MUL, a, c), p.binary(fjo.B_MUL, b, s_)))
    p.output(1, p.binary(fjo.B_ADD, p.binary(fjo.B_MUL, b, c), p.binary(fjo.B_MUL, a, s_)))
    return p


def rope_pairs(theta, rotary_dim, axis=2):
    p = fjo.Program(fjo.MAP)
    a, b, pos = p.input(0), p.input(1), p.input(2)
    freq = p.cast(fjo.V_F32, p.index(axis))
    expo = p.binary(fjo.B_MUL, freq, p.constant(-2.0 / rotary_dim))
    angle = p.binary(fjo.B_MUL, pos, p.binary(fjo.B_POW, p.constant(theta), expo))
    c, s_ = p.unary(fjo.U_COS, angle), p.unary(fjo.U_SIN, angle)
    p.output(0, p.binary(fjo.B_SUB, p.binary(fjo.B_MUL, a, c), p.binary(fjo.B_MUL, b, s_)))
    p.output(1, p.binary(fjo.B_ADD, p.binary(fjo.B_MUL, b, c), p.binary(fjo.B_MUL, a, s_)))
    return p


def silu_mul():
    p = fjo.Program(fjo.MAP)
    g, u = p.input(0), p.input(1)
    p.output(0, p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, g, p.unary(fjo.U_SIGMOID, g)), u))
    return p


def gated_up():
    """The matmul epilogue of engines/smollm2/src/optimized.rs:249-252: gate * sigmoid(gate) * up with up = input 0
    (the accumulator) and gate = input 1 (the extra operand)."""
    p = fjo.Program(fjo.MAP)
    up, gate = p.input(0), p.input(1)
    p.output(0, p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, gate, p.unary(fjo.U_SIGMOID, gate)), up))
    return p


def add():
    p = fjo.Program(fjo.MAP)
    p.output(0, p.binary(fjo.B_ADD, p.input(0), p.input(1)))
    return p


def softmax():
    p = fjo.Program(fjo.ROW)
    v = p.input(0)
    e = p.unary(fjo.U_EXP, p.binary(fjo.B_SUB, v, p.reduce(fjo.R_MAX, v)))
    p.output(0, p.binary(fjo.B_DIV, e, p.reduce(fjo.R_SUM, e)))
    return p
