"""Pins the CPU oracle to the known-answer vectors of the reference's own unit tests.

Each test restates the inputs and expected outputs of one reference test (cited by file:line,
paths relative to the reference repository); expectations are computed here independently of
the oracle (closed forms, numpy f64, or Python's own sort) exactly as the reference tests do.
"""
import math
import struct

import numpy as np
import pytest

from oracle import fjo


def bits(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


def total_key(x):
    b = int(np.array([x], np.float32).view(np.int32)[0])
    return b ^ (((b >> 31) & 0xFFFFFFFF) >> 1)


def assert_relative(actual, expected, tol):
    actual = np.asarray(actual, np.float64).ravel()
    expected = np.asarray(expected, np.float64).ravel()
    assert actual.shape == expected.shape
    assert np.all(np.abs(actual - expected) <= tol * np.maximum(1.0, np.abs(expected)))


# ---- conversions -----------------------------------------------------------------------------

def test_f16_bf16_round_trip_matches_ieee_rne():
    import torch
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-10, 10, 20000).astype(np.float32),
        np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 65519.99, 1e-8, 6e-8, 5.9604645e-8, 2.98e-8, 3.4e38, 1.0 + 2 ** -8, 1.0 + 2 ** -9, 1.0 + 3 * 2 ** -9], np.float32),
    ])
    t = torch.from_numpy(vals)
    want_bf16 = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    want_f16 = t.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(fjo.encode(vals, fjo.BF16), want_bf16)
    assert np.array_equal(fjo.encode(vals, fjo.F16).view(np.uint16), want_f16)
    all16 = np.arange(65536, dtype=np.uint16)
    f16 = all16.view(np.float16)
    finite = ~np.isnan(f16)
    assert np.array_equal(fjo.decode(f16, fjo.F16)[finite].view(np.uint32), f16.astype(np.float32)[finite].view(np.uint32))
    want = torch.from_numpy(all16.view(np.int16)).view(torch.bfloat16).to(torch.float32).numpy()
    got = fjo.decode(all16, fjo.BF16)
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok].view(np.uint32), want[ok].view(np.uint32))
    assert np.all(np.isnan(got[~ok]))


# ---- crates/forja-cpu/src/lib.rs:1883-1924 -----------------------------------------------------

def test_paged_copy_converts_directly_into_reduced_storage():
    values = (np.arange(21, dtype=np.float32) / 8.0).reshape(7, 3)
    pool = np.zeros((3, 4, 3), np.float16)
    table = np.array([[2, 5], [0, 7]], np.uint32)
    generations = np.array([7, 0, 5], np.uint32)
    fjo.paged_copy_in(values, fjo.F32, pool, fjo.F16, table, generations, start=1, page_tokens=4)
    out = fjo.paged_copy_out(pool, fjo.F16, table, generations, 1, 7, 4, fjo.F32)
    assert np.array_equal(out, values.astype(np.float16).astype(np.float32))
    # token 1..3 land in physical page 2 rows 1..3, tokens 4..7 in page 0 rows 0..3; page 1 untouched
    assert np.array_equal(pool[2, 1:4].astype(np.float32), values[0:3].astype(np.float16).astype(np.float32))
    assert np.array_equal(pool[0, 0:4].astype(np.float32), values[3:7].astype(np.float16).astype(np.float32))
    assert not pool[1].any() and not pool[2, 0].any()


# ---- crates/forja-cpu/src/paged.rs:409-419 -----------------------------------------------------

def test_paged_copy_crosses_nonconsecutive_pages():
    pool = np.zeros((3, 4, 2), np.float32)
    table = np.array([[2, 1], [0, 1]], np.uint32)
    gens = np.array([1, 1, 1], np.uint32)
    values = np.arange(12, dtype=np.uint32).view(np.float32).reshape(6, 2)
    fjo.paged_copy_in(values, fjo.F32, pool, fjo.F32, table, gens, 2, 4)
    out = fjo.paged_copy_out(pool, fjo.F32, table, gens, 2, 6, 4, fjo.F32)
    assert np.array_equal(out.view(np.uint32), values.view(np.uint32))


# ---- crates/forja-cpu/src/paged.rs:458-476 -----------------------------------------------------

def test_paged_attention_matches_a_hand_checked_case():
    pool = np.zeros((2, 4, 1, 2), np.float32)
    table = np.array([[1, 4], [0, 3]], np.uint32)
    gens = np.array([3, 4], np.uint32)
    fjo.paged_copy_in(np.array([[1.0, 0.0], [0.0, 1.0]], np.float32), fjo.F32, pool.reshape(2, 4, 2), fjo.F32, table, gens, 0, 4)
    out = fjo.paged_sdpa(np.array([[[1.0, 0.0]]], np.float32), fjo.F32, pool, fjo.F32, pool, fjo.F32, table, gens,
                         key_length=2, q_start=0, scale=1.0, causal=False, page_tokens=4)
    expected = math.e / (math.e + 1.0)
    assert abs(out[0, 0, 0] - expected) < 1e-6
    assert abs(out[0, 0, 1] - (1.0 - expected)) < 1e-6


# ---- crates/forja-cpu/src/lib.rs:1927-1970 -----------------------------------------------------

def test_paged_append_stores_both_planes_before_attention():
    q = np.zeros((16, 1, 128), np.float32)
    k = np.zeros((1, 8, 128), np.float32)
    v = np.ones((1, 8, 128), np.float32)
    table = np.array([[0, 1]], np.uint32)
    gens = np.array([1], np.uint32)
    kp = np.zeros((1, 16, 8, 128), np.float16)
    vp = np.zeros((1, 16, 8, 128), np.float16)
    out = fjo.paged_sdpa_append(q, fjo.F32, k, fjo.F32, v, fjo.F32, kp, fjo.F16, vp, fjo.F16, table, gens, 0, 0.125, 16)
    assert np.array_equal(out, np.ones((16, 1, 128), np.float32))
    raw = vp.view(np.uint16).ravel()
    assert np.all(raw[:1024] == 0x3C00) and not raw[1024:].any()
    with pytest.raises(fjo.OracleError):
        fjo.paged_sdpa_append(q, fjo.F32, k, fjo.F32, v, fjo.F32, kp, fjo.F16, vp, fjo.F16, table, gens, 0xFFFFFFFF, 0.125, 16)


def test_inactive_lane_writes_zeros_and_skips_copies():
    # crates/forja-cpu/src/lib.rs:197-199, 319-328
    q = np.ones((2, 1, 4), np.float32)
    kp = np.ones((1, 2, 1, 4), np.float32)
    table = np.array([[0, 0xFFFFFFFF]], np.uint32)  # poisoned: must never be dereferenced
    gens = np.array([0], np.uint32)
    out = fjo.paged_sdpa(q, fjo.F32, kp, fjo.F32, kp, fjo.F32, table, gens, 1, 0, 1.0, True, 2, activity=0)
    assert not out.any()
    pool = np.zeros((1, 2, 4), np.float32)
    fjo.paged_copy_in(np.ones((1, 4), np.float32), fjo.F32, pool, fjo.F32, table, gens, 0, 2, activity=0)
    assert not pool.any()
    with pytest.raises(fjo.OracleError):  # an active lane refuses the poisoned entry
        fjo.paged_copy_in(np.ones((1, 4), np.float32), fjo.F32, pool, fjo.F32, table, gens, 0, 2)


# ---- crates/forja-core/src/paged.rs:346-420 ----------------------------------------------------

def test_page_layout_and_table_authentication():
    assert fjo.paged_layout_page_bytes(33, fjo.F16, 1024, 256) == 67584
    with pytest.raises(fjo.OracleError):
        fjo.paged_layout_page_bytes(0, fjo.F16, 1024, 256)
    with pytest.raises(fjo.OracleError):
        fjo.paged_layout_page_bytes(16, fjo.F16, 1024, 3)
    table = np.array([[1, 7], [0, 0xFFFFFFFF]], np.uint32)
    gens = np.array([3, 7], np.uint32)
    assert fjo.page_table_resolve(table, gens, 0) == (0, 1)
    assert fjo.page_table_resolve(table, gens, 1)[0] == 3  # poisoned entry is a stale generation
    assert fjo.page_table_resolve(table, gens, 2)[0] == 1  # logical out of bounds
    assert fjo.page_table_resolve(np.array([[5, 1]], np.uint32), gens, 0)[0] == 2  # physical out of bounds
    assert fjo.page_table_resolve(np.array([[1, 6]], np.uint32), gens, 0)[0] == 3  # stale


# ---- crates/forja-cpu/src/lib.rs:2786-2845 -----------------------------------------------------

@pytest.mark.parametrize("bits_,p_dt", [(4, fjo.BF16), (8, fjo.F16)])
@pytest.mark.parametrize("rows", [1, 7, 33])
def test_quant_matmul_dequantizes_q4_and_q8_in_mlx_order(bits_, p_dt, rows):
    inner = 64
    act = (np.arange(rows * inner) % 17).astype(np.float32) / 8.0 - 1.0
    vpw = 32 // bits_
    repeats = inner // vpw
    pattern = 0x11111111 if bits_ == 4 else 0x01010101
    maximum = (1 << bits_) - 1
    words = np.repeat(np.array([0, pattern, pattern * maximum], np.uint64), repeats).astype(np.uint32).reshape(3, repeats)
    scale_values, bias_values = [0.5, -0.25, 0.125], [1.0, 2.0, -1.0]
    scales = fjo.encode(np.array(scale_values, np.float32).reshape(3, 1), p_dt)
    biases = fjo.encode(np.array(bias_values, np.float32).reshape(3, 1), p_dt)
    out = fjo.quant_matmul(act.reshape(rows, inner), fjo.F32, words, scales, biases, p_dt, bits_, 64, fjo.F32)
    sums = act.reshape(rows, inner).astype(np.float64).sum(axis=1)
    expected = np.stack([sums * bias_values[0], sums * (scale_values[1] + bias_values[1]),
                         sums * (scale_values[2] * maximum + bias_values[2])], axis=1)
    assert_relative(out, expected, 1e-5)


# ---- crates/forja-cpu/src/lib.rs:2848-2951 -----------------------------------------------------

def test_gathered_quantized_matmul_selects_duplicate_routes_and_reports_lowest_bad_index():
    x = np.ones((1, 64), np.float32)
    packed = np.repeat((np.arange(6, dtype=np.uint64) * 0x11111111).astype(np.uint32), 8).reshape(3, 2, 8)
    scales = fjo.encode(np.ones((3, 2, 1), np.float32), fjo.BF16)
    biases = fjo.encode(np.zeros((3, 2, 1), np.float32), fjo.BF16)
    idx = np.array([[2, 0, 2]], np.uint32)
    out = fjo.gather_quant_matmul(x, fjo.F32, packed, scales, biases, fjo.BF16, idx, 4, 64, fjo.F32)
    assert out.ravel().tolist() == [256.0, 320.0, 0.0, 64.0, 256.0, 320.0]
    # paired form + epilogue gate*sigmoid(gate)*up written in the reference's IR
    p = fjo.Program(fjo.MAP)
    a, b = p.input(0), p.input(1)
    neg = p.unary(fjo.U_NEG, a)
    ex = p.unary(fjo.U_EXP, neg)
    one = p.constant(1.0)
    den = p.binary(fjo.B_ADD, one, ex)
    sil = p.binary(fjo.B_DIV, a, den)
    p.output(0, p.binary(fjo.B_MUL, sil, b))
    fused, = fjo.program(p, out.shape, [out, out], [fjo.F32, fjo.F32], [fjo.F32])
    expected = [v / (1.0 + math.exp(-v)) * v for v in [256.0, 320.0, 0.0, 64.0, 256.0, 320.0]]
    assert_relative(fused, expected, 1e-5)
    bad, index = fjo.gather_quant_matmul(x, fjo.F32, packed, scales, biases, fjo.BF16, np.array([[99, 7]], np.uint32), 4, 64, fjo.F32, raise_on_bad=False)
    assert index == 7 and not bad.any()


# ---- crates/forja-cpu/src/lib.rs:2954-3017 -----------------------------------------------------

def test_gathered_matmul_selects_duplicate_routes_and_reports_lowest_bad_index():
    # crates/forja-cpu/src/lib.rs:2449-2488
    x = np.array([[1.0, 2.0], [3.0, 4.0]], np.float32)
    weights = np.array([1.0, 0.0, 0.0, 1.0, 1.0, 1.0, 1.0, 1.0, 2.0, 0.0, 0.0, 3.0], np.float32).reshape(3, 2, 2)
    out = fjo.gather_matmul(x, fjo.F32, weights, fjo.F32, np.array([[2, 0, 2], [0, 2, 0]], np.uint32))
    assert out.ravel().tolist() == [2.0, 6.0, 1.0, 2.0, 2.0, 6.0, 3.0, 4.0, 6.0, 12.0, 3.0, 4.0]
    out, bad = fjo.gather_matmul(x, fjo.F32, weights, fjo.F32, np.array([[99], [7]], np.uint32), raise_on_bad=False)
    assert bad == 7 and not out.any()


def test_combined_quantized_matmul_keeps_valid_routes_and_reports_lowest_bad_index():
    act = np.repeat(np.arange(1, 6, dtype=np.float32), 64).reshape(1, 5, 64)
    packed = np.repeat((np.arange(1, 7, dtype=np.uint64) * 0x11111111).astype(np.uint32), 8).reshape(3, 2, 8)
    scales = fjo.encode(np.full((3, 2, 1), 0.5, np.float32), fjo.BF16)
    biases = fjo.encode(np.full((3, 2, 1), 0.25, np.float32), fjo.BF16)
    idx = np.array([[2, 99, 0, 7, 1]], np.uint32)
    weights = np.array([[0.5, 1.0, -0.25, 2.0, 0.75]], np.float32)
    acc, index = fjo.gather_quant_weighted_sum(act, fjo.F32, packed, scales, biases, fjo.BF16, idx, weights, fjo.F32, 4, 64, fjo.F32, raise_on_bad=False)
    assert index == 7
    out = fjo.prog_add(acc, np.array([[1.5, -2.0]], np.float32), fjo.F32)
    assert out.ravel().tolist() == [473.5, 582.0]


# ---- crates/forja-cpu/src/lib.rs:3020-3037, 2760-2783 ------------------------------------------

def test_embed_zeros_bad_rows_and_reports_the_lowest_bad_id():
    table = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    out, index = fjo.embed(table, fjo.F32, [2, 100, 0, 99], raise_on_bad=False)
    assert index == 99
    assert out.ravel().tolist() == [5.0, 6.0, 0.0, 0.0, 1.0, 2.0, 0.0, 0.0]
    values = (np.arange(1000 * 1024) % 251).astype(np.float32).reshape(1000, 1024)
    got = fjo.embed(values, fjo.F32, [0, 1, 998, 999])
    assert np.array_equal(got, values[[0, 1, 998, 999]])


# ---- crates/forja-cpu/src/lib.rs:2387-2447, 2491-2521 ------------------------------------------

def test_argmax_prefers_the_last_equal_value():
    assert fjo.argmax(np.array([[1.0, 9.0, 2.0, 9.0, 3.0]], np.float32), fjo.F32).tolist() == [3]
    wide = np.zeros((1, 151936), np.float32)
    assert fjo.argmax(wide, fjo.F32).tolist() == [151935]
    wide[0, 77] = np.float32(np.nan)  # +NaN is the greatest value under total order
    assert fjo.argmax(wide, fjo.F32).tolist() == [77]


@pytest.mark.parametrize("width,k", [(1, 1), (64, 8), (128, 8), (2050, 64)])
def test_top_k_orders_rows_for_edge_widths_ties_and_nans(width, k):
    values = (np.arange(width) % 11).astype(np.float32)
    if width >= 128:
        values.view(np.uint32)[3] = 0x7FC00001
        values.view(np.uint32)[9] = 0x7FC00002
        values.view(np.uint32)[17] = 0xFFC00001
    if width == 2050:
        values[2048], values[2049] = 1000.0, 999.0
    order = sorted(range(width), key=lambda i: (-total_key(values[i]), i))[:k]
    got_v, got_i = fjo.top_k(values.reshape(1, width), fjo.F32, k, False)
    assert got_i.ravel().tolist() == order
    assert got_v.view(np.uint32).ravel().tolist() == [int(values.view(np.uint32)[i]) for i in order]


def test_top_k_normalizes_over_the_selected_set():
    v, i = fjo.top_k(np.array([[1.0, 4.0, 2.0, 3.0]], np.float32), fjo.F32, 2, True)
    den = 1.0 + math.exp(-1.0)
    assert_relative(v, [1.0 / den, math.exp(-1.0) / den], 1e-6)
    assert i.ravel().tolist() == [1, 3]


# ---- crates/forja-cpu/src/lib.rs:2689-2757 -----------------------------------------------------

def test_normalizes_1024_wide_rows_with_epsilon():
    values = np.concatenate([np.full(1024, 2.0), np.full(1024, -4.0), np.tile([3.0, 4.0], 512)]).astype(np.float32).reshape(3, 1024)
    out = fjo.rms_norm(values, fjo.F32, np.full(1024, 0.5, np.float32), fjo.F32, 0.25)
    expected = np.concatenate([np.full(1024, 1.0 / math.sqrt(4.25)), np.full(1024, -2.0 / math.sqrt(16.25)),
                               np.tile([1.5 / math.sqrt(12.75), 2.0 / math.sqrt(12.75)], 512)])
    assert_relative(out, expected, 1e-5)
    # the guest-program form (blocks.rs:392-400) agrees with the trusted op
    assert_relative(fjo.prog_rms_norm(values, fjo.F32, np.full(1024, 0.5, np.float32), fjo.F32, 0.25), expected, 1e-5)


def test_rope_identity_rotation_and_independent_f64_check():
    x = np.array([1.0, -2.0, 3.0, -4.0], np.float32).reshape(1, 1, 4)
    assert fjo.rope(x, fjo.F32, [0], 10000.0).ravel().tolist() == [1.0, -2.0, 3.0, -4.0]
    got = fjo.rope(np.array([1.0, 2.0, 3.0, 4.0], np.float32).reshape(1, 1, 4), fjo.F32, [1], 100.0)
    c1, s1, c2, s2 = math.cos(1.0), math.sin(1.0), math.cos(0.1), math.sin(0.1)
    assert_relative(got, [c1 - 3 * s1, 2 * c2 - 4 * s2, 3 * c1 + s1, 4 * c2 + 2 * s2], 1e-5)
    values = ((np.arange(14336) % 33).astype(np.float32) / 16.0 - 1.0).reshape(7, 16, 128)
    got = fjo.rope(values, fjo.F32, np.arange(7), 1e6)
    idx = np.arange(64, dtype=np.float64)
    angle = np.arange(7, dtype=np.float64)[:, None, None] / (1e6 ** (2.0 * idx / 128.0))[None, None, :]
    first, second = values[..., :64].astype(np.float64), values[..., 64:].astype(np.float64)
    expected = np.concatenate([first * np.cos(angle) - second * np.sin(angle), second * np.cos(angle) + first * np.sin(angle)], axis=-1)
    assert_relative(got, expected.astype(np.float32), 1e-5)


# ---- crates/forja-cpu/src/lib.rs:3041-3153 -----------------------------------------------------

def test_matmul_accepts_a_permuted_weight_view_and_sdpa_decode_equals_last_prefill_row():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 1024)).astype(np.float32)
    w = rng.standard_normal((96, 1024)).astype(np.float32)  # stored [out, in], used as its transpose
    a = fjo.matmul(x, fjo.F32, np.ascontiguousarray(w.T), fjo.F32, fjo.F32)
    b = fjo.matmul(x, fjo.F32, w, fjo.F32, fjo.F32, right_transposed=True)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert_relative(a, x.astype(np.float64) @ w.T.astype(np.float64), 1e-4)
    q = rng.standard_normal((16, 5, 128)).astype(np.float32)
    k = rng.standard_normal((8, 5, 128)).astype(np.float32)
    v = rng.standard_normal((8, 5, 128)).astype(np.float32)
    full = fjo.sdpa(q, fjo.F32, k, fjo.F32, v, fjo.F32, 0.088, True, 0)
    last = fjo.sdpa(q[:, 4:5], fjo.F32, k, fjo.F32, v, fjo.F32, 0.088, True, 4)
    assert np.array_equal(full[:, 4:5].view(np.uint32), last.view(np.uint32))


# ---- crates/forja-cpu/src/interpreter.rs:437-609 -----------------------------------------------

def _run(kind, build, shape, inputs, dts):
    p = fjo.Program(kind)
    p.output(0, build(p))
    return fjo.program(p, shape, inputs, dts, [fjo.F32])[0]


def test_interpreter_reductions_casts_and_corner_cases():
    row = np.array([1e20, -1e20, 3.0], np.float32)
    assert _run(fjo.ROW, lambda p: p.reduce(fjo.R_SUM, p.input(0)), (3,), [row], [fjo.F32]).tolist() == [3.0, 3.0, 3.0]

    def later(p):
        a = p.input(0)
        s = p.reduce(fjo.R_SUM, a)
        return p.reduce(fjo.R_SUM, p.binary(fjo.B_MUL, a, s))
    assert _run(fjo.ROW, later, (3,), [np.array([1, 2, 3], np.float32)], [fjo.F32]).tolist() == [36.0] * 3
    for op in (fjo.R_MIN, fjo.R_MAX):
        out = _run(fjo.ROW, lambda p: p.reduce(op, p.input(0)), (3,), [np.array([1.0, np.nan, 2.0], np.float32)], [fjo.F32])
        assert np.all(np.isnan(out))
    casted = _run(fjo.MAP, lambda p: p.cast(fjo.V_F32, p.cast(fjo.V_U32, p.input(0))), (3,), [np.array([np.nan, -1.0, np.inf], np.float32)], [fjo.F32])
    assert casted.tolist() == [0.0, 0.0, 4294967296.0]

    def wrapped(p):
        return p.cast(fjo.V_F32, p.binary(fjo.B_ADD, p.input(0), p.extent(0)))
    assert _run(fjo.MAP, wrapped, (1,), [np.array([0xFFFFFFFF], np.uint32)], [fjo.U32]).tolist() == [0.0]

    def coords(p):
        return p.cast(fjo.V_F32, p.binary(fjo.B_ADD, p.index(0), p.extent(0)))
    assert _run(fjo.MAP, coords, (1,), [], []).tolist() == [1.0]

    def select(p):
        z0, z1 = p.constant(0.0), p.constant(0.0)
        nan = p.binary(fjo.B_DIV, z0, z1)
        one = p.constant(1.0)
        cond = p.binary(fjo.B_EQ, z0, z0)
        return p.select(cond, one, nan)
    assert _run(fjo.MAP, select, (1,), [], []).tolist() == [1.0]
    inf = _run(fjo.MAP, lambda p: p.binary(fjo.B_DIV, p.constant(1.0), p.input(0)), (1,), [np.zeros(1, np.float32)], [fjo.F32])
    assert np.isposinf(inf[0])
    nan = _run(fjo.MAP, lambda p: p.binary(fjo.B_POW, p.input(0), p.input(1)), (1,), [np.array([-2.0], np.float32), np.array([0.5], np.float32)], [fjo.F32, fjo.F32])
    assert np.isnan(nan[0])
    mn = _run(fjo.MAP, lambda p: p.binary(fjo.B_MIN, p.input(0), p.constant(1.0)), (1,), [np.array([np.nan], np.float32)], [fjo.F32])
    assert np.isnan(mn[0])
    x = np.array([1e-20, -1e-20, 0.0, -0.0, -1.0, -2.0], np.float32)
    lp = _run(fjo.MAP, lambda p: p.unary(fjo.U_LOG1P, p.input(0)), (6,), [x], [fjo.F32])
    assert np.array_equal(lp[:4].view(np.uint32), x[:4].view(np.uint32)) and np.isneginf(lp[4]) and np.isnan(lp[5])


# ---- guest programs: direct restatements == interpreter on the reference's IR ------------------
# IR from support/forja-testing/src/representative.rs:7-126

def _ir_rms_norm(eps, axis):
    p = fjo.Program(fjo.ROW)
    v, w = p.input(0), p.input(1)
    s = p.reduce(fjo.R_SUM, p.binary(fjo.B_MUL, v, v))
    mean = p.binary(fjo.B_DIV, s, p.cast(fjo.V_F32, p.extent(axis)))
    inv = p.unary(fjo.U_RSQRT, p.binary(fjo.B_ADD, mean, p.constant(eps)))
    p.output(0, p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, v, inv), w))
    return p


def _ir_residual_norm(eps, axis):
    p = fjo.Program(fjo.ROW)
    r, u, w = p.input(0), p.input(1), p.input(2)
    v = p.binary(fjo.B_ADD, r, u)
    s = p.reduce(fjo.R_SUM, p.binary(fjo.B_MUL, v, v))
    mean = p.binary(fjo.B_DIV, s, p.cast(fjo.V_F32, p.extent(axis)))
    inv = p.unary(fjo.U_RSQRT, p.binary(fjo.B_ADD, mean, p.constant(eps)))
    p.output(0, v)
    p.output(1, p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, v, inv), w))
    return p


def _ir_qk_norm_rope(eps, theta, head_dim):
    p = fjo.Program(fjo.ROW)
    a, b, wa, wb, pos = (p.input(i) for i in range(5))
    sq = p.binary(fjo.B_ADD, p.binary(fjo.B_MUL, a, a), p.binary(fjo.B_MUL, b, b))
    s = p.reduce(fjo.R_SUM, sq)
    mean = p.binary(fjo.B_DIV, s, p.constant(head_dim))
    inv = p.unary(fjo.U_RSQRT, p.binary(fjo.B_ADD, mean, p.constant(eps)))
    a = p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, a, inv), wa)
    b = p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, b, inv), wb)
    freq = p.cast(fjo.V_F32, p.index(2))
    expo = p.binary(fjo.B_MUL, freq, p.constant(-2.0 / head_dim))
    scale = p.binary(fjo.B_POW, p.constant(theta), expo)
    angle = p.binary(fjo.B_MUL, pos, scale)
    c, s_ = p.unary(fjo.U_COS, angle), p.unary(fjo.U_SIN, angle)
    p.output(0, p.binary(fjo.B_SUB, p.binary(fjo.B_MUL, a, c), p.binary(fjo.B_MUL, b, s_)))
    p.output(1, p.binary(fjo.B_ADD, p.binary(fjo.B_MUL, b, c), p.binary(fjo.B_MUL, a, s_)))
    return p


@pytest.mark.parametrize("dt", [fjo.F32, fjo.BF16])
def test_direct_program_restatements_are_bit_identical_to_the_interpreter(dt):
    rng = np.random.default_rng(11)
    rows, width = 5, 96
    x = fjo.encode(rng.standard_normal((rows, width)).astype(np.float32), dt)
    u = fjo.encode(rng.standard_normal((rows, width)).astype(np.float32), dt)
    w = fjo.encode(1.0 + 0.02 * rng.standard_normal(width).astype(np.float32), dt)
    a, = fjo.program(_ir_rms_norm(1e-6, 1), (rows, width), [x, w], [dt, dt], [dt])
    assert np.array_equal(a.view(np.uint8), fjo.prog_rms_norm(x, dt, w, dt, 1e-6).view(np.uint8))
    s, n = fjo.program(_ir_residual_norm(1e-6, 1), (rows, width), [x, u, w], [dt, dt, dt], [dt, dt])
    s2, n2 = fjo.prog_residual_norm(x, u, dt, w, dt, 1e-6)
    assert np.array_equal(s.view(np.uint8), s2.view(np.uint8)) and np.array_equal(n.view(np.uint8), n2.view(np.uint8))
    # qk-norm + rope over [tokens, heads, 128] split into lo/hi halves (blocks.rs:181-226, 419-444)
    t, h, d = 3, 4, 128
    q = fjo.encode(rng.standard_normal((t, h, d)).astype(np.float32), dt)
    wq = fjo.encode(1.0 + 0.1 * rng.standard_normal(d).astype(np.float32), dt)
    pos = np.array([0.0, 17.0, 4099.0], np.float32)
    lo, hi = fjo.program(_ir_qk_norm_rope(1e-6, 1e6, 128.0), (t, h, d // 2),
                         [q[..., :64], q[..., 64:], wq[:64], wq[64:], pos[:, None, None]], [dt, dt, dt, dt, fjo.F32], [dt, dt])
    direct = fjo.prog_qk_norm_rope(q, dt, wq, dt, pos, 1e-6, 1e6)
    assert np.array_equal(np.concatenate([lo, hi], axis=-1).view(np.uint8), direct.view(np.uint8))
    # silu_mul / add maps (representative.rs:106-126)
    p = fjo.Program(fjo.MAP)
    g, up = p.input(0), p.input(1)
    p.output(0, p.binary(fjo.B_MUL, p.binary(fjo.B_MUL, g, p.unary(fjo.U_SIGMOID, g)), up))
    m, = fjo.program(p, (rows, width), [x, u], [dt, dt], [dt])
    assert np.array_equal(m.view(np.uint8), fjo.prog_silu_mul(x, u, dt).view(np.uint8))


# ---- greedy selection: crates/forja-cpu/src/lib.rs:1597-1613 -----------------------------------

def test_greedy_sample_equals_argmax_and_seeded_sampling_is_reproducible():
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((4, 1000)).astype(np.float32)
    logits[1, 10] = logits[1, 500] = 9.0
    greedy = fjo.sample(logits, fjo.F32, [bits(0.0), 0, bits(1.0), 1, 2], position=3)
    assert np.array_equal(greedy, fjo.argmax(logits, fjo.F32))
    params = [bits(0.8), 40, bits(0.95), 123, 456]
    a = fjo.sample(logits, fjo.F32, params, position=7)
    assert np.array_equal(a, fjo.sample(logits, fjo.F32, params, position=7))
    allow = np.zeros(32, np.uint32)
    allow[0] = 0b1010
    masked = fjo.sample(logits, fjo.F32, params, position=7, allow=allow)
    assert set(masked.tolist()) <= {1, 3}
    with pytest.raises(fjo.OracleError):
        fjo.sample(logits, fjo.F32, [bits(-1.0), 0, bits(1.0), 0, 0], position=0)


# ---- further known answers of the reference's backend tests -------------------------------------------------------------

def test_copies_permuted_attention_heads_to_contiguous_bf16():  # lib.rs:2345-2371
    values = np.arange(7 * 16 * 128, dtype=np.float32).reshape(7, 16, 128)
    got = fjo.copy(np.ascontiguousarray(values.transpose(1, 0, 2)), fjo.F32, fjo.BF16)
    want = fjo.encode(np.ascontiguousarray(values.transpose(1, 0, 2)), fjo.BF16)
    assert got.shape == (16, 7, 128) and np.array_equal(got, want)
    # index (sequence * 16 + head) * 128 + column, rounded to bf16 with ties to even: 257 -> 256, 259 -> 260
    assert fjo.decode(got, fjo.BF16)[2, 0, 1] == 256.0 and fjo.decode(got, fjo.BF16)[2, 0, 3] == 260.0


def test_matmul_handles_unit_contraction_and_row_dimensions():  # lib.rs:3080-3092
    got = fjo.matmul(np.array([[2.0], [3.0]], np.float32), fjo.F32, np.array([[4.0, 5.0, 6.0]], np.float32), fjo.F32, fjo.F32)
    assert got.ravel().tolist() == [8.0, 10.0, 12.0, 12.0, 15.0, 18.0]
    left = np.array([1.0, 2.0, 3.0, 4.0], np.float32).reshape(2, 1, 2)
    right = np.array([5.0, 6.0, 7.0, 8.0], np.float32).reshape(2, 2, 1)
    assert fjo.matmul(left, fjo.F32, right, fjo.F32, fjo.F32).ravel().tolist() == [17.0, 53.0]


def test_matmul_with_bias_epilogue_inputs_sums_in_index_order():  # lib.rs:1985-2070 (the fused and the decomposed form share this sum)
    left = (np.arange(7 * 33, dtype=np.float32) / np.float32(97.0) - np.float32(1.0)).reshape(7, 33)
    right = (np.arange(33 * 17, dtype=np.float32) / np.float32(113.0) - np.float32(2.0)).reshape(33, 17)
    bias = np.arange(17, dtype=np.float32) / np.float32(17.0)
    acc = fjo.matmul(left, fjo.F32, right, fjo.F32, fjo.F32)
    want = np.zeros((7, 17), np.float32)
    for k in range(33):  # k ascending, product rounded, then added
        want = (want + (left[:, k:k + 1] * right[k:k + 1, :]).astype(np.float32)).astype(np.float32)
    assert np.array_equal(acc.view(np.uint32), want.view(np.uint32))
    fused = fjo.prog_add(acc, np.broadcast_to(bias, (7, 17)).copy(), fjo.F32)
    assert np.array_equal(fused.view(np.uint32), (want + bias).astype(np.float32).view(np.uint32))


def test_embeds_rows_near_both_ends_of_a_1024_wide_table():  # lib.rs:2760-2783
    values = (np.arange(1000 * 1024) % 251).astype(np.float32).reshape(1000, 1024)
    ids = np.array([0, 1, 998, 999], np.uint32)
    assert np.array_equal(fjo.embed(values, fjo.F32, ids), values[ids])


def test_sdpa_hand_checked_two_key_case_and_grouped_heads():  # lib.rs:3095-3153
    q = np.array([1.0, 0.0], np.float32).reshape(1, 1, 2)
    k = np.array([1.0, 0.0, 0.0, 1.0], np.float32).reshape(1, 2, 2)
    v = np.array([10.0, 20.0], np.float32).reshape(1, 2, 1)
    e = np.exp(np.float32(1.0))
    got = fjo.sdpa(q, fjo.F32, k, fjo.F32, v, fjo.F32, 1.0, False, 0)
    assert abs(float(got.ravel()[0]) - float((10.0 * e + 20.0) / (e + 1.0))) <= 1e-5 * 20
    # 16 query heads over 8 cache heads, 7 keys of width 128, all-zero keys: every query head returns its cache head's value
    keys = np.zeros((8, 7, 128), np.float32)
    values = np.repeat(np.arange(8, dtype=np.float32), 7 * 128).reshape(8, 7, 128)
    got = fjo.sdpa(np.zeros((16, 1, 128), np.float32), fjo.F32, keys, fjo.F32, values, fjo.F32, float(1.0 / np.sqrt(np.float32(128.0))), True, 6)
    assert np.allclose(got.ravel(), np.repeat(np.arange(8, dtype=np.float32), 2 * 128), rtol=1e-5)
    # a causal window that would reach past the cache is refused
    key = np.array([1.0, 0.0, 0.0, 1.0, 1.0, 1.0, -1.0, 1.0], np.float32).reshape(1, 4, 2)
    with pytest.raises(fjo.OracleError):
        fjo.sdpa(np.array([7.0, 8.0], np.float32).reshape(1, 1, 2), fjo.F32, key, fjo.F32, key, fjo.F32, 0.5, True, 4)


def test_paged_lane_activity_defaults_active_and_reads_u32():  # lib.rs:1973-1982
    """No activity word = active; 0 = inactive (zeros out, nothing copied); any other value (7) = active."""
    page = 16
    table = np.array([[0, 0]], np.uint32)
    generations = np.zeros(2, np.uint32)
    rows = fjo.encode(np.arange(4 * 8, dtype=np.float32).reshape(4, 8), fjo.F32)
    for activity, written in ((None, True), (0, False), (7, True)):
        pool = np.zeros((2, page, 8), np.float32)
        fjo.paged_copy_in(rows, fjo.F32, pool, fjo.F32, table, generations, 0, page, activity=activity)
        assert bool(np.any(pool != 0.0)) == written
