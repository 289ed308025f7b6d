"""GPU parity: dense and quantised projections through the C ABI against the CPU oracle, on the
reference's own test shapes (rows 1/7/33, K 64/768/2048/4096, odd columns 33/65) plus the
benchmark shapes at sizes the scalar oracle finishes quickly."""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200.backend import Op
from oracle import fjo
from tests import ir_programs as ir
from tests.gpu_util import QUANT_TOL, TOL, assert_close, backend, down, down_raw, max_abs_rel, up, up_u32

pytestmark = pytest.mark.gpu


def prepare(prog):
    insts, outs = prog.words()
    return backend().prepare_program(prog.kind, insts, outs)


@pytest.mark.parametrize("dt", [fb.F32, fb.BF16, fb.F16])
@pytest.mark.parametrize("m,k,n", [(1, 64, 33), (7, 768, 65), (33, 2048, 96), (1, 1024, 3072), (8, 576, 192), (64, 1024, 640), (128, 1024, 4096),
                                   (130, 3072, 1024), (300, 576, 1536), (512, 2048, 257)])
def test_matmul_with_transposed_weight_view(dt, m, k, n):
    """Weight stored [out, in] and used through a permuted view (crates/forja-cpu/src/lib.rs:3041-3077)."""
    rng = np.random.default_rng(m * 7 + n)
    be = backend()
    x, xh = up(rng.standard_normal((m, k)), dt)
    w, wh = up(rng.standard_normal((n, k)) * 0.05, dt)
    out = be.alloc(dt, (m, n))
    be.run(Op.Matmul(), [x, w.permute([1, 0])], [out])
    want = fjo.matmul(xh, dt, wh, dt, dt, right_transposed=True)
    if dt == fb.F32:
        # one thread per output, k ascending, separate multiply and add: the reference's sum bit for bit
        assert np.array_equal(down_raw(out).view(np.uint32), want.view(np.uint32))
    else:
        assert_close(down(out), fjo.decode(want, dt), TOL[dt])


@pytest.mark.parametrize("dt", [fb.BF16, fb.F16])
@pytest.mark.parametrize("m,k,n", [(2048, 256, 1280), (300, 128, 8000), (128, 1024, 19000), (4096, 64, 600), (1500, 1984, 1666)])
def test_large_grids_run_on_tensor_memory_tiles(dt, m, k, n):
    """At least one 128 x 128 output tile per SM and K a multiple of 64: the tcgen05 kernel (TMEM accumulators);
    ragged M and N edges, one to 31 k steps. None of its bounded waits may run out."""
    rng = np.random.default_rng(m + k + n)
    be = backend()
    x, xh = up(rng.standard_normal((m, k)), dt)
    w, wh = up(rng.standard_normal((n, k)) * 0.05, dt)
    out = be.alloc(dt, (m, n))
    be.run(Op.Matmul(), [x, w.permute([1, 0])], [out])
    assert be.tcgen05_wait_giveups() == 0
    fjo.set_threads(fjo.max_threads())
    want = fjo.matmul(xh, dt, wh, dt, dt, right_transposed=True)
    fjo.set_threads(1)
    assert_close(down(out), fjo.decode(want, dt), TOL[dt])


def test_matmul_generic_layouts_and_batches():
    rng = np.random.default_rng(2)
    be = backend()
    a, ah = up(rng.standard_normal((3, 5, 16)), fb.F32)
    b, bh = up(rng.standard_normal((3, 16, 9)), fb.F32)
    out = be.alloc(fb.F32, (3, 5, 9))
    be.run(Op.Matmul(), [a, b], [out])
    assert np.array_equal(down_raw(out).view(np.uint32), fjo.matmul(ah, fjo.F32, bh, fjo.F32, fjo.F32).view(np.uint32))
    # row-major right operand [K, N] in bf16 (not the transposed fast path)
    x, xh = up(rng.standard_normal((7, 64)), fb.BF16)
    w, wh = up(rng.standard_normal((64, 33)), fb.BF16)
    out = be.alloc(fb.BF16, (7, 33))
    be.run(Op.Matmul(), [x, w], [out])
    assert_close(down(out), fjo.decode(fjo.matmul(xh, fjo.BF16, wh, fjo.BF16, fjo.BF16), fjo.BF16), TOL[fb.BF16])


def test_tied_lm_head_shape_argmax_agrees():
    """Qwen3-0.6B lm_head: 1024 -> 151936 through the transposed embedding table, then greedy argmax."""
    rng = np.random.default_rng(9)
    be = backend()
    m, k, n = 4, 1024, 151936
    x, xh = up(rng.standard_normal((m, k)), fb.BF16)
    w, wh = up(rng.standard_normal((n, k)) * 0.02, fb.BF16)
    out = be.alloc(fb.BF16, (m, n))
    be.run(Op.Matmul(), [x, w.permute([1, 0])], [out])
    fjo.set_threads(fjo.max_threads())
    want = fjo.matmul(xh, fjo.BF16, wh, fjo.BF16, fjo.BF16, right_transposed=True)
    fjo.set_threads(1)
    got = down(out)
    assert max_abs_rel(got, fjo.decode(want, fjo.BF16)) <= 2e-2
    assert_close(got, fjo.decode(want, fjo.BF16), TOL[fb.BF16])


# ---- MLX affine group quantisation -------------------------------------------------------------

def quant_weights(rng, n, k, bits, group, p_dt, experts=None):
    shape = (n, k * bits // 32) if experts is None else (experts, n, k * bits // 32)
    gshape = (n, k // group) if experts is None else (experts, n, k // group)
    packed = rng.integers(0, 2 ** 32, shape, dtype=np.uint64).astype(np.uint32)  # uniform nibbles 0..15
    scales = fjo.encode((rng.standard_normal(gshape) * 0.01).astype(np.float32), p_dt)
    biases = fjo.encode((rng.standard_normal(gshape) * 0.01).astype(np.float32), p_dt)
    return packed, scales, biases


@pytest.mark.parametrize("bits,p_dt", [(4, fb.BF16), (8, fb.F16)])
@pytest.mark.parametrize("rows", [1, 7, 33])
def test_quant_matmul_known_answer_in_mlx_order(bits, p_dt, rows):
    # crates/forja-cpu/src/lib.rs:2786-2845
    be = backend()
    inner = 64
    act = (np.arange(rows * inner) % 17).astype(np.float32) / 8.0 - 1.0
    repeats = inner * bits // 32
    pattern = 0x11111111 if bits == 4 else 0x01010101
    maximum = (1 << bits) - 1
    words = np.repeat(np.array([0, pattern, pattern * maximum], np.uint64), repeats).astype(np.uint32).reshape(3, repeats)
    sv, bv = [0.5, -0.25, 0.125], [1.0, 2.0, -1.0]
    x = be.tensor_from(act.reshape(rows, inner), fb.F32)
    pk, _ = up_u32(words)
    sc, _ = up(np.array(sv).reshape(3, 1), p_dt)
    bi, _ = up(np.array(bv).reshape(3, 1), p_dt)
    out = be.alloc(fb.F32, (rows, 3))
    be.run(Op.QuantMatmul(bits, 64), [x, pk, sc, bi], [out])
    sums = act.reshape(rows, inner).astype(np.float64).sum(axis=1)
    expected = np.stack([sums * bv[0], sums * (sv[1] + bv[1]), sums * (sv[2] * maximum + bv[2])], axis=1)
    got = down(out)
    assert np.all(np.abs(got - expected) <= 1e-5 * np.maximum(1.0, np.abs(expected)))


@pytest.mark.parametrize("x_dt", [fb.BF16, fb.F16, fb.F32])
@pytest.mark.parametrize("bits,group", [(4, 64), (8, 64), (4, 32), (4, 128)])
@pytest.mark.parametrize("m,k,n", [(1, 2048, 768), (8, 4096, 512), (7, 768, 2048), (33, 2048, 130), (64, 2048, 384), (12, 4096, 264), (16, 1024, 6144), (300, 1024, 2048)])
def test_quant_matmul_matches_oracle(x_dt, bits, group, m, k, n):
    rng = np.random.default_rng(m + k + n + bits + group)
    be = backend()
    packed, scales, biases = quant_weights(rng, n, k, bits, group, fb.BF16)
    x, xh = up(rng.standard_normal((m, k)), x_dt)
    pk, _ = up_u32(packed)
    sc, bi = be.tensor_from(scales, fb.BF16), be.tensor_from(biases, fb.BF16)
    out = be.alloc(x_dt, (m, n))
    be.run(Op.QuantMatmul(bits, group), [x, pk, sc, bi], [out])
    fjo.set_threads(fjo.max_threads())
    want = fjo.decode(fjo.quant_matmul(xh, x_dt, packed, scales, biases, fjo.BF16, bits, group, x_dt), x_dt)
    fjo.set_threads(1)
    assert_close(down(out), want, QUANT_TOL)
    assert max_abs_rel(down(out), want) <= 2e-2


def test_gather_quant_matmul_known_answers():
    # crates/forja-cpu/src/lib.rs:2848-2951
    be = backend()
    x = be.tensor_from(np.ones((1, 64), np.float32), fb.F32)
    packed = np.repeat((np.arange(6, dtype=np.uint64) * 0x11111111).astype(np.uint32), 8).reshape(3, 2, 8)
    pk, _ = up_u32(packed)
    sc, _ = up(np.ones((3, 2, 1)), fb.BF16)
    bi, _ = up(np.zeros((3, 2, 1)), fb.BF16)
    idx, _ = up_u32(np.array([[2, 0, 2]]))
    out = be.alloc(fb.F32, (1, 3, 2))
    be.run(Op.GatherQuantMatmul(4, 64), [x, pk, sc, bi, idx], [out])
    assert down(out).ravel().tolist() == [256.0, 320.0, 0.0, 64.0, 256.0, 320.0]
    fused = be.alloc(fb.F32, (1, 3, 2))
    be.run(Op.GatherQuantMatmul(4, 64, epilogue=prepare(ir.silu_mul())), [x, pk, sc, bi, pk, sc, bi, idx], [fused])
    expected = [v / (1.0 + np.exp(-v)) * v for v in [256.0, 320.0, 0.0, 64.0, 256.0, 320.0]]
    assert_close(down(fused), expected, 1e-5)
    bad, _ = up_u32(np.array([[99, 7]]))
    out = be.alloc(fb.F32, (1, 2, 2))
    with pytest.raises(fb.BackendError) as e:
        be.run(Op.GatherQuantMatmul(4, 64), [x, pk, sc, bi, bad], [out])
    assert e.value.status == fb.backend.INDEX_OUT_OF_RANGE and e.value.index == 7
    assert not down(out).any()


def test_gather_quant_weighted_sum_known_answer():
    # crates/forja-cpu/src/lib.rs:2954-3017
    be = backend()
    act = be.tensor_from(np.repeat(np.arange(1, 6, dtype=np.float32), 64).reshape(1, 5, 64), fb.F32)
    pk, _ = up_u32(np.repeat((np.arange(1, 7, dtype=np.uint64) * 0x11111111).astype(np.uint32), 8).reshape(3, 2, 8))
    sc, _ = up(np.full((3, 2, 1), 0.5), fb.BF16)
    bi, _ = up(np.full((3, 2, 1), 0.25), fb.BF16)
    idx, _ = up_u32(np.array([[2, 99, 0, 7, 1]]))
    wts = be.tensor_from(np.array([[0.5, 1.0, -0.25, 2.0, 0.75]], np.float32), fb.F32)
    residual = be.tensor_from(np.array([[1.5, -2.0]], np.float32), fb.F32)
    out = be.alloc(fb.F32, (1, 2))
    with pytest.raises(fb.BackendError) as e:
        be.run(Op.GatherQuantMatmul(4, 64, epilogue=prepare(ir.add())), [act, pk, sc, bi, idx, wts, residual], [out])
    assert e.value.index == 7
    assert down(out).ravel().tolist() == [473.5, 582.0]


# 1 and 7 rows x 8 routes: one pass per route. 8 to 100 rows (64 to 800 routes, fewer than 72 per expert): routes bucketed by
# expert into 16-row tiles that stream the expert's weights (8-row and 16-row forms, experts with several tiles).
# 200 and 300 rows (100 / 150 per expert): 128-row tiles on the tcgen05 tensor cores, with experts that need a second, ragged tile.
@pytest.mark.parametrize("rows", [1, 7, 8, 16, 33, 47, 100, 200, 300])
def test_moe_expert_projections_match_oracle(rows):
    """Qwen3-30B-A3B expert shapes at a reduced expert count: gate/up pair 2048 -> 768 with the
    gate*sigmoid(gate)*up epilogue, then the weighted down projection 768 -> 2048 plus residual
    (engines/qwen3-coder/src/lib.rs:505-603)."""
    rng = np.random.default_rng(rows)
    be = backend()
    experts, hidden, inter, top_k = 16, 2048, 768, 8
    dt = fb.BF16
    g_pk, g_sc, g_bi = quant_weights(rng, inter, hidden, 4, 64, fb.BF16, experts)
    u_pk, u_sc, u_bi = quant_weights(rng, inter, hidden, 4, 64, fb.BF16, experts)
    d_pk, d_sc, d_bi = quant_weights(rng, hidden, inter, 4, 64, fb.BF16, experts)
    x, xh = up(rng.standard_normal((rows, hidden)), dt)
    logits = rng.standard_normal((rows, experts)).astype(np.float32)
    wv, wi = fjo.top_k(logits, fjo.F32, top_k, True)
    idx, _ = up_u32(wi)
    wts, wth = up(wv, dt)
    res, resh = up(rng.standard_normal((rows, hidden)), dt)
    t = lambda a, d: be.tensor_from(a, d)
    act = be.alloc(dt, (rows, top_k, inter))
    be.run(Op.GatherQuantMatmul(4, 64, epilogue=prepare(ir.silu_mul())),
           [x, t(g_pk, fb.U32), t(g_sc, fb.BF16), t(g_bi, fb.BF16), t(u_pk, fb.U32), t(u_sc, fb.BF16), t(u_bi, fb.BF16), idx], [act])
    fjo.set_threads(fjo.max_threads())
    gate = fjo.gather_quant_matmul(xh, dt, g_pk, g_sc, g_bi, fjo.BF16, wi, 4, 64, fjo.F32)
    upp = fjo.gather_quant_matmul(xh, dt, u_pk, u_sc, u_bi, fjo.BF16, wi, 4, 64, fjo.F32)
    want_act = fjo.prog_silu_mul(gate, upp, fjo.F32, dt)
    assert_close(down(act), fjo.decode(want_act, dt), QUANT_TOL)
    out = be.alloc(dt, (rows, hidden))
    be.run(Op.GatherQuantMatmul(4, 64, epilogue=prepare(ir.add())), [act, t(d_pk, fb.U32), t(d_sc, fb.BF16), t(d_bi, fb.BF16), idx, wts, res], [out])
    acc = fjo.gather_quant_weighted_sum(down_raw(act), dt, d_pk, d_sc, d_bi, fjo.BF16, wi, wth, dt, 4, 64, fjo.F32)
    want = fjo.prog_add(acc, fjo.decode(resh, dt), fjo.F32, dt)
    fjo.set_threads(1)
    assert_close(down(out), fjo.decode(want, dt), QUANT_TOL)


@pytest.mark.parametrize("rows", [40, 80, 200])  # 160 and 320 routes: streamed 16-row tiles; 800: 128-row tcgen05 tiles
def test_bucketed_expert_path_zeroes_bad_routes_and_reports_the_lowest_id(rows):
    """Bucketed routes with two out-of-range expert ids: their rows are zero, every other row is computed,
    and the submission fails with the lowest offending id (crates/forja-cpu/src/lib.rs:1078-1088)."""
    rng = np.random.default_rng(5)
    be = backend()
    experts, hidden, inter, top_k = 8, 512, 128, 4
    dt = fb.BF16
    pk, sc, bi = quant_weights(rng, inter, hidden, 4, 64, fb.BF16, experts)
    x, xh = up(rng.standard_normal((rows, hidden)), dt)
    ids = rng.integers(0, experts, (rows, top_k)).astype(np.uint32)
    ids[3, 1], ids[17, 0] = 99, 77
    idx, _ = up_u32(ids)
    out = be.alloc(dt, (rows, top_k, inter))
    with pytest.raises(fb.BackendError) as info:
        be.run(Op.GatherQuantMatmul(4, 64), [x, be.tensor_from(pk, fb.U32), be.tensor_from(sc, fb.BF16), be.tensor_from(bi, fb.BF16), idx], [out])
    assert info.value.index == 77
    got = down(out)
    assert np.all(got[3, 1] == 0.0) and np.all(got[17, 0] == 0.0)
    good = ids.copy()
    good[3, 1], good[17, 0] = 0, 0
    want = fjo.decode(fjo.gather_quant_matmul(xh, dt, pk, sc, bi, fjo.BF16, good, 4, 64, dt), dt)
    mask = np.ones((rows, top_k), bool)
    mask[3, 1] = mask[17, 0] = False
    assert_close(got[mask], want[mask], QUANT_TOL)


@pytest.mark.parametrize("inter", [64, 96])  # one 64-column block; two blocks of which the second is ragged
def test_bucketed_expert_path_narrow_and_ragged_column_blocks(inter):
    """128-row tcgen05 tiles with an output narrower than, or not a multiple of, the column block."""
    rng = np.random.default_rng(inter)
    be = backend()
    experts, hidden, top_k, rows = 4, 256, 4, 128
    dt = fb.BF16
    pk, sc, bi = quant_weights(rng, inter, hidden, 4, 64, fb.BF16, experts)
    x, xh = up(rng.standard_normal((rows, hidden)), dt)
    ids = rng.integers(0, experts, (rows, top_k)).astype(np.uint32)
    idx, _ = up_u32(ids)
    out = be.alloc(dt, (rows, top_k, inter))
    be.run(Op.GatherQuantMatmul(4, 64), [x, be.tensor_from(pk, fb.U32), be.tensor_from(sc, fb.BF16), be.tensor_from(bi, fb.BF16), idx], [out])
    fjo.set_threads(fjo.max_threads())
    want = fjo.decode(fjo.gather_quant_matmul(xh, dt, pk, sc, bi, fjo.BF16, ids, 4, 64, dt), dt)
    fjo.set_threads(1)
    assert_close(down(out), want, QUANT_TOL)


@pytest.mark.parametrize("rows", [48, 96])  # 48 / 96 routes per expert: 64-row mma.sync tiles; 128-row tcgen05 tiles
def test_bucketed_expert_path_with_k_that_the_streamed_form_refuses(rows):
    """hidden = 320 is a multiple of the group size but not of the 256-k unit of the streamed form."""
    rng = np.random.default_rng(rows)
    be = backend()
    experts, hidden, inter, top_k = 4, 320, 128, 4
    dt = fb.BF16
    pk, sc, bi = quant_weights(rng, inter, hidden, 4, 64, fb.BF16, experts)
    x, xh = up(rng.standard_normal((rows, hidden)), dt)
    ids = rng.integers(0, experts, (rows, top_k)).astype(np.uint32)
    idx, _ = up_u32(ids)
    out = be.alloc(dt, (rows, top_k, inter))
    be.run(Op.GatherQuantMatmul(4, 64), [x, be.tensor_from(pk, fb.U32), be.tensor_from(sc, fb.BF16), be.tensor_from(bi, fb.BF16), idx], [out])
    fjo.set_threads(fjo.max_threads())
    want = fjo.decode(fjo.gather_quant_matmul(xh, dt, pk, sc, bi, fjo.BF16, ids, 4, 64, dt), dt)
    fjo.set_threads(1)
    assert_close(down(out), want, QUANT_TOL)


@pytest.mark.parametrize("dt,m,k,n", [(fb.F32, 7, 576, 1536), (fb.BF16, 33, 256, 192), (fb.BF16, 128, 1024, 3072), (fb.F32, 1, 64, 48)])
def test_matmul_epilogues_see_the_f32_accumulator(dt, m, k, n):
    """Op::Matmul with a scalar epilogue (crates/forja-cpu/src/lib.rs:443-493; SmolLM2's fused-epilogues tuning,
    engines/smollm2/src/optimized.rs:190-204): the Map program gets the unrounded accumulator and the extra operand and
    its result is rounded once. Oracle: matmul to f32, then the interpreted program."""
    rng = np.random.default_rng(m + n)
    be = backend()
    x, xh = up(rng.standard_normal((m, k)), dt)
    w, wh = up(rng.standard_normal((n, k)) * 0.05, dt)
    extra, eh = up(rng.standard_normal((m, n)), dt)
    fjo.set_threads(fjo.max_threads())
    acc = fjo.matmul(xh, dt, wh, dt, fjo.F32, right_transposed=True)
    fjo.set_threads(1)
    for name, prog in (("gated_up", ir.gated_up()), ("add", ir.add()), ("silu_mul", ir.silu_mul())):
        out = be.alloc(dt, (m, n))
        be.run(Op.Matmul(epilogue=prepare(prog)), [x, w.permute([1, 0]), extra], [out])
        want = fjo.program(prog, (m, n), [acc, eh], [fjo.F32, dt], [dt])[0]
        if dt == fb.F32:
            assert_close(down(out), want, 1e-5)
        else:
            assert_close(down(out), fjo.decode(want, dt), TOL[dt])
    # an epilogue the library does not know is refused, not emulated
    with pytest.raises(fb.BackendError) as e:
        be.run(Op.Matmul(epilogue=prepare(ir.rms_norm(1e-5))), [x, w.permute([1, 0]), extra], [be.alloc(dt, (m, n))])
    assert e.value.status in (fb.backend.UNSUPPORTED_OPERATION, fb.backend.INVALID_INPUT)


def test_quant_matmul_epilogue_adds_a_residual():
    rng = np.random.default_rng(12)
    be = backend()
    m, k, n = 5, 512, 256
    pk, sc, bi = quant_weights(rng, n, k, 4, 64, fb.BF16)
    x, xh = up(rng.standard_normal((m, k)), fb.BF16)
    res, rh = up(rng.standard_normal((m, n)), fb.BF16)
    out = be.alloc(fb.BF16, (m, n))
    be.run(Op.QuantMatmul(4, 64, epilogue=prepare(ir.add())), [x, be.tensor_from(pk, fb.U32), be.tensor_from(sc, fb.BF16), be.tensor_from(bi, fb.BF16), res], [out])
    acc = fjo.quant_matmul(xh, fb.BF16, pk, sc, bi, fb.BF16, 4, 64, fjo.F32)
    want = fjo.program(ir.add(), (m, n), [acc, rh], [fjo.F32, fb.BF16], [fb.BF16])[0]
    assert_close(down(out), fjo.decode(want, fb.BF16), QUANT_TOL)
