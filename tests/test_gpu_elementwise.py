"""GPU parity: copy, norms, guest programs, rope, embed, argmax, top-k through the C ABI against the
CPU oracle on the same seeded inputs (differential backend tests in the style of
support/forja-testing/src/lib.rs:610-681 and crates/forja-metal/tests/*.rs)."""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200.backend import CommandList, Op
from oracle import fjo
from tests import ir_programs as ir
from tests.gpu_util import TOL, assert_close, backend, down, down_raw, up, up_u32

pytestmark = pytest.mark.gpu

DTYPES = [fb.F32, fb.F16, fb.BF16]


def prepare(prog):
    insts, outs = prog.words()
    return backend().prepare_program(prog.kind, insts, outs)


@pytest.mark.parametrize("src,dst", [(fb.F32, fb.BF16), (fb.BF16, fb.F32), (fb.F32, fb.F16), (fb.F16, fb.BF16), (fb.F32, fb.F32)])
def test_copy_casts_and_follows_strided_views(src, dst):
    rng = np.random.default_rng(1)
    be = backend()
    x, xh = up(rng.standard_normal((6, 10, 8)) * 3, src)
    out = be.alloc(dst, (10, 6, 4))
    view = x.permute([1, 0, 2]).slice([(0, 10, 1), (0, 6, 1), (1, 4, 2)])
    be.run(Op.Copy(), [view], [out])
    want = fjo.copy(np.ascontiguousarray(xh.transpose(1, 0, 2)[:, :, 1::2]), src, dst)
    assert np.array_equal(down_raw(out).view(np.uint8), want.view(np.uint8))
    # scatter into a strided destination
    dest = be.alloc(dst, (6, 10, 8))
    be.run(Op.Copy(), [view], [dest.permute([1, 0, 2]).slice([(0, 10, 1), (0, 6, 1), (0, 4, 2)])])
    got = down_raw(dest)
    assert np.array_equal(np.ascontiguousarray(got.transpose(1, 0, 2)[:, :, 0:8:2]).view(np.uint8), want.view(np.uint8))
    assert not np.ascontiguousarray(got[:, :, 1::2]).view(np.uint8).any()


def test_copy_moves_u32_bits():
    be = backend()
    x, xh = up_u32(np.arange(24).reshape(4, 6) * 0x01010101)
    out = be.alloc(fb.U32, (6, 4))
    be.run(Op.Copy(), [x.permute([1, 0])], [out])
    assert np.array_equal(down_raw(out), xh.T)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 64), (7, 576), (33, 1024), (3, 2048), (2, 33)])
def test_rms_norm_op_and_program(dt, rows, width):
    rng = np.random.default_rng(rows * 1000 + width)
    be = backend()
    x, xh = up(rng.standard_normal((rows, width)), dt)
    w, wh = up(1.0 + 0.1 * rng.standard_normal(width), dt)
    out = be.alloc(dt, (rows, width))
    be.run(Op.RmsNorm(1e-5), [x, w], [out])
    assert_close(down(out), fjo.decode(fjo.rms_norm(xh, dt, wh, dt, 1e-5), dt), TOL[dt])
    handle = prepare(ir.rms_norm(1e-6))
    out2 = be.alloc(dt, (rows, width))
    be.run(Op.Program(handle), [x, w.broadcast((rows, width))], [out2])
    assert_close(down(out2), fjo.decode(fjo.prog_rms_norm(xh, dt, wh, dt, 1e-6), dt), TOL[dt])


def test_rms_norm_known_answer():
    # crates/forja-cpu/src/lib.rs:2689-2711
    be = backend()
    values = np.concatenate([np.full(1024, 2.0), np.full(1024, -4.0), np.tile([3.0, 4.0], 512)]).reshape(3, 1024)
    x, _ = up(values, fb.F32)
    w, _ = up(np.full(1024, 0.5), fb.F32)
    out = be.alloc(fb.F32, (3, 1024))
    be.run(Op.RmsNorm(0.25), [x, w], [out])
    expected = np.concatenate([np.full(1024, 1.0 / np.sqrt(4.25)), np.full(1024, -2.0 / np.sqrt(16.25)), np.tile([1.5 / np.sqrt(12.75), 2.0 / np.sqrt(12.75)], 512)])
    assert_close(down(out), expected, 1e-5)


@pytest.mark.parametrize("dt", DTYPES)
def test_residual_norm_add_and_silu_mul_programs(dt):
    rng = np.random.default_rng(7)
    be = backend()
    rows, width = 9, 1024
    r, rh = up(rng.standard_normal((rows, width)), dt)
    u, uh = up(rng.standard_normal((rows, width)), dt)
    w, wh = up(1.0 + 0.1 * rng.standard_normal(width), dt)
    total, norm = be.alloc(dt, (rows, width)), be.alloc(dt, (rows, width))
    be.run(Op.Program(prepare(ir.residual_norm(1e-6))), [r, u, w.broadcast((rows, width))], [total, norm])
    want_total, want_norm = fjo.prog_residual_norm(rh, uh, dt, wh, dt, 1e-6)
    # the sum is a single f32 addition rounded once: bit-exact
    assert np.array_equal(down_raw(total).view(np.uint8), want_total.view(np.uint8))
    assert_close(down(norm), fjo.decode(want_norm, dt), TOL[dt])
    out = be.alloc(dt, (rows, width))
    be.run(Op.Program(prepare(ir.add())), [r, u], [out])
    assert np.array_equal(down_raw(out).view(np.uint8), fjo.prog_add(rh, uh, dt).view(np.uint8))
    out = be.alloc(dt, (rows, width))
    be.run(Op.Program(prepare(ir.silu_mul())), [r, u], [out])
    assert_close(down(out), fjo.decode(fjo.prog_silu_mul(rh, uh, dt), dt), TOL[dt])


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("heads,stacked", [(16, False), (8, False), (36, True)])
def test_qk_norm_rope_program_over_half_views(dt, heads, stacked):
    # view plumbing of crates/forja-sdk/src/nn/blocks.rs:181-226: lo/hi halves, broadcast weight and positions
    rng = np.random.default_rng(heads)
    be = backend()
    t, d = 7, 128
    theta = 1e7 if stacked else 1e6
    x, xh = up(rng.standard_normal((t, heads, d)), dt)
    wshape = (heads, d) if stacked else (d,)
    w, wh = up(1.0 + 0.1 * rng.standard_normal(wshape), dt)
    positions = np.array([0, 1, 17, 255, 256, 4099, 8191], np.float32)
    pos = be.tensor_from(positions, fb.F32)
    out = be.alloc(dt, (t, heads, d))
    half = [(0, t, 1), (0, heads, 1)]
    lo, hi = x.slice(half + [(0, 64, 1)]), x.slice(half + [(64, 64, 1)])
    olo, ohi = out.slice(half + [(0, 64, 1)]), out.slice(half + [(64, 64, 1)])
    if stacked:
        wlo, whi = w.slice([(0, heads, 1), (0, 64, 1)]).broadcast((t, heads, 64)), w.slice([(0, heads, 1), (64, 64, 1)]).broadcast((t, heads, 64))
    else:
        wlo, whi = w.slice([(0, 64, 1)]).broadcast((t, heads, 64)), w.slice([(64, 64, 1)]).broadcast((t, heads, 64))
    p = pos.reshape((t, 1, 1)).broadcast((t, heads, 64))
    be.run(Op.Program(prepare(ir.qk_norm_rope(1e-6, theta, 128.0))), [lo, hi, wlo, whi, p], [olo, ohi])
    want = fjo.decode(fjo.prog_qk_norm_rope(xh, dt, wh, dt, positions, 1e-6, theta), dt)
    assert_close(down(out), want, TOL[dt])


@pytest.mark.parametrize("dt", [fb.F32, fb.BF16])
def test_rope_op_matches_oracle_and_identity_at_zero(dt):
    rng = np.random.default_rng(3)
    be = backend()
    x, xh = up(rng.standard_normal((7, 9, 64)), dt)
    positions = np.array([0, 1, 2, 33, 300, 4000, 100000], np.uint32)
    pos, _ = up_u32(positions)
    out = be.alloc(dt, (7, 9, 64))
    be.run(Op.Rope(1e5), [x, pos], [out])
    got = down(out)
    assert_close(got, fjo.decode(fjo.rope(xh, dt, positions, 1e5), dt), TOL[dt])
    assert np.array_equal(got[0], fjo.decode(xh, dt)[0])  # position 0 is the identity (lib.rs:2714-2718)
    # rope_pairs program (crates/forja-sdk/src/nn/blocks.rs:446-464) agrees with its interpreter run
    fpos = be.tensor_from(positions.astype(np.float32), fb.F32)
    out2 = be.alloc(dt, (7, 9, 64))
    spec = [(0, 7, 1), (0, 9, 1)]
    be.run(Op.Program(prepare(ir.rope_pairs(1e5, 64.0))), [x.slice(spec + [(0, 32, 1)]), x.slice(spec + [(32, 32, 1)]), fpos.reshape((7, 1, 1)).broadcast((7, 9, 32))],
           [out2.slice(spec + [(0, 32, 1)]), out2.slice(spec + [(32, 32, 1)])])
    lo, hi = fjo.program(ir.rope_pairs(1e5, 64.0), (7, 9, 32), [xh[..., :32], xh[..., 32:], positions.astype(np.float32)[:, None, None]], [dt, dt, fjo.F32], [dt, dt])
    assert_close(down(out2), fjo.decode(np.concatenate([lo, hi], axis=-1), dt), TOL[dt])


@pytest.mark.parametrize("dt", DTYPES)
def test_embed_gathers_rows_and_reports_lowest_bad_id(dt):
    rng = np.random.default_rng(5)
    be = backend()
    table, th = up(rng.standard_normal((1000, 1024)), dt)
    ids, _ = up_u32([0, 1, 998, 999, 5])
    out = be.alloc(dt, (5, 1024))
    be.run(Op.Embed(), [table, ids], [out])
    assert np.array_equal(down_raw(out).view(np.uint8), th[[0, 1, 998, 999, 5]].view(np.uint8))
    small, sh = up(np.array([[1, 2], [3, 4], [5, 6]], np.float32), dt)
    bad, _ = up_u32([2, 100, 0, 99])
    out = be.alloc(dt, (4, 2))
    with pytest.raises(fb.BackendError) as e:
        be.run(Op.Embed(), [small, bad], [out])
    assert e.value.status == fb.backend.INDEX_OUT_OF_RANGE and e.value.index == 99
    assert down(out).ravel().tolist() == [5.0, 6.0, 0.0, 0.0, 1.0, 2.0, 0.0, 0.0]


@pytest.mark.parametrize("bits,p_dt", [(4, fb.BF16), (8, fb.F16)])
def test_quant_embed_dequantises_rows(bits, p_dt):
    rng = np.random.default_rng(bits)
    be = backend()
    vocab, width, group = 300, 256, 64
    packed = rng.integers(0, 2 ** 32, (vocab, width * bits // 32), dtype=np.uint64).astype(np.uint32)
    pk, _ = up_u32(packed)
    sc, sch = up(rng.standard_normal((vocab, width // group)) * 0.01, p_dt)
    bi, bih = up(rng.standard_normal((vocab, width // group)) * 0.01, p_dt)
    ids = np.array([0, 299, 17, 300, 5], np.uint32)
    idt, _ = up_u32(ids)
    out = be.alloc(fb.BF16, (5, width))
    with pytest.raises(fb.BackendError) as e:
        be.run(Op.QuantEmbed(bits, group), [pk, sc, bi, idt], [out])
    assert e.value.index == 300
    want, bad = fjo.quant_embed(packed, sch, bih, p_dt, ids, bits, group, fjo.BF16, raise_on_bad=False)
    assert bad == 300
    assert np.array_equal(down_raw(out), want)  # one multiply-add per element, same rounding: bit-exact


@pytest.mark.parametrize("width", [1, 5, 64, 2050, 49152, 151936])
def test_argmax_is_bit_exact_with_ties_and_nans(width):
    rng = np.random.default_rng(width)
    be = backend()
    rows = 5
    values = rng.standard_normal((rows, width)).astype(np.float32)
    if width >= 5:
        values[1, 1] = values[1, 3] = 9.0  # last equal value wins (lib.rs:2387-2395)
        values[2, :] = 0.0
        values[3, width // 2] = np.float32(np.nan)
        values.view(np.uint32)[4, 0] = 0xFFC00001  # -NaN is the least value under total order
    for dt in (fb.F32, fb.BF16):
        x, xh = up(values, dt)
        out = be.alloc(fb.U32, (rows,))
        be.run(Op.Argmax(), [x], [out])
        assert down_raw(out).tolist() == fjo.argmax(xh, dt).tolist()


@pytest.mark.parametrize("width,k", [(1, 1), (64, 8), (128, 8), (2050, 64)])
def test_top_k_indices_are_bit_exact(width, k):
    # crates/forja-cpu/src/lib.rs:2398-2447
    be = backend()
    values = (np.arange(width) % 11).astype(np.float32)
    if width >= 128:
        values.view(np.uint32)[3] = 0x7FC00001
        values.view(np.uint32)[9] = 0x7FC00002
        values.view(np.uint32)[17] = 0xFFC00001
    if width == 2050:
        values[2048], values[2049] = 1000.0, 999.0
    x = be.tensor_from(values.reshape(1, width), fb.F32)
    vals, idx = be.alloc(fb.F32, (1, k)), be.alloc(fb.U32, (1, k))
    be.run(Op.TopK(k, False), [x], [vals, idx])
    want_v, want_i = fjo.top_k(values.reshape(1, width), fjo.F32, k, False)
    assert np.array_equal(down_raw(idx), want_i)
    assert np.array_equal(down_raw(vals).view(np.uint32), want_v.view(np.uint32))


def test_top_k_router_shape_normalises_selected_logits():
    rng = np.random.default_rng(11)
    be = backend()
    logits = rng.standard_normal((256, 128)).astype(np.float32)  # N(0,1) router logits, 128 experts, top-8
    logits[3, 5] = logits[3, 77] = logits[3].max() + 1.0  # a tie at the top: lower index first
    x = be.tensor_from(logits, fb.F32)
    vals, idx = be.alloc(fb.F32, (256, 8)), be.alloc(fb.U32, (256, 8))
    be.run(Op.TopK(8, True), [x], [vals, idx])
    want_v, want_i = fjo.top_k(logits, fjo.F32, 8, True)
    assert np.array_equal(down_raw(idx), want_i)
    assert_close(down(vals), want_v, 1e-5)
    v, i = be.alloc(fb.F32, (1, 2)), be.alloc(fb.U32, (1, 2))
    be.run(Op.TopK(2, True), [be.tensor_from(np.array([[1.0, 4.0, 2.0, 3.0]], np.float32), fb.F32)], [v, i])
    den = 1.0 + np.exp(-1.0)
    assert down_raw(i).ravel().tolist() == [1, 3]
    assert_close(down(v), [1.0 / den, np.exp(-1.0) / den], 1e-6)


def test_submission_reports_time_serial_and_launches():
    be = backend()
    x, _ = up(np.ones((4, 64)), fb.F32)
    out = be.alloc(fb.F32, (4, 64))
    cl = CommandList().dispatch(Op.Copy(), [x], out).dispatch(Op.Copy(), [out], x)
    a = be.submit(cl, profiled=True)
    a.wait()
    b = be.submit(cl)
    b.wait(timeout_ns=10_000_000_000)
    assert b.completion_serial() == a.completion_serial() + 1
    assert a.kernel_launches() == 2 and a.gpu_time_ns() > 0
    prof = a.profile()
    assert [p[0] for p in prof] == [fb.backend.OP_COPY] * 2 and all(p[1] == 1 for p in prof)
    with pytest.raises(fb.BackendError) as e:  # unsupported operations are refused, not emulated
        be.run(Op(18), [x], [out])  # Op::State, the recurrent-state update, is not on this path
    assert e.value.status == fb.backend.UNSUPPORTED_OPERATION
    with pytest.raises(fb.BackendError):  # read-only imports cannot be written
        ro = be.import_readonly(np.ones(4, np.float32), fb.F32)
        be.run(Op.Copy(), [x.narrow(0, 0, 1).reshape((64,)).narrow(0, 0, 4)], [ro])


def test_profiled_submission_reports_the_cost_of_each_dispatch():
    """fj_dispatch_profile carries the reference's KernelCost (crates/forja-core/src/cost.rs:109-153, test :293-312;
    attention: cost/attention.rs:141-230): bytes and flops per dispatch, so a roofline can be computed per dispatch."""
    be = backend()
    rng = np.random.default_rng(2)
    m, k, n = 3, 256, 64
    x, _ = up(rng.standard_normal((m, k)), fb.BF16)
    packed = be.tensor_from(rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32), fb.U32)
    scales, _ = up(rng.standard_normal((n, k // 64)) * 0.01, fb.BF16)
    biases, _ = up(rng.standard_normal((n, k // 64)) * 0.01, fb.BF16)
    out = be.alloc(fb.BF16, (m, n))
    # paged decode attention: 8 q / 2 kv heads of width 128, 37 keys on 16-token pages
    hq, kvh, d, page, length = 8, 2, 128, 16, 37
    q, _ = up(rng.standard_normal((1, hq, d)), fb.BF16)
    kp, vp = be.alloc(fb.BF16, (4, page, kvh, d)), be.alloc(fb.BF16, (4, page, kvh, d))
    table = be.tensor_from(np.array([[0, 1], [1, 1], [2, 1], [3, 1]], np.uint32), fb.U32)
    gens = be.tensor_from(np.ones(4, np.uint32), fb.U32)
    attn = be.alloc(fb.BF16, (1, hq, d))
    cl = CommandList()
    cl.dispatch(Op.QuantMatmul(4, 64), [x, packed, scales, biases], out)
    cl.dispatch(Op.PagedSdpa(0.1, True, length - 1, length, page), [q.permute([1, 0, 2]), kp, vp, table, gens], attn.permute([1, 0, 2]))
    sub = be.submit(cl, profiled=True)
    sub.wait()
    quant, attention = sub.profile_costs()
    weight_bytes = n * (k // 8) * 4 + 2 * n * (k // 64) * 2            # 0.5625 bytes per weight
    assert weight_bytes == int(0.5625 * n * k)
    assert quant["read_bytes"] == m * k * 2 + weight_bytes and quant["write_bytes"] == m * n * 2 and quant["flops"] == 2 * m * k * n
    assert attention["read_bytes"] == hq * d * 2 + kvh * length * 2 * d * 2 + 12 * 3 and attention["write_bytes"] == hq * d * 2
    assert attention["flops"] == 2 * hq * length * 2 * d
    assert quant["ns"] > 0 and attention["ns"] > 0
    plain = be.submit(cl)
    plain.wait()
    assert all(p["read_bytes"] == 0 and p["flops"] == 0 for p in plain.profile_costs())
