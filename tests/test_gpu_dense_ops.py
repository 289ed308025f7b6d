"""GPU parity of the two operators next to the paged path: attention over a contiguous cache (Op::Sdpa) and
the dense-expert gathered matmul (Op::GatherMatmul). Known answers from crates/forja-cpu/src/lib.rs:2449-2488
and :3095-3153, then random cases against the oracle."""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200.backend import Op
from oracle import fjo
from tests.gpu_util import TOL, assert_close, backend, down, down_raw, up, up_u32

pytestmark = pytest.mark.gpu


def run_sdpa(q, k, v, scale, causal, q_start, out_dt=None):
    be = backend()
    out = be.alloc(out_dt if out_dt is not None else q.dtype, (q.shape[0], q.shape[1], v.shape[2]))
    be.run(Op.Sdpa(scale, causal, q_start), [q, k, v], [out])
    return down(out)


def test_sdpa_known_answers():
    be = backend()
    f32 = lambda values, shape: be.tensor_from(np.array(values, np.float32).reshape(shape), fb.F32)
    # a hand-checked two-key case
    got = run_sdpa(f32([1.0, 0.0], (1, 1, 2)), f32([1.0, 0.0, 0.0, 1.0], (1, 2, 2)), f32([10.0, 20.0], (1, 2, 1)), 1.0, False, 0)
    e = np.exp(np.float32(1.0))
    assert abs(got.ravel()[0] - (10.0 * e + 20.0) / (e + 1.0)) <= 1e-5 * 20
    # 16 query heads over 8 cache heads, the cache a strided slice [8, 7, 128] of [8, 4096, 128]
    keys = be.alloc(fb.F32, (8, 4096, 128))
    values = be.tensor_from(np.repeat(np.arange(8, dtype=np.float32), 4096 * 128).reshape(8, 4096, 128), fb.F32)
    window = [(0, 8, 1), (0, 7, 1), (0, 128, 1)]
    got = run_sdpa(be.alloc(fb.F32, (16, 1, 128)), keys.slice(window), values.slice(window), float(1.0 / np.sqrt(np.float32(128.0))), True, 6)
    assert np.allclose(got.ravel(), np.repeat(np.arange(8, dtype=np.float32), 2 * 128), rtol=1e-5)
    # decode equals the last prefill row
    key = f32([1.0, 0.0, 0.0, 1.0, 1.0, 1.0, -1.0, 1.0], (1, 4, 2))
    value = f32([1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0], (1, 4, 2))
    query = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0]
    prefill = run_sdpa(f32(query, (1, 4, 2)), key, value, 0.5, True, 0)
    decode = run_sdpa(f32(query[6:], (1, 1, 2)), key, value, 0.5, True, 3)
    assert np.array_equal(decode.ravel(), prefill.ravel()[6:])
    # a causal window that would reach past the cache is refused
    with pytest.raises(fb.BackendError) as err:
        run_sdpa(f32(query[6:], (1, 1, 2)), key, value, 0.5, True, 4)
    assert err.value.status == fb.backend.INVALID_INPUT


@pytest.mark.parametrize("dt,hq,kvh,d,dv", [(fb.F32, 9, 3, 64, 64), (fb.BF16, 16, 8, 128, 128), (fb.F16, 4, 4, 32, 48)])
@pytest.mark.parametrize("q_len,kv_len,q_start,causal", [(1, 300, 299, True), (33, 45, 12, True), (7, 700, 0, False), (5, 5, 0, True)])
def test_sdpa_matches_oracle(dt, hq, kvh, d, dv, q_len, kv_len, q_start, causal):
    rng = np.random.default_rng(hq * 1000 + q_len)
    q, qh = up(rng.standard_normal((hq, q_len, d)), dt)
    k, kh = up(rng.standard_normal((kvh, kv_len, d)), dt)
    v, vh = up(rng.standard_normal((kvh, kv_len, dv)), dt)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    got = run_sdpa(q, k, v, scale, causal, q_start)
    want = fjo.decode(fjo.sdpa(qh, dt, kh, dt, vh, dt, scale, causal, q_start), dt)
    assert_close(got, want, TOL[dt])


def test_sdpa_takes_the_engine_layout_of_queries_and_outputs():
    """Engines keep activations [tokens, heads, width] and pass permuted views (crates/forja-sdk/src/nn/blocks.rs:181-226)."""
    rng = np.random.default_rng(5)
    be = backend()
    dt, hq, kvh, d, q_len, kv_len = fb.BF16, 8, 2, 64, 6, 40
    q, qh = up(rng.standard_normal((q_len, hq, d)), dt)
    k, kh = up(rng.standard_normal((kvh, kv_len, d)), dt)
    v, vh = up(rng.standard_normal((kvh, kv_len, d)), dt)
    out = be.alloc(dt, (q_len, hq, d))
    be.run(Op.Sdpa(0.125, True, kv_len - q_len), [q.permute([1, 0, 2]), k, v], [out.permute([1, 0, 2])])
    want = fjo.decode(fjo.sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, 0.125, True, kv_len - q_len), dt)
    assert_close(down(out).transpose(1, 0, 2), want, TOL[dt])


def test_gather_matmul_known_answer_and_bad_routes():
    be = backend()
    x = be.tensor_from(np.array([[1.0, 2.0], [3.0, 4.0]], np.float32), fb.F32)
    weights = be.tensor_from(np.array([1.0, 0.0, 0.0, 1.0, 1.0, 1.0, 1.0, 1.0, 2.0, 0.0, 0.0, 3.0], np.float32).reshape(3, 2, 2), fb.F32)
    out = be.alloc(fb.F32, (2, 3, 2))
    be.run(Op.GatherMatmul(), [x, weights, up_u32([[2, 0, 2], [0, 2, 0]])[0]], [out])
    assert down(out).ravel().tolist() == [2.0, 6.0, 1.0, 2.0, 2.0, 6.0, 3.0, 4.0, 6.0, 12.0, 3.0, 4.0]
    out = be.tensor_from(np.full((2, 1, 2), 9.0, np.float32), fb.F32)
    with pytest.raises(fb.BackendError) as err:
        be.run(Op.GatherMatmul(), [x, weights, up_u32([[99], [7]])[0]], [out])
    assert err.value.status == fb.backend.INDEX_OUT_OF_RANGE and err.value.index == 7
    assert not down_raw(out).any()


@pytest.mark.parametrize("dt", [fb.F32, fb.BF16, fb.F16])
@pytest.mark.parametrize("rows,inner,experts,cols,routes", [(1, 64, 4, 48, 2), (37, 256, 8, 200, 3), (5, 2048, 64, 1024, 8)])
def test_gather_matmul_matches_oracle(dt, rows, inner, experts, cols, routes):
    rng = np.random.default_rng(rows + cols)
    x, xh = up(rng.standard_normal((rows, inner)), dt)
    w, wh = up(rng.standard_normal((experts, inner, cols)) * 0.05, dt)
    ids = rng.integers(0, experts, (rows, routes)).astype(np.uint32)
    be = backend()
    out = be.alloc(dt, (rows, routes, cols))
    be.run(Op.GatherMatmul(), [x, w, up_u32(ids)[0]], [out])
    fjo.set_threads(fjo.max_threads())
    want = fjo.gather_matmul(xh, dt, wh, dt, ids)
    fjo.set_threads(1)
    if dt == fb.F32:
        assert np.array_equal(down_raw(out), want)  # the sequential sum is reproduced bit for bit
    else:
        assert_close(down(out), fjo.decode(want, dt), TOL[dt])
