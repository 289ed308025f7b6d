"""Graph templates (Backend::prepare_graph / replay, crates/forja-core/src/backend.rs:858-920): a decode step
recorded once with its position as a parameter replays like the equivalent direct submissions; values that
overflow a field or name a missing parameter are refused."""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200 import backend as B
from forja_b200.backend import CommandList, Op
from oracle import fjo
from tests.gpu_util import TOL, assert_close, backend, down, down_raw, up, up_u32

pytestmark = pytest.mark.gpu


def test_replayed_decode_template_equals_direct_submissions():
    rng = np.random.default_rng(8)
    be = backend()
    dt, page, hq, kvh, d, steps, start = fb.BF16, 16, 16, 8, 128, 5, 30
    physical = 6
    table = np.zeros((4, 2), np.uint32)
    table[:, 0] = [3, 0, 5, 1]
    generations = np.array([4, 9, 1, 7, 1, 2], np.uint32)
    table[:, 1] = generations[table[:, 0]]
    kh = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    vh = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    q, qh = up(rng.standard_normal((steps, hq, d)), dt)
    kn, knh = up(rng.standard_normal((steps, kvh, d)), dt)
    vn, vnh = up(rng.standard_normal((steps, kvh, d)), dt)
    tb, gn = up_u32(table)[0], up_u32(generations)[0]
    scale = 0.088388346
    row = lambda t, i, heads: t.slice([(i, 1, 1), (0, heads, 1), (0, d, 1)])

    def run(replayed):
        kp, vp = be.tensor_from(kh, dt), be.tensor_from(vh, dt)
        out = be.alloc(dt, (steps, hq, d))
        if replayed:
            # one template: step i reads row i of q / k_new / v_new, appends at start + i, writes row i of out
            cl = CommandList()
            cl.dispatch_many(Op.PagedSdpaAppend(scale, 0, page), [row(q, 0, hq).permute([1, 0, 2]), row(kn, 0, kvh), row(vn, 0, kvh), tb, gn],
                             [row(out, 0, hq).permute([1, 0, 2]), kp, vp])
            bindings = [(0, B.GRAPH_FIELD_U1, 0, 1, start),
                        (0, B.GRAPH_FIELD_INPUT_OFFSET | (0 << 4), 0, hq * d, 0), (0, B.GRAPH_FIELD_INPUT_OFFSET | (1 << 4), 0, kvh * d, 0),
                        (0, B.GRAPH_FIELD_INPUT_OFFSET | (2 << 4), 0, kvh * d, 0), (0, B.GRAPH_FIELD_OUTPUT_OFFSET | (0 << 4), 0, hq * d, 0)]
            graph = be.prepare_graph(cl, bindings, 1)
            for i in range(steps):
                graph.replay([i]).wait()
            graph.close()
        else:
            for i in range(steps):
                be.run(Op.PagedSdpaAppend(scale, start + i, page), [row(q, i, hq).permute([1, 0, 2]), row(kn, i, kvh), row(vn, i, kvh), tb, gn],
                       [row(out, i, hq).permute([1, 0, 2]), kp, vp])
        return down_raw(out), down_raw(kp), down_raw(vp)

    direct, replay = run(False), run(True)
    for a, b in zip(direct, replay):
        assert np.array_equal(a, b)
    # and both equal the oracle
    k_ref, v_ref = kh.copy(), vh.copy()
    for i in range(steps):
        want = fjo.paged_sdpa_append(np.ascontiguousarray(qh[i:i + 1].transpose(1, 0, 2)), dt, knh[i:i + 1].reshape(1, kvh * d), dt, vnh[i:i + 1].reshape(1, kvh * d), dt,
                                     k_ref, dt, v_ref, dt, table, generations, start + i, scale, page)
        assert_close(fjo.decode(replay[0][i], dt), fjo.decode(want, dt).transpose(1, 0, 2)[0], TOL[dt])
    assert np.array_equal(replay[1], k_ref) and np.array_equal(replay[2], v_ref)


def test_replay_refuses_bad_values_and_bad_bindings():
    be = backend()
    x = be.tensor_from(np.arange(32, dtype=np.float32).reshape(4, 8), fb.F32)
    out = be.alloc(fb.F32, (1, 8))
    cl = CommandList()
    cl.dispatch(Op.Copy(), [x.narrow(0, 0, 1)], out)
    graph = be.prepare_graph(cl, [(0, B.GRAPH_FIELD_INPUT_OFFSET, 0, 8, 0)], 1)
    graph.replay([2]).wait()
    assert down(out).ravel().tolist() == list(range(16, 24))
    with pytest.raises(fb.BackendError) as e:   # row 4 lies outside the allocation: refused by the submission's own bounds check
        graph.replay([4])
    assert e.value.status == fb.backend.INVALID_INPUT
    with pytest.raises(fb.BackendError):        # wrong number of values
        graph.replay([1, 2])
    graph.close()
    # a 32-bit field that the affine expression overflows
    cl = CommandList()
    pool = be.alloc(fb.F32, (2, 4, 8))
    cl.dispatch(Op.PagedCopy(True, 0, 4), [x, up_u32([[0, 1], [1, 1]])[0], up_u32([1, 1])[0]], pool)
    graph = be.prepare_graph(cl, [(0, B.GRAPH_FIELD_U1, 0, 1 << 31, 0)], 1)
    with pytest.raises(fb.BackendError) as e:
        graph.replay([2])
    assert e.value.status == fb.backend.INVALID_INPUT
    graph.close()
    for bad in ([(1, B.GRAPH_FIELD_U0, 0, 1, 0)], [(0, B.GRAPH_FIELD_U0, 3, 1, 0)], [(0, B.GRAPH_FIELD_INPUT_OFFSET | (5 << 4), 0, 1, 0)], [(0, 0x900, 0, 1, 0)]):
        with pytest.raises(fb.BackendError):
            be.prepare_graph(cl, bad, 1)
