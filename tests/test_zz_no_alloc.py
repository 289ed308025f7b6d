"""The allocation-free decode attention entry point (fj_paged_decode_attention_static).

It serves hosts that have handed all device memory to the KV planes or that must stay out of the
driver's allocator during a decode step: its scratch is a fixed array inside the library. The test
drives it through the C ABI twice in a row - the second batch has different lengths, so whatever
the first call left in the shared array must not matter - and compares each result with the
regular FJ_OP_PAGED_SDPA path on the same inputs, within the bf16 tolerance of the other tests.
It also checks that an oversized batch is refused instead of allocating.
"""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200.backend import CommandList, Op
from oracle import fjo
from tests.gpu_util import TOL, assert_close, backend, down, up, up_u32

pytestmark = pytest.mark.gpu
POISON = 0xFFFFFFFF


def make_batch(rng, lengths, page, physical, table_pages):
    generations = rng.integers(1, 500, physical).astype(np.uint32)
    perm = rng.permutation(physical).astype(np.uint32)
    tables = np.zeros((len(lengths), table_pages, 2), np.uint32)
    tables[..., 1] = POISON
    cursor = 0
    for lane, n in enumerate(lengths):
        pages = (n + page - 1) // page
        tables[lane, :pages, 0] = perm[cursor:cursor + pages]
        tables[lane, :pages, 1] = generations[tables[lane, :pages, 0]]
        cursor += pages
    return tables, generations


def regular_path(be, q, kt, vt, tables_t, gens_t, lengths, hq, d, dt, scale, page):
    """One FJ_OP_PAGED_SDPA dispatch per lane (coalesced by the backend into a ragged launch)."""
    lanes = len(lengths)
    out = be.alloc(dt, (lanes, hq, d))
    cl = CommandList()
    for lane, n in enumerate(lengths):
        row = [(lane, 1, 1), (0, hq, 1), (0, d, 1)]
        table = tables_t.narrow(0, lane, 1).reshape((tables_t.shape[1], 2))
        cl.dispatch(Op.PagedSdpa(scale, True, n - 1, n, page), [q.slice(row).permute([1, 0, 2]), kt, vt, table, gens_t], out.slice(row).permute([1, 0, 2]))
    be.submit(cl).wait()
    return down(out)


def test_static_scratch_decode_attention_matches_the_regular_path_twice():
    rng = np.random.default_rng(2024)
    be = backend()
    dt, page, hq, kvh, d = fb.BF16, 16, 16, 8, 128
    scale = 0.088388346
    table_pages, physical = 140, 700
    kh = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    vh = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    kt, vt = be.tensor_from(kh, dt), be.tensor_from(vh, dt)
    status = be.alloc(fb.U32, (2,))
    for lengths in ([2049, 1, 700, 33, 16, 513, 1500, 64], [5, 2200, 129, 1024, 77, 300]):
        tables, generations = make_batch(rng, lengths, page, physical, table_pages)
        tables_t, gens_t = up_u32(tables)[0], up_u32(generations)[0]
        q, _ = up(rng.standard_normal((len(lengths), hq, d)), dt)
        want = regular_path(be, q, kt, vt, tables_t, gens_t, lengths, hq, d, dt, scale, page)
        out = be.tensor_from(np.full((len(lengths), hq, d), 0x7FC0, np.uint16), dt)  # NaN-filled: every row must be written
        used_before, _ = be.memory_usage()
        assert be.decode_attention_static(q, out, kt, vt, tables_t, gens_t, lengths, scale, status) == fb.backend.OK
        be.synchronize()
        assert be.memory_usage()[0] == used_before
        got = down(out)
        assert np.isfinite(got).all()
        assert_close(got, want, TOL[dt])
        assert be.read(status).tolist() == [0, POISON]
        # and against the CPU oracle directly, lane by lane
        qh = fjo.encode(down(q), dt)
        fjo.set_threads(fjo.max_threads())
        for lane, n in enumerate(lengths):
            ref = fjo.paged_sdpa(np.ascontiguousarray(qh[lane:lane + 1].transpose(1, 0, 2)), dt, kh, dt, vh, dt, tables[lane], generations, n, n - 1, scale, True, page)
            assert_close(got[lane], fjo.decode(ref, dt)[:, 0, :], TOL[dt])
        fjo.set_threads(1)


def test_static_scratch_refuses_batches_beyond_its_limits_and_reports_bad_pages():
    rng = np.random.default_rng(7)
    be = backend()
    dt, page, hq, kvh, d = fb.BF16, 16, 8, 4, 128
    table_pages, physical = 8, 80
    kt = be.alloc(dt, (physical, page, kvh, d))
    lanes = 65  # one more than FJ_STATIC_ATTENTION_MAX_LANES
    tables, generations = make_batch(rng, [16] * lanes, page, physical, table_pages)
    tables_t, gens_t = up_u32(tables)[0], up_u32(generations)[0]
    q = be.alloc(dt, (lanes, hq, d))
    out = be.alloc(dt, (lanes, hq, d))
    assert be.decode_attention_static(q, out, kt, kt, tables_t, gens_t, [16] * lanes, 0.1) == fb.backend.QUOTA_EXCEEDED
    # a stale page entry is reported through the caller's status words and the lane reads as zero
    lengths = [40, 90]
    tables, generations = make_batch(rng, lengths, page, physical, table_pages)
    tables[1, 3, 1] ^= 1
    status = be.alloc(fb.U32, (2,))
    q2, _ = up(rng.standard_normal((2, hq, d)), dt)
    kt2, _ = up(rng.standard_normal((physical, page, kvh, d)), dt)
    out2 = be.tensor_from(np.full((2, hq, d), 0x3F80, np.uint16), dt)
    assert be.decode_attention_static(q2, out2, kt2, kt2, up_u32(tables)[0], up_u32(generations)[0], lengths, 0.1, status) == fb.backend.OK
    be.synchronize()
    assert be.read(status).tolist() == [2, 3]
    got = down(out2)
    assert not got[1].any() and got[0].any()
