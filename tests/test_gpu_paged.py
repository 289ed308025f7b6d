"""GPU parity: paged copy, paged GQA attention (split-K tensor-core decode and the generic f32-math
kernel), fused append, ragged coalescing of per-lane dispatches, and the safety contract (corrupt
page-table entries set an error status, write nothing / zero the rows, never fault)."""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200.backend import CommandList, Layout, Op, Tensor
from oracle import fjo
from tests.gpu_util import TOL, assert_close, backend, down, down_raw, max_abs_rel, up, up_u32

pytestmark = pytest.mark.gpu
POISON = 0xFFFFFFFF


def random_table(rng, tokens, page_tokens, physical_pages, table_pages=None):
    """Randomly permuted physical pages with nonzero generations; unused suffix poisoned."""
    pages = (tokens + page_tokens - 1) // page_tokens
    table_pages = table_pages or pages + 2
    generations = rng.integers(1, 1000, physical_pages).astype(np.uint32)
    chosen = rng.permutation(physical_pages)[:pages].astype(np.uint32)
    table = np.zeros((table_pages, 2), np.uint32)
    table[:, 1] = POISON
    table[:pages, 0] = chosen
    table[:pages, 1] = generations[chosen]
    return table, generations


def test_paged_copy_known_answer_converts_into_reduced_storage():
    # crates/forja-cpu/src/lib.rs:1883-1924
    be = backend()
    values = (np.arange(21, dtype=np.float32) / 8.0).reshape(7, 3)
    src = be.tensor_from(values, fb.F32)
    pool = be.alloc(fb.F16, (3, 4, 3))
    table, _ = up_u32(np.array([[2, 5], [0, 7]]))
    gens, _ = up_u32(np.array([7, 0, 5]))
    out = be.alloc(fb.F32, (7, 3))
    cl = CommandList()
    cl.dispatch(Op.PagedCopy(True, 1, 4), [src, table, gens], pool)
    cl.dispatch(Op.PagedCopy(False, 1, 4), [pool, table, gens], out)
    be.submit(cl).wait()
    assert np.array_equal(down(out), values.astype(np.float16).astype(np.float32))
    raw = down_raw(pool)
    assert not raw[1].any() and not raw[2, 0].any()


@pytest.mark.parametrize("o_dt,p_dt", [(fb.F32, fb.BF16), (fb.BF16, fb.BF16), (fb.F32, fb.F32)])
def test_paged_copy_round_trip_through_permuted_pages(o_dt, p_dt):
    rng = np.random.default_rng(4)
    be = backend()
    page, physical, elements, start, tokens = 16, 40, 192, 13, 300
    table, generations = random_table(rng, start + tokens, page, physical)
    src, srch = up(rng.standard_normal((tokens, 3, 64)), o_dt)
    pool = be.alloc(p_dt, (physical, page, elements))
    tb, gn = up_u32(table)[0], up_u32(generations)[0]
    be.run(Op.PagedCopy(True, start, page), [src, tb, gn], [pool])
    want_pool = np.zeros((physical, page, elements), fjo.NP_OF[p_dt])
    fjo.paged_copy_in(srch.reshape(tokens, elements), o_dt, want_pool, p_dt, table, generations, start, page)
    assert np.array_equal(down_raw(pool).view(np.uint8), want_pool.view(np.uint8))
    out = be.alloc(o_dt, (tokens, 3, 64))
    be.run(Op.PagedCopy(False, start, page), [pool, tb, gn], [out])
    want = fjo.paged_copy_out(want_pool, p_dt, table, generations, start, tokens, page, o_dt)
    assert np.array_equal(down_raw(out).reshape(tokens, elements).view(np.uint8), want.view(np.uint8))


def test_paged_copy_refuses_corrupt_entries_and_writes_nothing():
    rng = np.random.default_rng(5)
    be = backend()
    page, physical = 16, 8
    table, generations = random_table(rng, 64, page, physical)
    src, _ = up(np.ones((40, 32)), fb.F32)
    for corrupt in ("stale", "out_of_bounds", "poisoned"):
        bad = table.copy()
        if corrupt == "stale":
            bad[1, 1] += 1
        elif corrupt == "out_of_bounds":
            bad[1, 0] = physical + 3
        else:
            bad[1] = [0, POISON]
        pool = be.alloc(fb.F32, (physical, page, 32))
        with pytest.raises(fb.BackendError) as e:
            be.run(Op.PagedCopy(True, 0, page), [src, up_u32(bad)[0], up_u32(generations)[0]], [pool])
        assert e.value.status == fb.backend.DEVICE_ERROR_FLAG and e.value.flag == 2 and e.value.index == 1
        assert not down_raw(pool).any()
    # an inactive lane copies nothing and never dereferences its poisoned table
    pool = be.alloc(fb.F32, (physical, page, 32))
    poisoned = np.zeros((4, 2), np.uint32)
    poisoned[:, 1] = POISON
    be.run(Op.PagedCopy(True, 0, page), [src, up_u32(poisoned)[0], up_u32(generations)[0], up_u32([0])[0]], [pool])
    assert not down_raw(pool).any()


def fill_pools(rng, physical, page, kvh, d, dt):
    k = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    v = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    be = backend()
    return be.tensor_from(k, dt), k, be.tensor_from(v, dt), v


@pytest.mark.parametrize("hq,kvh", [(16, 8), (32, 4)])
@pytest.mark.parametrize("length", [1, 7, 33, 512, 513, 2048, 2049, 4000, 4001])
def test_decode_attention_matches_oracle_on_page_edge_lengths(hq, kvh, length):
    rng = np.random.default_rng(length * 31 + hq)
    be = backend()
    dt, page, d = fb.BF16, 16, 128
    physical = (length + page - 1) // page + 5
    table, generations = random_table(rng, length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((1, hq, d)), dt)
    out = be.alloc(dt, (1, hq, d))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    be.run(Op.PagedSdpa(scale, True, length - 1, length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    fjo.set_threads(fjo.max_threads())
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, length, length - 1, scale, True, page)
    fjo.set_threads(1)
    got = down(out).transpose(1, 0, 2)
    assert_close(got, fjo.decode(want, dt), TOL[dt])
    assert max_abs_rel(got, fjo.decode(want, dt)) <= 2e-2


def test_attention_known_answers():
    be = backend()
    # crates/forja-cpu/src/paged.rs:458-476: two keys, f32, page of 4
    pool_h = np.zeros((2, 4, 1, 2), np.float32)
    table = np.array([[1, 4], [0, 3]], np.uint32)
    gens = np.array([3, 4], np.uint32)
    fjo.paged_copy_in(np.array([[1.0, 0.0], [0.0, 1.0]], np.float32), fjo.F32, pool_h.reshape(2, 4, 2), fjo.F32, table, gens, 0, 4)
    pool = be.tensor_from(pool_h, fb.F32)
    q = be.tensor_from(np.array([[[1.0, 0.0]]], np.float32), fb.F32)
    out = be.alloc(fb.F32, (1, 1, 2))
    be.run(Op.PagedSdpa(1.0, False, 0, 2, 4), [q, pool, pool, up_u32(table)[0], up_u32(gens)[0]], [out])
    expected = np.e / (np.e + 1.0)
    got = down(out).ravel()
    assert abs(got[0] - expected) < 1e-6 and abs(got[1] - (1.0 - expected)) < 1e-6
    # crates/forja-cpu/src/lib.rs:1927-1970: append stores both planes, V = 1 gives out = 1
    q = be.alloc(fb.F32, (16, 1, 128))
    k = be.alloc(fb.F32, (1, 8, 128))
    v = be.tensor_from(np.ones((1, 8, 128), np.float32), fb.F32)
    kp, vp = be.alloc(fb.F16, (1, 16, 8, 128)), be.alloc(fb.F16, (1, 16, 8, 128))
    out = be.alloc(fb.F32, (16, 1, 128))
    tb, gn = up_u32(np.array([[0, 1]]))[0], up_u32(np.array([1]))[0]
    be.run(Op.PagedSdpaAppend(0.125, 0, 16), [q, k, v, tb, gn], [out, kp, vp])
    assert np.array_equal(down(out), np.ones((16, 1, 128), np.float32))
    raw = down_raw(vp).view(np.uint16).ravel()
    assert np.all(raw[:1024] == 0x3C00) and not raw[1024:].any()
    with pytest.raises(fb.BackendError):
        be.run(Op.PagedSdpaAppend(0.125, 0xFFFFFFFF, 16), [q, k, v, tb, gn], [out, kp, vp])


@pytest.mark.parametrize("dt,hq,kvh,d", [(fb.F32, 9, 3, 64), (fb.BF16, 16, 8, 128), (fb.F16, 4, 4, 32)])
@pytest.mark.parametrize("q_len,q_start", [(7, 0), (33, 12), (1, 299)])
def test_generic_attention_prefill_and_decode(dt, hq, kvh, d, q_len, q_start):
    """SmolLM2 shape (9 q / 3 kv heads, d 64, f32) and multi-row causal chunks."""
    rng = np.random.default_rng(q_len + q_start)
    be = backend()
    page = 16
    key_length = q_start + q_len
    physical = (key_length + page - 1) // page + 3
    table, generations = random_table(rng, key_length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((q_len, hq, d)), dt)
    out = be.alloc(dt, (q_len, hq, d))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    be.run(Op.PagedSdpa(scale, True, q_start, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, key_length, q_start, scale, True, page)
    assert_close(down(out).transpose(1, 0, 2), fjo.decode(want, dt), TOL[dt] * (10 if dt == fb.F32 else 1))


def test_short_causal_chunk_runs_on_the_tensor_core_kernel():
    """q_len * group <= 16: a 4-token chunk with 16/8 heads stays on the split-K kernel; each row has its own causal limit."""
    rng = np.random.default_rng(12)
    be = backend()
    dt, page, hq, kvh, d, q_len, q_start = fb.BF16, 16, 16, 8, 128, 4, 1021
    key_length = q_start + q_len
    physical = key_length // page + 4
    table, generations = random_table(rng, key_length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((q_len, hq, d)), dt)
    out = be.alloc(dt, (q_len, hq, d))
    scale = 0.088388346
    be.run(Op.PagedSdpa(scale, True, q_start, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, key_length, q_start, scale, True, page)
    assert_close(down(out).transpose(1, 0, 2), fjo.decode(want, dt), TOL[dt])


def test_batched_append_attention_equals_single_lane_and_is_one_ragged_launch():
    """Per-lane PagedSdpaAppend dispatches over shared planes (engines/qwen3-coder/src/lib.rs:917-935)
    coalesce into one attention launch; results equal lane-by-lane submission and the oracle."""
    rng = np.random.default_rng(21)
    be = backend()
    dt, page, hq, kvh, d, lanes = fb.BF16, 16, 32, 4, 128, 6
    lengths = [64, 1, 700, 33, 2049, 15]
    pages_needed = sum((n + page) // page + 1 for n in lengths)
    physical = pages_needed + 4
    generations = rng.integers(1, 100, physical).astype(np.uint32)
    perm = rng.permutation(physical).astype(np.uint32)
    kh = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    vh = fjo.encode(rng.standard_normal((physical, page, kvh, d)).astype(np.float32), dt)
    tables, cursor = [], 0
    for n in lengths:
        pages = (n + page) // page + 1
        t = np.zeros((pages + 1, 2), np.uint32)
        t[:, 1] = POISON
        t[:pages, 0] = perm[cursor:cursor + pages]
        t[:pages, 1] = generations[t[:pages, 0]]
        cursor += pages
        tables.append(t)
    q, qh = up(rng.standard_normal((lanes, hq, d)), dt)
    kn, knh = up(rng.standard_normal((lanes, kvh, d)), dt)
    vn, vnh = up(rng.standard_normal((lanes, kvh, d)), dt)
    gn = up_u32(generations)[0]
    scale = 0.088388346
    activity = [1, 1, 1, 0, 1, 1]  # lane 3 is inactive: zero output, nothing appended

    def run(batched):
        kp, vp = be.tensor_from(kh, dt), be.tensor_from(vh, dt)
        out = be.alloc(dt, (lanes, hq, d))
        cls = [CommandList()] if batched else [CommandList() for _ in range(lanes)]
        for lane, n in enumerate(lengths):
            row = [(lane, 1, 1), (0, hq, 1), (0, d, 1)]
            ins = [q.slice(row).permute([1, 0, 2]), kn.narrow(0, lane, 1), vn.narrow(0, lane, 1), up_u32(tables[lane])[0], gn, up_u32([activity[lane]])[0]]
            (cls[0] if batched else cls[lane]).dispatch_many(Op.PagedSdpaAppend(scale, n, page), ins, [out.slice(row).permute([1, 0, 2]), kp, vp])
        subs = [be.submit(c) for c in cls]
        for s in subs:
            s.wait()
        return down_raw(out), down_raw(kp), down_raw(vp), subs

    got, got_k, got_v, subs = run(True)
    # one append kernel for every lane's new K and V rows, one that builds the split-K work list, ONE attention kernel
    assert subs[0].kernel_launches() == 3
    one, one_k, one_v, _ = run(False)
    assert np.array_equal(got, one) and np.array_equal(got_k, one_k) and np.array_equal(got_v, one_v)
    want_k, want_v = kh.copy(), vh.copy()
    for lane, n in enumerate(lengths):
        want = fjo.paged_sdpa_append(qh[lane][:, None, :], dt, knh[lane:lane + 1], dt, vnh[lane:lane + 1], dt, want_k, dt, want_v, dt, tables[lane], generations, n, scale, page,
                                     activity=activity[lane])
        assert_close(fjo.decode(got[lane], dt), fjo.decode(want[:, 0, :], dt), TOL[dt])
    assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)
    assert not got[3].any()


def test_attention_reports_corrupt_page_entries_and_zeroes_the_lane():
    rng = np.random.default_rng(8)
    be = backend()
    dt, page, hq, kvh, d, length = fb.BF16, 16, 16, 8, 128, 1500
    physical = length // page + 4
    table, generations = random_table(rng, length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, _ = up(rng.standard_normal((1, hq, d)), dt)
    for kind in ("stale", "out_of_bounds"):
        bad = table.copy()
        if kind == "stale":
            bad[40, 1] ^= 1
        else:
            bad[40, 0] = physical + 100
        out = be.tensor_from(np.full((1, hq, d), 0x3F80, np.uint16), dt)
        with pytest.raises(fb.BackendError) as e:
            be.run(Op.PagedSdpa(0.0884, True, length - 1, length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(bad)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
        assert e.value.status == fb.backend.DEVICE_ERROR_FLAG and e.value.flag == 2 and e.value.index == 40
        assert not down_raw(out).any()
    # the device is still usable afterwards
    out = be.alloc(dt, (1, hq, d))
    be.run(Op.PagedSdpa(0.0884, True, length - 1, length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    assert np.isfinite(down(out)).all() and down(out).any()


def test_long_context_split_k_matches_oracle():
    """kv length 32768 (the longest of the isolated attention benchmark), 32 q / 4 kv heads."""
    rng = np.random.default_rng(99)
    be = backend()
    dt, page, hq, kvh, d, length = fb.BF16, 16, 32, 4, 128, 32768
    physical = length // page + 8
    table, generations = random_table(rng, length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((1, hq, d)), dt)
    out = be.alloc(dt, (1, hq, d))
    scale = 0.088388346
    be.run(Op.PagedSdpa(scale, True, length - 1, length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    fjo.set_threads(fjo.max_threads())
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, length, length - 1, scale, True, page)
    fjo.set_threads(1)
    assert_close(down(out).transpose(1, 0, 2), fjo.decode(want, dt), TOL[dt])


@pytest.mark.parametrize("hq,kvh", [(32, 4), (16, 8), (8, 8), (16, 1)])
@pytest.mark.parametrize("q_len,q_start", [(512, 0), (512, 1536), (70, 33), (9, 1000), (257, 15)])
def test_chunked_prefill_attention_on_tensor_cores_matches_oracle(hq, kvh, q_len, q_start):
    """Prefill chunks (config 3: 32 q / 4 kv heads, d 128, 512-token chunks) and ragged tails through
    the 128-row tcgen05 blocks: permuted pages, causal limit per row, chunk start inside a page."""
    rng = np.random.default_rng(q_len * 7 + q_start + hq)
    be = backend()
    dt, page, d = fb.BF16, 16, 128
    key_length = q_start + q_len
    physical = (key_length + page - 1) // page + 3
    table, generations = random_table(rng, key_length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((q_len, hq, d)), dt)
    out = be.alloc(dt, (q_len, hq, d))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    be.run(Op.PagedSdpa(scale, True, q_start, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    fjo.set_threads(fjo.max_threads())
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, key_length, q_start, scale, True, page)
    fjo.set_threads(1)
    got = down(out).transpose(1, 0, 2)
    assert_close(got, fjo.decode(want, dt), TOL[dt])
    assert max_abs_rel(got, fjo.decode(want, dt)) <= 2e-2


@pytest.mark.parametrize("dt,hq,kvh,q_len,q_start", [(fb.BF16, 32, 4, 16, 20000), (fb.BF16, 16, 8, 20, 33000), (fb.F16, 32, 4, 200, 100), (fb.F16, 8, 8, 33, 17000)])
def test_prefill_attention_beyond_one_page_table_window_and_in_f16(dt, hq, kvh, q_len, q_start):
    """The tcgen05 prefill kernel authenticates the lane's page table into shared memory 1024 pages (16384 keys) at a time:
    contexts past that refill the window inside the tile loop. f16 runs the same kernel with the other operand format."""
    rng = np.random.default_rng(q_len + q_start + hq)
    be = backend()
    page, d = 16, 128
    key_length = q_start + q_len
    physical = (key_length + page - 1) // page + 3
    table, generations = random_table(rng, key_length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((q_len, hq, d)), dt)
    out = be.alloc(dt, (q_len, hq, d))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    be.run(Op.PagedSdpa(scale, True, q_start, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    assert be.tcgen05_wait_giveups() == 0
    fjo.set_threads(fjo.max_threads())
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, key_length, q_start, scale, True, page)
    fjo.set_threads(1)
    got = down(out).transpose(1, 0, 2)
    assert_close(got, fjo.decode(want, dt), TOL[dt])
    assert max_abs_rel(got, fjo.decode(want, dt)) <= 2e-2


def test_prefill_attention_non_causal_inactive_and_corrupt_lanes():
    rng = np.random.default_rng(77)
    be = backend()
    dt, page, d, hq, kvh, q_len, key_length = fb.BF16, 16, 128, 16, 8, 40, 100
    physical = key_length // page + 4
    table, generations = random_table(rng, key_length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((q_len, hq, d)), dt)
    scale = 0.088388346
    # non-causal: every row attends to all 100 keys
    out = be.alloc(dt, (q_len, hq, d))
    be.run(Op.PagedSdpa(scale, False, 0, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, key_length, 0, scale, False, page)
    assert_close(down(out).transpose(1, 0, 2), fjo.decode(want, dt), TOL[dt])
    # inactive lane: zeros, whatever the output held before
    out2, _ = up(np.ones((q_len, hq, d)), dt)
    idle, _ = up_u32(np.zeros(1, np.uint32))
    be.run(Op.PagedSdpa(scale, True, 60, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0], idle], [out2.permute([1, 0, 2])])
    assert np.all(down(out2) == 0.0)
    # a stale generation in a page the chunk needs: error flag with the logical page, zero rows
    bad = table.copy()
    bad[2, 1] += 1
    out3 = be.alloc(dt, (q_len, hq, d))
    with pytest.raises(fb.BackendError) as info:
        be.run(Op.PagedSdpa(scale, True, 60, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(bad)[0], up_u32(generations)[0]], [out3.permute([1, 0, 2])])
    assert info.value.flag == 2 and info.value.index == 2
    assert np.all(down(out3) == 0.0)


@pytest.mark.parametrize("q_len,q_start", [(70, 33), (1, 40)])
def test_attention_output_view_at_an_odd_element_offset(q_len, q_start):
    """A 16-bit output view may start at an odd element of its buffer (2-byte aligned): the
    tensor-core kernels must not use packed 4-byte stores there."""
    rng = np.random.default_rng(77 + q_len)
    be = backend()
    dt, page, hq, kvh, d = fb.BF16, 16, 16, 8, 128
    key_length = q_start + q_len
    physical = key_length // page + 4
    table, generations = random_table(rng, key_length, page, physical)
    kt, kh, vt, vh = fill_pools(rng, physical, page, kvh, d, dt)
    q, qh = up(rng.standard_normal((q_len, hq, d)), dt)
    flat = be.alloc(dt, (q_len * hq * d + 3,))
    out = Tensor(flat.buffer, Layout.contiguous(dt, (q_len, hq, d), offset=1), flat.byte_len, True)
    scale = 0.088388346
    be.run(Op.PagedSdpa(scale, True, q_start, key_length, page), [q.permute([1, 0, 2]), kt, vt, up_u32(table)[0], up_u32(generations)[0]], [out.permute([1, 0, 2])])
    want = fjo.paged_sdpa(np.ascontiguousarray(qh.transpose(1, 0, 2)), dt, kh, dt, vh, dt, table, generations, key_length, q_start, scale, True, page)
    assert_close(down(out).transpose(1, 0, 2), fjo.decode(want, dt), TOL[dt])
    raw = down_raw(flat)
    assert raw[0] == 0 and not raw[-2:].any()


def test_coalesced_run_reports_a_bad_lane_under_its_own_dispatch():
    """Per-lane attention dispatches over shared planes run as one launch, but a refused page entry is still reported with
    the index of the dispatch it belongs to (the reference runs the dispatches one by one), for decode and append runs."""
    rng = np.random.default_rng(31)
    be = backend()
    dt, page, hq, kvh, d, lanes = fb.BF16, 16, 16, 8, 128, 5
    lengths = [40, 300, 17, 1000, 64]
    physical = sum((n + page) // page + 1 for n in lengths) + 2
    generations = rng.integers(1, 50, physical).astype(np.uint32)
    perm = rng.permutation(physical).astype(np.uint32)
    tables, cursor = [], 0
    for n in lengths:
        pages = (n + page) // page + 1
        t = np.zeros((pages, 2), np.uint32)
        t[:, 0] = perm[cursor:cursor + pages]
        t[:, 1] = generations[t[:, 0]]
        cursor += pages
        tables.append(t)
    bad_lane = 3
    tables[bad_lane][lengths[bad_lane] // page, 1] ^= 1  # the page that holds the newest token is stale
    kt, _, vt, _ = fill_pools(rng, physical, page, kvh, d, dt)
    q, _ = up(rng.standard_normal((lanes, hq, d)), dt)
    kn, _ = up(rng.standard_normal((lanes, kvh, d)), dt)
    gn = up_u32(generations)[0]
    for append in (False, True):
        out = be.tensor_from(np.full((lanes, hq, d), 0x3F80, np.uint16), dt)
        cl = CommandList()
        cl.dispatch(Op.Copy(), [q], be.alloc(dt, (lanes, hq, d)))  # dispatch 0 is something else
        for lane, n in enumerate(lengths):
            row = [(lane, 1, 1), (0, hq, 1), (0, d, 1)]
            if append:
                cl.dispatch_many(Op.PagedSdpaAppend(0.0884, n, page), [q.slice(row).permute([1, 0, 2]), kn.narrow(0, lane, 1), kn.narrow(0, lane, 1), up_u32(tables[lane])[0], gn],
                                 [out.slice(row).permute([1, 0, 2]), kt, vt])
            else:
                cl.dispatch(Op.PagedSdpa(0.0884, True, n, n + 1, page), [q.slice(row).permute([1, 0, 2]), kt, vt, up_u32(tables[lane])[0], gn], out.slice(row).permute([1, 0, 2]))
        with pytest.raises(fb.BackendError) as e:
            be.submit(cl).wait()
        assert e.value.status == fb.backend.DEVICE_ERROR_FLAG and e.value.flag == 2 and e.value.index == lengths[bad_lane] // page
        assert e.value.dispatch == 1 + bad_lane
        got = down_raw(out)
        assert not got[bad_lane].any()
        assert all(got[lane].any() for lane in range(lanes) if lane != bad_lane)
