"""Pins the oracle's allocator and scheduler restatements to the reference's own unit tests:
crates/forja-core/src/paged_pool.rs:1363-1757, crates/forja-serve/src/scheduler.rs:202-290,
crates/forja-host/src/prompt.rs:48-63, crates/forja-serve/src/engine/continuous/batch.rs:1188-1192,
crates/forja-sdk/src/nn/blocks.rs:1429-1481.
"""
import numpy as np
import pytest

from oracle import fjo

U32_MAX = 0xFFFFFFFF


def pool(limit, slab=2):
    # layout(): page of 4 tokens, one f32 plane of 2 elements -> 32 bytes per page
    return fjo.Pool(4, 32, slab, limit)


def err(fn, *a):
    with pytest.raises(fjo.OracleError) as e:
        fn(*a)
    return e.value.status


def test_poison_generation_is_never_allocated_and_exhaustion_is_atomic():
    p = pool(1024)
    p.debug_set_generation(0, U32_MAX - 2)
    last = p.reserve(4)
    assert last.table()[0, 1] == U32_MAX - 1
    last.drop()
    before, free = p.memory(), p.free_list().tolist()
    assert err(p.reserve, 12) == fjo.ARITHMETIC_OVERFLOW
    assert p.memory() == before and p.free_list().tolist() == free
    assert fjo.page_table_resolve(np.array([[0, U32_MAX]], np.uint32), np.array([U32_MAX - 1], np.uint32), 0)[0] != 0


def test_quota_refusal_is_atomic_and_fixed_pool_refuses_to_grow():
    p = pool(72)
    before = p.memory()
    assert err(p.reserve, 12) == fjo.QUOTA_EXCEEDED
    assert p.memory() == before
    f = fjo.Pool(4, 32, 2, 1024, fixed=True)
    resident = f.reserve(8)
    before = f.memory()
    assert err(f.reserve, 4) == fjo.QUOTA_EXCEEDED
    assert f.memory() == before
    resident.drop()


def test_dropped_pages_are_reused_lifo_and_in_flight_pages_are_not():
    p = pool(1024)
    s = p.reserve(4)
    old = int(s.table()[0, 0])
    assert old == 0  # slab pages are pushed reversed so page 0 pops first
    s.drop()
    r = p.reserve(4)
    assert int(r.table()[0, 0]) == old and int(r.table()[0, 1]) == 2
    r.drop()
    s = p.reserve(4)
    old = int(s.table()[0, 0])
    s.mark_submitted(7)
    s.drop()
    replacement = p.reserve(4)
    assert int(replacement.table()[0, 0]) != old
    replacement.drop()
    p.observe_completion(7)
    reused = p.reserve(4)
    assert int(reused.table()[0, 0]) == old


def test_fork_shares_prefix_until_tail_copy_on_write():
    p = pool(1024)
    original = p.reserve(8)
    assert original.commit_write(7) == 0
    sibling = original.fork(7)
    assert np.array_equal(original.table(), sibling.table())
    assert original.validate_write(7, 1) == fjo.SHARED_TAIL
    src, dst, count = original.cow_tail()
    assert src != dst and count == 3
    assert original.commit_write(1) == 0
    assert not np.array_equal(original.table(), sibling.table())


def test_reserved_fork_shares_prefix_and_owns_suffix_pages():
    p = pool(2048)
    original = p.reserve(8)
    original.commit_write(7)
    sibling = original.fork_reserved(7, 12)
    assert sibling.logical_len == 7 and sibling.reserved_tokens == 12
    assert sibling.validate_write(7, 1) == fjo.SHARED_TAIL
    assert sibling.cow_tail() is not None
    assert sibling.commit_write(5) == 0
    assert sibling.logical_len == 12 and original.logical_len == 7


def test_refused_reserved_fork_preserves_memory_and_references():
    p = pool(100)
    original = p.reserve(8)
    original.commit_write(7)
    before_memory, before_refs = p.memory(), original.refcounts().tolist()
    assert err(original.fork_reserved, 7, 12) == fjo.QUOTA_EXCEEDED
    assert p.memory() == before_memory and original.refcounts().tolist() == before_refs


def test_page_aligned_fork_appends_without_copying_the_full_tail():
    p = pool(1024)
    original = p.reserve(12)
    original.commit_write(8)
    sibling = original.fork_reserved(8, 12)
    assert sibling.cow_tail() is None
    assert sibling.commit_write(1) == 0 and sibling.logical_len == 9


def test_copy_on_write_and_rollback_restore_the_shared_tail():
    p = pool(1024)
    original = p.reserve(8)
    original.commit_write(7)
    sibling = original.fork(7)
    cp = original.checkpoint()
    assert original.owns_checkpoint(cp) and not sibling.owns_checkpoint(cp)
    assert original.cow_tail() is not None
    original.commit_write(1)
    assert original.rollback(cp) == 0
    assert original.logical_len == 7
    assert np.array_equal(original.table(), sibling.table())


def test_rollback_crosses_a_cow_tail_and_private_page_boundary():
    p = pool(2048)
    original = p.reserve(12)
    original.commit_write(7)
    sibling = original.fork(7)
    cp = original.checkpoint()
    shared = sibling.table()
    original.cow_tail()
    original.commit_write(5)
    assert original.logical_len == 12
    assert original.rollback(cp) == 0
    assert original.logical_len == 7
    assert np.array_equal(original.table()[:2], shared[:2])


def test_rollback_restores_refcounts_after_interleaved_cow():
    p = fjo.Pool(4, 32, 8, 4096)
    original = p.reserve(8)
    original.commit_write(7)
    before_counts, before_memory = original.refcounts().tolist(), p.memory()
    sibling = original.fork(7)
    cp = original.checkpoint()
    original.cow_tail()
    sibling.cow_tail()
    assert original.rollback(cp) == 0
    sibling.drop()
    assert original.refcounts().tolist() == before_counts
    assert p.memory() == before_memory


def test_private_rewind_rules():
    p = pool(1024)
    s = p.reserve(12)
    s.commit_write(9)
    assert s.rewind_private(3) == 0
    assert s.commit_write(9) == 0
    assert s.logical_len == 12 and s.reserved_tokens == 12
    for end, cut in [(7, 5), (7, 4), (8, 7), (9, 7)]:
        q = pool(4096)
        seq = q.reserve(12)
        seq.commit_write(end)
        sib = seq.fork(end)
        before = seq.table()
        assert seq.rewind_private(cut) == fjo.SHARED_TAIL
        assert seq.logical_len == end and np.array_equal(seq.table(), before) and sib.logical_len == end
    q = pool(2048)
    original = q.reserve(8)
    original.commit_write(4)
    sibling = original.fork_reserved(4, 12)
    sibling.commit_write(5)
    assert sibling.rewind_private(7) == 0
    assert sibling.logical_len == 7 and original.logical_len == 4


def test_inactive_slots_stay_poisoned_across_bank_rebinding():
    p = pool(4096)
    s = p.reserve(8)
    s.commit_write(4)
    banks = fjo.Banks(p, 2, 2)
    assert banks.bind(0, 0, s) == 0
    assert banks.slot(0, 0)[1]["active"]
    assert banks.open_append(0, 0, 3, 4) == 0
    assert banks.slot(0, 0)[1]["logical_len"] == 4
    entries, info = banks.slot(0, 1)
    assert not info["active"] and entries.tolist() == [[0, U32_MAX], [0, U32_MAX]]
    banks.mark_submitted(0, 9)
    assert banks.poison(0, 0) == fjo.BANK_IN_FLIGHT
    assert banks.bind(1, 1, s) == 0
    p.observe_completion(9)
    assert banks.poison(0, 0) == 0
    assert banks.slot(0, 0)[0].tolist() == [[0, U32_MAX], [0, U32_MAX]]
    assert banks.slot(1, 1)[1]["active"]


def test_slot_append_window_opens_and_closes_on_rebind():
    p = pool(4096)
    s = p.reserve(8)
    s.commit_write(4)
    banks = fjo.Banks(p, 2, 2)
    banks.bind(0, 0, s)
    info = banks.slot(0, 0)[1]
    assert (info["append_start"], info["logical_len"]) == (4, 4)
    s.commit_write(3)
    assert banks.open_append(0, 0, 4, 7) == 0
    info = banks.slot(0, 0)[1]
    assert (info["append_start"], info["logical_len"]) == (4, 7)
    assert banks.open_append(0, 0, 8, 7) == fjo.UNRESERVED_WRITE
    assert banks.open_append(0, 1, 0, 0) == fjo.FOREIGN_RESOURCE
    banks.bind(0, 0, s)
    info = banks.slot(0, 0)[1]
    assert (info["append_start"], info["logical_len"]) == (7, 7)


def test_append_validation_admits_only_the_private_open_window():
    p = pool(4096)
    s = p.reserve(8)
    s.commit_write(7)
    w = (5, 7)
    assert s.validate_append(w, 5, 2) == 0
    assert s.validate_append(w, 6, 1) == 0
    assert s.validate_append(w, 4, 1) == fjo.UNRESERVED_WRITE
    assert s.validate_append(w, 6, 2) == fjo.UNRESERVED_WRITE
    assert s.validate_append((5, 9), 7, 2) == fjo.UNRESERVED_WRITE
    assert s.validate_append(w, 2 ** 64 - 1, 2) == fjo.ARITHMETIC_OVERFLOW
    _published = s.fork(7)
    assert s.validate_append(w, 5, 2) == fjo.SHARED_TAIL


def test_slots_refuse_sequences_from_another_pool_and_aux_charges_respect_quota():
    primary = pool(4096)
    foreign = pool(4096).reserve(4)
    banks = fjo.Banks(primary, 1, 1)
    assert banks.bind(0, 0, foreign) == fjo.FOREIGN_RESOURCE
    p = pool(512)
    assert p.set_graph_arena_bytes(32) == 0
    assert p.set_scratch_bytes(40, 8) == 0
    usage, limit = p.memory()
    assert usage[3] == 64 and usage[4] == 48
    assert p.set_graph_arena_bytes(512) == fjo.QUOTA_EXCEEDED
    assert p.memory() == (usage, 512)


# ---- scheduler ---------------------------------------------------------------------------------

def test_admits_fifo_with_bounded_smaller_request_bypass():
    s = fjo.Scheduler([1, 2, 4, 8], 8, 8, 2048, 2048)
    s.enqueue(1, 4096)
    s.enqueue(2, 64)
    assert s.admit_below(1000) == [2]
    for rid in range(3, 11):
        s.enqueue(rid, 64)
    assert len(s.admit_below(1000)) == 7
    for rid in range(2, 10):
        s.complete(rid)
    assert s.admit_below(1000) == []


def test_prompt_budget_buckets_rotation_and_chunking():
    s = fjo.Scheduler([1, 2, 4, 8], 8, 1, 2048, 2048)
    s.ready_prompt(7, 2000)
    s.ready_prompt(8, 1000)
    assert s.prompt_batch(True) == [(7, 2000)]
    assert s.decode_bucket([0, 2]) == 4
    s = fjo.Scheduler([1, 2], 2, 2, 4, 4)
    s.ready_prompt(1, 33)
    assert s.prompt_batch(True) == [(1, 4)]
    s.ready_prompt(2, 1)
    assert s.prompt_batch(True) == [(2, 1)]
    assert s.prompt_batch(True) == [(1, 4)]
    with pytest.raises(fjo.OracleError):
        fjo.Scheduler([1], 1, 1, 1, 0)
    s = fjo.Scheduler([1, 2], 2, 2, 512, 2048)
    s.ready_prompt(1, 4097)
    assert s.prompt_batch(False) == [(1, 2048)]
    assert s.prompt_batch(True) == [(1, 512)]
    assert s.prompt_batch(False) == [(1, 1537)]
    s = fjo.Scheduler([1, 2], 2, 1, 512, 2048)
    s.chunk_multiple(512)
    s.ready_prompt(1, 2752)
    assert s.prompt_batch(False) == [(1, 2048)]
    assert s.prompt_batch(True) == [(1, 512)]
    assert s.prompt_batch(False) == [(1, 192)]


def test_transient_admission_retry_keeps_the_request_at_the_head():
    s = fjo.Scheduler([1, 2], 2, 2, 16, 16)
    s.enqueue(1, 8)
    s.enqueue(2, 4)
    assert s.admit_below(2 ** 63) == [1, 2]
    s.retry_admission(1, 8)
    s.complete(2)
    assert s.admit_below(2 ** 63) == [1]


def test_chunking_reservations_and_prefill_plan():
    assert fjo.chunk_work(512, 4097, 2047) == 1536
    assert fjo.chunk_work(512, 4097, 511) == 0
    assert fjo.chunk_work(512, 33, 511) == 33
    assert fjo.chunk_merged_work(512, 2752, 2048) == 2048
    assert fjo.chunk_merged_work(512, 704, 2048) == 512
    assert fjo.chunk_merged_work(512, 192, 2048) == 192
    assert fjo.chunk_merged_work(512, 2048, 1537) == 1536
    assert fjo.chunk_merged_work(512, 512, 511) == 0
    assert fjo.reservations_fit(64, 32768, [4225] * 7)
    assert not fjo.reservations_fit(64, 32768, [4225] * 8)
    assert fjo.prefill_plan(1500, 512, 512) == [512, 512, 476]
    assert fjo.prefill_plan(300, 512, 512) == [300]
    assert fjo.prefill_plan(1024, 512, 64) == [512, 512]
    assert fjo.prefill_plan(600, 512, 64) == [512, 64, 24]


def test_pack_step_reference_metadata():
    # two active lanes (decode at position 20; 3-token prompt piece from 14) and one inactive
    tables = np.zeros((3, 4, 2), np.uint32)
    tables[..., 1] = U32_MAX
    tables[0, :2] = [[5, 1], [2, 3]]
    tables[2, :2] = [[7, 1], [1, 9]]
    out = fjo.pack_step([20, 0, 14], [1, 0, 3], [20, 0, 14], tables, 16)
    assert out["rows"] == 4
    assert out["cu_seqlens"].tolist() == [0, 1, 1, 4]
    assert out["positions"].tolist() == [20, 14, 15, 16]
    assert out["slot_mapping"].tolist() == [2 * 16 + 4, 7 * 16 + 14, 7 * 16 + 15, 1 * 16 + 0]
    assert out["row_lane"].tolist() == [0, 2, 2, 2]
    assert out["absolute_positions"].tolist() == [20, 0, 16]
    assert out["query_starts"].tolist() == [20, 0, 14]
    assert out["activity"].tolist() == [1, 0, 1]


def test_cow_copy_preserves_shared_prefix_bytes():
    """crates/forja-cpu/src/paged.rs:422-455: seven rows are written, the sequence is forked at seven, the original copies its
    shared tail page (three rows) on write; both sequences still read the same seven rows through their own tables."""
    p = pool(4096, slab=4)
    original = p.reserve(8)
    assert original.commit_write(7) == 0
    storage = np.zeros((p.physical_pages(), 4, 2), np.float32)  # page of 4 tokens x one plane of 2 elements
    prefix = np.arange(14, dtype=np.float32).reshape(7, 2)
    fjo.paged_copy_in(prefix, fjo.F32, storage, fjo.F32, original.table(), p.generations(), 0, 4)
    sibling = original.fork(7)
    src, dst, count = original.cow_tail()
    assert count == 3
    tail = fjo.paged_copy_out(storage, fjo.F32, sibling.table(), p.generations(), 4, 3, 4, fjo.F32)
    fjo.paged_copy_in(tail, fjo.F32, storage, fjo.F32, original.table(), p.generations(), 4, 4)
    for sequence in (original, sibling):
        assert np.array_equal(fjo.paged_copy_out(storage, fjo.F32, sequence.table(), p.generations(), 0, 7, 4, fjo.F32), prefix)
