"""The library's host scheduler (fj_sched_*) against the reference's own unit tests
(crates/forja-serve/src/scheduler.rs:202-290, crates/forja-host/src/prompt.rs:44-80,
crates/forja-serve/src/engine/continuous/batch.rs reservations_fit tests) and, on random request
streams, bit for bit against the CPU oracle's restatement of the same policy."""
import numpy as np
import pytest

import forja_b200 as fb
from oracle import fjo


def test_admits_fifo_with_bounded_smaller_request_bypass():
    s = fb.SchedulerPolicy([1, 2, 4, 8], 8, 8, 2048, 2048)
    s.enqueue(1, 4096)
    s.enqueue(2, 64)
    assert s.admit(lambda rid, tokens: tokens < 1000) == [2]
    for rid in range(3, 11):
        s.enqueue(rid, 64)
    assert len(s.admit(lambda rid, tokens: tokens < 1000)) == 7
    for rid in range(2, 10):
        s.complete(rid)
    # the head has been overtaken 8 times: nothing may pass it any more
    assert s.admit(lambda rid, tokens: tokens < 1000) == []
    assert s.waiting == 2


def test_prompt_budget_buckets_rotation_and_chunking():
    s = fb.SchedulerPolicy([1, 2, 4, 8], 8, 1, 2048, 2048)
    s.ready_prompt(7, 2000)
    s.ready_prompt(8, 1000)
    assert s.prompt_batch(True) == [(7, 2000)]
    assert s.decode_bucket([0, 2]) == 4
    assert s.decode_bucket([]) is None
    assert s.decode_bucket([8]) is None
    assert s.decode_bucket([0xFFFFFFFF]) is None
    s = fb.SchedulerPolicy([1, 2], 2, 2, 4, 4)
    s.ready_prompt(1, 33)
    assert s.prompt_batch(True) == [(1, 4)]
    s.ready_prompt(2, 1)
    assert s.prompt_batch(True) == [(2, 1)]
    assert s.prompt_batch(True) == [(1, 4)]
    with pytest.raises(ValueError):
        fb.SchedulerPolicy([1], 1, 1, 1, 0)
    with pytest.raises(ValueError):
        fb.SchedulerPolicy([2, 4], 4, 1, 1, 1)   # buckets must start at 1
    with pytest.raises(ValueError):
        fb.SchedulerPolicy([1, 2], 4, 1, 1, 1)   # and reach the active-lane ceiling
    s = fb.SchedulerPolicy([1, 2], 2, 2, 512, 2048)
    s.ready_prompt(1, 4097)
    assert s.prompt_batch(False) == [(1, 2048)]
    assert s.prompt_batch(True) == [(1, 512)]
    assert s.prompt_batch(False) == [(1, 1537)]
    s = fb.SchedulerPolicy([1, 2], 2, 1, 512, 2048).with_prompt_chunk_multiple(512)
    s.ready_prompt(1, 2752)
    assert s.prompt_batch(False) == [(1, 2048)]
    assert s.prompt_batch(True) == [(1, 512)]
    assert s.prompt_batch(False) == [(1, 192)]


def test_transient_admission_retry_keeps_the_request_at_the_head():
    s = fb.SchedulerPolicy([1, 2], 2, 2, 16, 16)
    s.enqueue(1, 8)
    s.enqueue(2, 4)
    assert s.admit(lambda rid, tokens: True) == [1, 2]
    s.retry_admission(1, 8)
    s.complete(2)
    assert s.admit(lambda rid, tokens: True) == [1]
    assert s.active == 1


def test_chunking_reservations_and_prefill_plan():
    assert fb.chunk_work(512, 4097, 2047) == 1536
    assert fb.chunk_work(512, 4097, 511) == 0
    assert fb.chunk_work(512, 33, 511) == 33
    assert fb.chunk_merged_work(512, 2752, 2048) == 2048
    assert fb.chunk_merged_work(512, 704, 2048) == 512
    assert fb.chunk_merged_work(512, 192, 2048) == 192
    assert fb.chunk_merged_work(512, 2048, 1537) == 1536
    assert fb.chunk_merged_work(512, 512, 511) == 0
    assert fb.reservations_fit(64, 32768, [4225] * 7)
    assert not fb.reservations_fit(64, 32768, [4225] * 8)
    assert not fb.reservations_fit(1, 16, [2 ** 64 - 1, 2])  # page count overflow
    assert fb.prefill_plan(1500, 512, 512) == [512, 512, 476]
    assert fb.prefill_plan(300, 512, 512) == [300]
    assert fb.prefill_plan(1024, 512, 64) == [512, 512]
    assert fb.prefill_plan(600, 512, 64) == [512, 64, 24]
    assert fb.prefill_plan(0, 512, 64) == []


@pytest.mark.parametrize("seed", range(6))
def test_random_request_streams_match_the_oracle(seed):
    """Drives both implementations with the same random mix of calls (C2 scale: 128 lanes) and
    demands identical decisions at every step."""
    rng = np.random.default_rng(seed)
    lanes = int(rng.choice([2, 8, 128]))
    buckets = sorted({1, 2, 4, 8, 16, 32, 64, 128, lanes})
    buckets = [b for b in buckets if b <= max(lanes, 1)] + ([lanes] if lanes not in buckets else [])
    prefill_limit = int(rng.integers(1, 9))
    budget, idle = int(rng.choice([256, 512, 2048])), int(rng.choice([512, 2048, 8192]))
    ours = fb.SchedulerPolicy(buckets, lanes, prefill_limit, budget, idle)
    ref = fjo.Scheduler(buckets, lanes, prefill_limit, budget, idle)
    if seed % 2:
        ours.with_prompt_chunk_multiple(256)
        ref.chunk_multiple(256)
    next_id, running, admitted_tokens = 1, [], {}
    page_tokens, free_pages = 16, 4000
    for step in range(400):
        action = rng.integers(0, 8)
        if action <= 1:
            for _ in range(int(rng.integers(1, 6))):
                tokens = int(rng.integers(1, 6000))
                ours.enqueue(next_id, tokens)
                ref.enqueue(next_id, tokens)
                admitted_tokens[next_id] = tokens
                next_id += 1
        elif action == 2:
            limit = int(rng.integers(1, 7000))
            got = ours.admit(lambda rid, tokens: tokens < limit)
            assert got == ref.admit_below(limit)
            running += got
        elif action == 3:
            got, left = ours.admit_pages(page_tokens, free_pages)
            want, want_left = ref.admit_pages(page_tokens, free_pages)
            assert (got, left) == (want, want_left)
            free_pages = left
            running += got
        elif action == 4 and running:
            rid = running.pop(int(rng.integers(0, len(running))))
            ours.complete(rid)
            ref.complete(rid)
            free_pages += -(-admitted_tokens[rid] // page_tokens)
        elif action == 5 and running:
            rid = running.pop(int(rng.integers(0, len(running))))
            ours.retry_admission(rid, admitted_tokens[rid])
            ref.retry_admission(rid, admitted_tokens[rid])
        elif action == 6 and running:
            for rid in rng.choice(running, size=min(len(running), 3), replace=False):
                tokens = int(rng.integers(1, 5000))
                ours.ready_prompt(int(rid), tokens)
                ref.ready_prompt(int(rid), tokens)
        else:
            decoding = bool(rng.integers(0, 2))
            assert ours.prompt_batch(decoding) == ref.prompt_batch(decoding)
            slots = rng.integers(0, lanes, size=int(rng.integers(0, 6))).tolist()
            assert ours.decode_bucket(slots) == ref.decode_bucket(slots)
        if step % 50 == 0:
            ours.reconcile_active(len(running))
            ref.reconcile_active(len(running))
