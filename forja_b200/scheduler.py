"""Host-side mirror of the reference's SchedulerPolicy (crates/forja-serve/src/scheduler.rs:16-196)
over the C-ABI scheduler in libforja_cuda.so: same method names and argument meaning."""
from __future__ import annotations

import ctypes as C
from typing import Callable, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from . import _lib


class SchedulerPolicy:
    def __init__(self, buckets: Sequence[int], active_limit: int, prefill_limit: int, prompt_budget: int, idle_prompt_budget: int):
        self._lib = _lib.load()
        arr = (C.c_uint32 * len(buckets))(*buckets)
        handle = C.c_void_p()
        status = self._lib.fj_sched_create(arr, len(buckets), active_limit, prefill_limit, prompt_budget, idle_prompt_budget, C.byref(handle))
        if status != 0:
            # the reference returns Err("decode buckets must span the active-lane ceiling" / "prefill limits must be positive")
            raise ValueError("invalid scheduler policy")
        self._h = handle

    def close(self):
        if self._h:
            self._lib.fj_sched_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def with_prompt_chunk_multiple(self, multiple: Optional[int]) -> "SchedulerPolicy":
        if multiple:
            self._lib.fj_sched_set_prompt_chunk_multiple(self._h, multiple)
        return self

    def enqueue(self, request_id: int, reserved_tokens: int):
        self._lib.fj_sched_enqueue(self._h, request_id, reserved_tokens)

    def reconcile_active(self, active: int):
        self._lib.fj_sched_reconcile_active(self._h, active)

    def complete(self, request_id: int):
        self._lib.fj_sched_complete(self._h, request_id)

    def retry_admission(self, request_id: int, reserved_tokens: int):
        self._lib.fj_sched_retry_admission(self._h, request_id, reserved_tokens)

    def admit(self, reserve: Callable[[int, int], bool], cap: int = 4096) -> List[int]:
        """reserve(id, reserved_tokens) -> bool, called in the reference's order."""
        ids = (C.c_uint64 * cap)()
        callback = _lib.SCHED_RESERVE_FN(lambda _user, rid, tokens: 1 if reserve(rid, tokens) else 0)
        n = self._lib.fj_sched_admit(self._h, callback, None, ids, cap)
        return [int(ids[i]) for i in range(min(n, cap))]

    def admit_pages(self, page_tokens: int, free_pages: int, cap: int = 4096) -> Tuple[List[int], int]:
        """Admission against a page budget; returns (admitted ids, pages left)."""
        ids = (C.c_uint64 * cap)()
        left = C.c_uint64(free_pages)
        n = self._lib.fj_sched_admit_pages(self._h, page_tokens, C.byref(left), ids, cap)
        return [int(ids[i]) for i in range(min(n, cap))], int(left.value)

    def decode_bucket(self, slots: Iterable[int]) -> Optional[int]:
        arr = np.ascontiguousarray(list(slots), dtype=np.uint32)
        got = self._lib.fj_sched_decode_bucket(self._h, arr.ctypes.data_as(C.c_void_p), arr.size)
        return None if got < 0 else int(got)

    def ready_prompt(self, request_id: int, tokens: int):
        self._lib.fj_sched_ready_prompt(self._h, request_id, tokens)

    def prompt_batch(self, decoding: bool, cap: int = 4096) -> List[Tuple[int, int]]:
        ids = (C.c_uint64 * cap)()
        spend = (C.c_uint32 * cap)()
        n = self._lib.fj_sched_prompt_batch(self._h, 1 if decoding else 0, ids, spend, cap)
        return [(int(ids[i]), int(spend[i])) for i in range(min(n, cap))]

    @property
    def waiting(self) -> int:
        return int(self._lib.fj_sched_waiting(self._h))

    @property
    def active(self) -> int:
        return int(self._lib.fj_sched_active(self._h))


def chunk_work(piece: int, remaining: int, allowance: int) -> int:
    return int(_lib.load().fj_prompt_chunk_work(piece, remaining, allowance))


def chunk_merged_work(piece: int, remaining: int, allowance: int) -> int:
    return int(_lib.load().fj_prompt_chunk_merged_work(piece, remaining, allowance))


def reservations_fit(page_tokens: int, max_context: int, reservations: Sequence[int]) -> bool:
    arr = np.ascontiguousarray(list(reservations), dtype=np.uint64)
    return bool(_lib.load().fj_reservations_fit(page_tokens, max_context, arr.ctypes.data_as(C.c_void_p), arr.size))


def prefill_plan(sequence: int, chunk: int, tail_chunk: int) -> List[int]:
    lib = _lib.load()
    n = lib.fj_prefill_plan(sequence, chunk, tail_chunk, None, 0)
    out = (C.c_uint32 * max(int(n), 1))()
    n = lib.fj_prefill_plan(sequence, chunk, tail_chunk, out, n)
    return [int(out[i]) for i in range(int(n))]
