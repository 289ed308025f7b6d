"""ctypes/numpy front end of the CPU oracle (oracle/libfjo_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg of
bench.py. The product package never imports this module.

Tensors are numpy arrays in logical (row-major) order. bf16 values travel as ``np.uint16`` bit
patterns tagged with the dtype code ``BF16``; use :func:`encode` / :func:`decode` to convert.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

F32, F16, BF16, I32, U32 = 0, 1, 2, 3, 4
OK, INVALID_INPUT, EXECUTION_FAILED, INDEX_OUT_OF_RANGE, QUOTA_EXCEEDED, ARITHMETIC_OVERFLOW, \
    UNRESERVED_WRITE, SHARED_TAIL, BANK_IN_FLIGHT, FOREIGN_RESOURCE, INVALID_CHECKPOINT, CORRUPT_STATE, \
    EMPTY_SLAB = range(13)

NP_OF = {F32: np.float32, F16: np.float16, BF16: np.uint16, I32: np.int32, U32: np.uint32}

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.build()
        _lib = C.CDLL(path)
        _lib.fjo_dtype_size.restype = C.c_size_t
        _lib.fjo_pool_physical_pages.restype = C.c_size_t
        _lib.fjo_pool_free_list.restype = C.c_size_t
        _lib.fjo_seq_pages.restype = C.c_size_t
        _lib.fjo_seq_logical_len.restype = C.c_uint64
        _lib.fjo_seq_reserved_tokens.restype = C.c_uint64
        _lib.fjo_sched_admit_below.restype = C.c_size_t
        _lib.fjo_sched_admit_pages.restype = C.c_size_t
        _lib.fjo_sched_prompt_batch.restype = C.c_size_t
        _lib.fjo_sched_decode_bucket.restype = C.c_int64
        _lib.fjo_prefill_plan.restype = C.c_size_t
        _lib.fjo_pack_step.restype = C.c_int64
        _lib.fjo_chunk_work.restype = C.c_uint32
        _lib.fjo_chunk_merged_work.restype = C.c_uint32
    return _lib


class OracleError(RuntimeError):
    def __init__(self, status, index=None):
        super().__init__(f"oracle status {status}" + (f" index {index}" if index is not None else ""))
        self.status = status
        self.index = index


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _c(a, np_dtype=None):
    a = np.ascontiguousarray(a) if np_dtype is None else np.ascontiguousarray(a, dtype=np_dtype)
    return a


def _sz(v):
    return C.c_size_t(int(v))


def _u32(v):
    return C.c_uint32(int(v))


def _u64(v):
    return C.c_uint64(int(v))


def _f(v):
    return C.c_float(float(v))


def code_of(a, dt=None):
    if dt is not None:
        return dt
    return {np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.uint32): U32,
            np.dtype(np.int32): I32}[a.dtype]


def set_threads(n):
    lib().fjo_set_threads(int(n))


def max_threads():
    return lib().fjo_get_max_threads()


def empty(shape, dt):
    return np.empty(shape, dtype=NP_OF[dt])


def encode(values, dt):
    """f32 array -> storage array of dtype code ``dt`` (round to nearest even)."""
    values = _c(values, np.float32)
    out = empty(values.shape, dt)
    st = lib().fjo_encode(_p(values), _p(out), dt, _sz(values.size))
    if st:
        raise OracleError(st)
    return out


def decode(a, dt=None):
    a = _c(a)
    dt = code_of(a, dt)
    out = np.empty(a.shape, np.float32)
    st = lib().fjo_decode(_p(a), dt, _p(out), _sz(a.size))
    if st:
        raise OracleError(st)
    return out


def _check(st, bad=None):
    if st == INDEX_OUT_OF_RANGE:
        raise OracleError(st, bad.value if bad is not None else None)
    if st:
        raise OracleError(st)


def copy(x, x_dt, out_dt):
    x = _c(x)
    out = empty(x.shape, out_dt)
    _check(lib().fjo_copy(_p(x), x_dt, _p(out), out_dt, _sz(x.size)))
    return out


def rms_norm(x, x_dt, w, w_dt, eps, out_dt=None):
    x, w = _c(x), _c(w)
    out_dt = x_dt if out_dt is None else out_dt
    out = empty(x.shape, out_dt)
    _check(lib().fjo_rms_norm(_p(x), x_dt, _p(w), w_dt, _p(out), out_dt, _sz(x.size // x.shape[-1]), _sz(x.shape[-1]), _f(eps)))
    return out


def argmax(x, x_dt):
    x = _c(x)
    rows = x.size // x.shape[-1]
    out = np.empty(x.shape[:-1], np.uint32)
    _check(lib().fjo_argmax(_p(x), x_dt, _p(out), _sz(rows), _sz(x.shape[-1])))
    return out


def top_k(x, x_dt, k, normalize, out_dt=None):
    x = _c(x)
    out_dt = x_dt if out_dt is None else out_dt
    rows = x.size // x.shape[-1]
    values = empty(x.shape[:-1] + (k,), out_dt)
    indices = np.empty(x.shape[:-1] + (k,), np.uint32)
    _check(lib().fjo_top_k(_p(x), x_dt, _p(values), out_dt, _p(indices), _sz(rows), _sz(x.shape[-1]), _u32(k), int(bool(normalize))))
    return values, indices


def sample(x, x_dt, params, position, allow=None):
    x = _c(x)
    params = _c(params, np.uint32)
    allow = None if allow is None else _c(allow, np.uint32)
    rows = x.size // x.shape[-1]
    out = np.empty(x.shape[:-1], np.uint32)
    _check(lib().fjo_sample(_p(x), x_dt, _p(params), _p(allow), _p(out), _sz(rows), _sz(x.shape[-1]), _u32(position)))
    return out


def rope(x, x_dt, positions, theta, out_dt=None):
    x = _c(x)
    positions = _c(positions, np.uint32)
    out_dt = x_dt if out_dt is None else out_dt
    out = empty(x.shape, out_dt)
    t, h, w = x.shape
    _check(lib().fjo_rope(_p(x), x_dt, _p(positions), _p(out), out_dt, _sz(t), _sz(h), _sz(w), _f(theta)))
    return out


def embed(table, t_dt, ids, out_dt=None, raise_on_bad=True):
    table, ids = _c(table), _c(ids, np.uint32)
    out_dt = t_dt if out_dt is None else out_dt
    out = empty((ids.size, table.shape[1]), out_dt)
    bad = C.c_uint32(0)
    st = lib().fjo_embed(_p(table), t_dt, _p(ids), _p(out), out_dt, _sz(table.shape[0]), _sz(table.shape[1]), _sz(ids.size), C.byref(bad))
    if st == INDEX_OUT_OF_RANGE and not raise_on_bad:
        return out, bad.value
    _check(st, bad)
    return (out, None) if not raise_on_bad else out


def quant_embed(packed, scales, biases, p_dt, ids, bits, group_size, out_dt, raise_on_bad=True):
    packed, scales, biases, ids = _c(packed, np.uint32), _c(scales), _c(biases), _c(ids, np.uint32)
    width = packed.shape[1] * (32 // bits)
    out = empty((ids.size, width), out_dt)
    bad = C.c_uint32(0)
    st = lib().fjo_quant_embed(_p(packed), _p(scales), _p(biases), p_dt, _p(ids), _p(out), out_dt, _sz(packed.shape[0]),
                               _sz(packed.shape[1]), _sz(ids.size), _u32(bits), _u32(group_size), C.byref(bad))
    if st == INDEX_OUT_OF_RANGE and not raise_on_bad:
        return out, bad.value
    _check(st, bad)
    return (out, None) if not raise_on_bad else out


def matmul(left, l_dt, right, r_dt, out_dt, right_transposed=False):
    """left [.., rows, inner]; right [.., inner, cols], or [.., cols, inner] when right_transposed."""
    left, right = _c(left), _c(right)
    rows, inner = left.shape[-2:]
    cols = right.shape[-2] if right_transposed else right.shape[-1]
    batch = left.size // (rows * inner)
    out = empty(left.shape[:-1] + (cols,), out_dt)
    _check(lib().fjo_matmul(_p(left), l_dt, _p(right), r_dt, _p(out), out_dt, _sz(batch), _sz(rows), _sz(inner), _sz(cols), int(right_transposed)))
    return out


def quant_matmul(x, x_dt, packed, scales, biases, p_dt, bits, group_size, out_dt=None):
    x, packed, scales, biases = _c(x), _c(packed, np.uint32), _c(scales), _c(biases)
    out_dt = x_dt if out_dt is None else out_dt
    rows, inner = x.shape
    cols = packed.shape[0]
    out = empty((rows, cols), out_dt)
    _check(lib().fjo_quant_matmul(_p(x), x_dt, _p(packed), _p(scales), _p(biases), p_dt, _p(out), out_dt, _sz(rows), _sz(inner), _sz(cols), _u32(bits), _u32(group_size)))
    return out


def gather_quant_matmul(x, x_dt, packed, scales, biases, p_dt, indices, bits, group_size, out_dt=None, raise_on_bad=True):
    x, packed, scales, biases, indices = _c(x), _c(packed, np.uint32), _c(scales), _c(biases), _c(indices, np.uint32)
    out_dt = x_dt if out_dt is None else out_dt
    rows, inner = x.shape
    experts, cols, _ = packed.shape
    k = indices.shape[1]
    out = empty((rows, k, cols), out_dt)
    bad = C.c_uint32(0)
    st = lib().fjo_gather_quant_matmul(_p(x), x_dt, _p(packed), _p(scales), _p(biases), p_dt, _p(indices), _p(out), out_dt, _sz(rows), _sz(inner),
                                       _sz(experts), _sz(cols), _sz(k), _u32(bits), _u32(group_size), C.byref(bad))
    if st == INDEX_OUT_OF_RANGE and not raise_on_bad:
        return out, bad.value
    _check(st, bad)
    return (out, None) if not raise_on_bad else out


def gather_quant_weighted_sum(act, a_dt, packed, scales, biases, p_dt, indices, weights, w_dt, bits, group_size, out_dt, raise_on_bad=True):
    act, packed, scales, biases = _c(act), _c(packed, np.uint32), _c(scales), _c(biases)
    indices, weights = _c(indices, np.uint32), _c(weights)
    rows, routes, inner = act.shape
    experts, cols, _ = packed.shape
    out = empty((rows, cols), out_dt)
    bad = C.c_uint32(0)
    st = lib().fjo_gather_quant_weighted_sum(_p(act), a_dt, _p(packed), _p(scales), _p(biases), p_dt, _p(indices), _p(weights), w_dt, _p(out), out_dt,
                                             _sz(rows), _sz(routes), _sz(inner), _sz(experts), _sz(cols), _u32(bits), _u32(group_size), C.byref(bad))
    if st == INDEX_OUT_OF_RANGE and not raise_on_bad:
        return out, bad.value
    _check(st, bad)
    return (out, None) if not raise_on_bad else out


def gather_matmul(x, x_dt, weights, w_dt, indices, out_dt=None, raise_on_bad=True):
    """Op::GatherMatmul: x [rows, inner], weights [experts, inner, columns], indices [rows, routes] -> [rows, routes, columns]."""
    x, weights, indices = _c(x), _c(weights), _c(indices, np.uint32)
    out_dt = x_dt if out_dt is None else out_dt
    rows, inner = x.shape
    experts, _, cols = weights.shape
    routes = indices.shape[1]
    out = empty((rows, routes, cols), out_dt)
    bad = C.c_uint32(0)
    st = lib().fjo_gather_matmul(_p(x), x_dt, _p(weights), w_dt, _p(indices), _p(out), out_dt, _sz(rows), _sz(inner), _sz(experts), _sz(cols), _sz(routes), C.byref(bad))
    if st == INDEX_OUT_OF_RANGE and not raise_on_bad:
        return out, bad.value
    _check(st, bad)
    return (out, None) if not raise_on_bad else out


def sdpa(q, q_dt, k, k_dt, v, v_dt, scale, causal, q_start, out_dt=None):
    q, k, v = _c(q), _c(k), _c(v)
    out_dt = q_dt if out_dt is None else out_dt
    hq, t, d = q.shape
    kvh, length, _ = k.shape
    dv = v.shape[2]
    out = empty((hq, t, dv), out_dt)
    _check(lib().fjo_sdpa(_p(q), q_dt, _p(k), k_dt, _p(v), v_dt, _p(out), out_dt, _sz(hq), _sz(t), _sz(d), _sz(kvh), _sz(length), _sz(dv), _f(scale), int(bool(causal)), _u32(q_start)))
    return out


# ---- scalar programs -------------------------------------------------------------------------

T_INPUT, T_CONST, T_INDEX, T_EXTENT, T_UNARY, T_BINARY, T_SELECT, T_CAST, T_REDUCE = range(9)
U_NEG, U_ABS, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_SIN, U_COS, U_TANH, U_SIGMOID, U_RECIP, U_FLOOR, U_LOG1P, U_EXPROUNDED = range(14)
B_ADD, B_SUB, B_MUL, B_DIV, B_MIN, B_MAX, B_POW, B_LT, B_LE, B_EQ, B_NE, B_GE, B_GT = range(13)
R_SUM, R_MAX, R_MIN = range(3)
V_F32, V_U32, V_BOOL = range(3)
MAP, ROW = 0, 1


def f32_bits(value):
    return int(np.array([value], np.float32).view(np.uint32)[0])


class Program:
    """Flat SSA scalar program in the reference's IR (crates/forja-core/src/program.rs:128-149)."""

    def __init__(self, kind):
        self.kind = kind
        self.insts = []
        self.outputs = []

    def _push(self, *words):
        self.insts.append(tuple(words) + (0,) * (4 - len(words)))
        return len(self.insts) - 1

    def input(self, slot): return self._push(T_INPUT, slot)
    def constant(self, value): return self._push(T_CONST, f32_bits(value))
    def index(self, axis): return self._push(T_INDEX, axis)
    def extent(self, axis): return self._push(T_EXTENT, axis)
    def unary(self, op, x): return self._push(T_UNARY, op, x)
    def binary(self, op, left, right): return self._push(T_BINARY, op, left, right)
    def select(self, c, a, b): return self._push(T_SELECT, c, a, b)
    def cast(self, to, x): return self._push(T_CAST, to, x)
    def reduce(self, op, x): return self._push(T_REDUCE, op, x)
    def output(self, slot, value): self.outputs.append((slot, value))

    def words(self):
        return np.array(self.insts, np.uint32).reshape(-1, 4), np.array(self.outputs, np.uint32).reshape(-1, 2)


def program(prog, shape, inputs, input_dts, out_dts):
    """Runs ``prog`` over ``shape``; inputs are broadcast to ``shape`` like the host's views."""
    insts, outs = prog.words()
    shape = tuple(int(s) for s in shape)
    arrays = [np.ascontiguousarray(np.broadcast_to(a, shape)) for a in inputs]
    in_ptrs = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    in_codes = (C.c_int * len(arrays))(*input_dts)
    results = [empty(shape, dt) for dt in out_dts]
    out_ptrs = (C.c_void_p * len(results))(*[a.ctypes.data for a in results])
    out_codes = (C.c_int * len(results))(*out_dts)
    shape_arr = np.array(shape, np.uint32)
    _check(lib().fjo_program(prog.kind, _p(insts), _sz(len(insts)), _p(outs), _sz(len(outs)), _p(shape_arr), _sz(len(shape)),
                             in_ptrs, in_codes, _sz(len(arrays)), out_ptrs, out_codes))
    return results


def prog_rms_norm(x, dt, w, w_dt, eps, out_dt=None):
    x, w = _c(x), _c(w)
    out_dt = dt if out_dt is None else out_dt
    out = empty(x.shape, out_dt)
    _check(lib().fjo_prog_rms_norm(_p(x), dt, _p(w), w_dt, _p(out), out_dt, _sz(x.size // x.shape[-1]), _sz(x.shape[-1]), _f(eps)))
    return out


def prog_residual_norm(residual, update, dt, w, w_dt, eps, out_dt=None):
    residual, update, w = _c(residual), _c(update), _c(w)
    out_dt = dt if out_dt is None else out_dt
    total, norm = empty(residual.shape, out_dt), empty(residual.shape, out_dt)
    _check(lib().fjo_prog_residual_norm(_p(residual), _p(update), dt, _p(w), w_dt, _p(total), _p(norm), out_dt,
                                        _sz(residual.size // residual.shape[-1]), _sz(residual.shape[-1]), _f(eps)))
    return total, norm


def prog_add(a, b, dt, out_dt=None):
    a, b = _c(a), _c(b)
    out_dt = dt if out_dt is None else out_dt
    out = empty(a.shape, out_dt)
    _check(lib().fjo_prog_add(_p(a), _p(b), dt, _p(out), out_dt, _sz(a.size)))
    return out


def prog_silu_mul(gate, up, dt, out_dt=None):
    gate, up = _c(gate), _c(up)
    out_dt = dt if out_dt is None else out_dt
    out = empty(gate.shape, out_dt)
    _check(lib().fjo_prog_silu_mul(_p(gate), _p(up), dt, _p(out), out_dt, _sz(gate.size)))
    return out


def prog_qk_norm_rope(x, dt, w, w_dt, positions, eps, theta, out_dt=None):
    x, w = _c(x), _c(w)
    positions = _c(positions, np.float32)
    out_dt = dt if out_dt is None else out_dt
    out = empty(x.shape, out_dt)
    t, h, width = x.shape
    _check(lib().fjo_prog_qk_norm_rope(_p(x), dt, _p(w), w_dt, int(w.ndim == 2), _p(positions), _p(out), out_dt, _sz(t), _sz(h), _sz(width), _f(eps), _f(theta)))
    return out


# ---- paged storage ---------------------------------------------------------------------------

def _activity(activity):
    return None if activity is None else np.array([activity], np.uint32)


def paged_copy_in(ordinary, o_dt, pool, p_dt, table, generations, start, page_tokens, activity=None):
    """Writes rows of ``ordinary`` [tokens, elements] into ``pool`` [P, page, elements] in place."""
    ordinary = _c(ordinary)
    assert pool.flags["C_CONTIGUOUS"]
    table, generations = _c(table, np.uint32), _c(generations, np.uint32)
    act = _activity(activity)
    tokens = ordinary.shape[0]
    elements = ordinary.size // max(tokens, 1)
    _check(lib().fjo_paged_copy(1, _p(ordinary), o_dt, _p(pool), p_dt, _p(table), _sz(table.size // 2), _p(generations), _sz(generations.size),
                                _u32(start), _u32(tokens), _u32(page_tokens), _sz(elements), _p(act)))


def paged_copy_out(pool, p_dt, table, generations, start, tokens, page_tokens, out_dt, activity=None, out=None):
    pool = _c(pool)
    table, generations = _c(table, np.uint32), _c(generations, np.uint32)
    act = _activity(activity)
    elements = pool.size // (pool.shape[0] * pool.shape[1])
    if out is None:
        out = np.zeros((tokens, elements), NP_OF[out_dt])
    _check(lib().fjo_paged_copy(0, _p(out), out_dt, _p(pool), p_dt, _p(table), _sz(table.size // 2), _p(generations), _sz(generations.size),
                                _u32(start), _u32(tokens), _u32(page_tokens), _sz(elements), _p(act)))
    return out


def paged_sdpa(q, q_dt, kpool, k_dt, vpool, v_dt, table, generations, key_length, q_start, scale, causal, page_tokens, out_dt=None, activity=None):
    """q [hq, T, d] logical; pools [P, page, kvh, d]."""
    q, kpool, vpool = _c(q), _c(kpool), _c(vpool)
    table, generations = _c(table, np.uint32), _c(generations, np.uint32)
    out_dt = q_dt if out_dt is None else out_dt
    hq, t, d = q.shape
    kvh, dv = kpool.shape[2], vpool.shape[3]
    out = empty((hq, t, dv), out_dt)
    act = _activity(activity)
    _check(lib().fjo_paged_sdpa(_p(q), q_dt, _p(kpool), k_dt, _p(vpool), v_dt, _p(table), _sz(table.size // 2), _p(generations), _sz(generations.size),
                                _p(out), out_dt, _u32(hq), _u32(t), _u32(kvh), _u32(d), _u32(dv), _u32(key_length), _u32(q_start), _f(scale),
                                int(bool(causal)), _u32(page_tokens), _p(act)))
    return out


def paged_sdpa_append(q, q_dt, k_new, kn_dt, v_new, vn_dt, kpool, k_dt, vpool, v_dt, table, generations, q_start, scale, page_tokens, out_dt=None, activity=None):
    """Appends in place into kpool/vpool, then attends. q [hq, 1, d]."""
    q, k_new, v_new = _c(q), _c(k_new), _c(v_new)
    assert kpool.flags["C_CONTIGUOUS"] and vpool.flags["C_CONTIGUOUS"]
    table, generations = _c(table, np.uint32), _c(generations, np.uint32)
    out_dt = q_dt if out_dt is None else out_dt
    hq, _, d = q.shape
    kvh, dv = kpool.shape[2], vpool.shape[3]
    out = empty((hq, 1, dv), out_dt)
    act = _activity(activity)
    _check(lib().fjo_paged_sdpa_append(_p(q), q_dt, _p(k_new), kn_dt, _p(v_new), vn_dt, _p(kpool), k_dt, _p(vpool), v_dt, _p(table), _sz(table.size // 2),
                                       _p(generations), _sz(generations.size), _p(out), out_dt, _u32(hq), _u32(kvh), _u32(d), _u32(dv), _u32(q_start), _f(scale),
                                       _u32(page_tokens), _p(act)))
    return out


def paged_layout_page_bytes(page_tokens, dtype, elements_per_token, alignment):
    out = C.c_uint64(0)
    _check(lib().fjo_paged_layout_page_bytes(_u32(page_tokens), dtype, _u64(elements_per_token), _u64(alignment), C.byref(out)))
    return out.value


def page_table_resolve(table, generations, logical_page):
    table, generations = _c(table, np.uint32), _c(generations, np.uint32)
    out = C.c_uint32(0)
    st = lib().fjo_page_table_resolve(_p(table), _sz(table.size // 2), _p(generations), _sz(generations.size), _u32(logical_page), C.byref(out))
    return st, out.value


# ---- allocator -------------------------------------------------------------------------------

class Sequence:
    def __init__(self, pool, handle):
        self.pool, self.h = pool, handle

    def drop(self):
        if self.h:
            lib().fjo_seq_drop(self.h)
            self.h = None

    @property
    def logical_len(self): return lib().fjo_seq_logical_len(self.h)
    @property
    def reserved_tokens(self): return lib().fjo_seq_reserved_tokens(self.h)

    def table(self):
        n = lib().fjo_seq_pages(self.h)
        out = np.zeros((n, 2), np.uint32)
        _check(lib().fjo_seq_table(self.h, _p(out), _sz(n)))
        return out

    def refcounts(self):
        n = lib().fjo_seq_pages(self.h)
        out = np.zeros(n, np.uint32)
        _check(lib().fjo_seq_refcounts(self.h, _p(out), _sz(n)))
        return out

    def validate_write(self, start, tokens): return lib().fjo_seq_validate_write(self.h, _u64(start), _u64(tokens))
    def validate_append(self, window, start, tokens): return lib().fjo_seq_validate_append(self.h, _u64(window[0]), _u64(window[1]), _u64(start), _u64(tokens))
    def commit_write(self, tokens): return lib().fjo_seq_commit_write(self.h, _u64(tokens))
    def rewind_private(self, n): return lib().fjo_seq_rewind_private(self.h, _u64(n))
    def mark_submitted(self, serial): return lib().fjo_seq_mark_submitted(self.h, _u64(serial))

    def fork_reserved(self, prefix, reserved):
        out = C.c_void_p()
        st = lib().fjo_seq_fork_reserved(self.h, _u64(prefix), _u64(reserved), C.byref(out))
        if st:
            raise OracleError(st)
        return Sequence(self.pool, out)

    def fork(self, prefix): return self.fork_reserved(prefix, prefix)

    def cow_tail(self):
        copied, src, dst, count = C.c_int(0), C.c_uint32(0), C.c_uint32(0), C.c_uint32(0)
        st = lib().fjo_seq_cow_tail(self.h, C.byref(copied), C.byref(src), C.byref(dst), C.byref(count))
        if st:
            raise OracleError(st)
        return (src.value, dst.value, count.value) if copied.value else None

    def checkpoint(self):
        out = C.c_void_p()
        st = lib().fjo_seq_checkpoint(self.h, C.byref(out))
        if st:
            raise OracleError(st)
        return out

    def rollback(self, checkpoint): return lib().fjo_seq_rollback(self.h, checkpoint)
    def owns_checkpoint(self, checkpoint): return bool(lib().fjo_checkpoint_belongs_to(checkpoint, self.h))


class Pool:
    def __init__(self, page_tokens, total_page_bytes, pages_per_slab, byte_limit, fixed=False):
        out = C.c_void_p()
        st = lib().fjo_pool_new(_u32(page_tokens), _u64(total_page_bytes), _u32(pages_per_slab), _u64(byte_limit), int(fixed), C.byref(out))
        if st:
            raise OracleError(st)
        self.h = out
        self.page_tokens = page_tokens

    def reserve(self, tokens):
        out = C.c_void_p()
        st = lib().fjo_pool_reserve(self.h, _u64(tokens), C.byref(out))
        if st:
            raise OracleError(st)
        return Sequence(self, out)

    def observe_completion(self, serial): return lib().fjo_pool_observe_completion(self.h, _u64(serial))

    def memory(self):
        usage = (C.c_uint64 * 5)()
        limit = C.c_uint64(0)
        lib().fjo_pool_memory(self.h, usage, C.byref(limit))
        return tuple(usage), limit.value

    def set_graph_arena_bytes(self, n): return lib().fjo_pool_set_graph_arena_bytes(self.h, _u64(n))
    def set_scratch_bytes(self, a, b): return lib().fjo_pool_set_scratch_bytes(self.h, _u64(a), _u64(b))
    def physical_pages(self): return lib().fjo_pool_physical_pages(self.h)

    def generations(self):
        n = self.physical_pages()
        out = np.zeros(n, np.uint32)
        _check(lib().fjo_pool_generations(self.h, _p(out), _sz(n)))
        return out

    def free_list(self):
        n = lib().fjo_pool_free_list(self.h, None, _sz(0))
        out = np.zeros(max(n, 1), np.uint32)
        lib().fjo_pool_free_list(self.h, _p(out), _sz(n))
        return out[:n]

    def debug_set_generation(self, page, generation): return lib().fjo_pool_debug_set_generation(self.h, _u32(page), _u32(generation))


class Banks:
    def __init__(self, pool, lanes, table_pages):
        out = C.c_void_p()
        st = lib().fjo_banks_new(pool.h, _sz(lanes), _sz(table_pages), C.byref(out))
        if st:
            raise OracleError(st)
        self.h, self.table_pages = out, table_pages

    def bind(self, bank, lane, seq): return lib().fjo_banks_bind(self.h, _sz(bank), _sz(lane), seq.h)
    def bind_all(self, lane, seq): return lib().fjo_banks_bind_all(self.h, _sz(lane), seq.h)
    def poison(self, bank, lane): return lib().fjo_banks_poison(self.h, _sz(bank), _sz(lane))
    def open_append(self, bank, lane, start, logical_len): return lib().fjo_banks_open_append(self.h, _sz(bank), _sz(lane), _u64(start), _u64(logical_len))
    def mark_submitted(self, bank, serial): return lib().fjo_banks_mark_submitted(self.h, _sz(bank), _u64(serial))

    def slot(self, bank, lane):
        entries = np.zeros((self.table_pages, 2), np.uint32)
        info = (C.c_uint64 * 3)()
        st = lib().fjo_banks_slot(self.h, _sz(bank), _sz(lane), _p(entries), info)
        if st:
            raise OracleError(st)
        return entries, {"logical_len": info[0], "append_start": info[1], "active": bool(info[2])}


# ---- scheduler -------------------------------------------------------------------------------

class Scheduler:
    def __init__(self, buckets, active_limit, prefill_limit, prompt_budget, idle_prompt_budget):
        out = C.c_void_p()
        b = np.array(buckets, np.uint32)
        st = lib().fjo_sched_new(_p(b), _sz(b.size), _sz(active_limit), _sz(prefill_limit), _u32(prompt_budget), _u32(idle_prompt_budget), C.byref(out))
        if st:
            raise OracleError(st)
        self.h = out

    def chunk_multiple(self, m): lib().fjo_sched_chunk_multiple(self.h, _u32(m))
    def enqueue(self, rid, reserved): lib().fjo_sched_enqueue(self.h, _u64(rid), _u64(reserved))
    def reconcile_active(self, n): lib().fjo_sched_reconcile_active(self.h, _sz(n))
    def complete(self, rid): lib().fjo_sched_complete(self.h, _u64(rid))
    def retry_admission(self, rid, reserved): lib().fjo_sched_retry_admission(self.h, _u64(rid), _u64(reserved))

    def admit_below(self, limit):
        ids = np.zeros(1024, np.uint64)
        n = lib().fjo_sched_admit_below(self.h, _u64(limit), _p(ids), _sz(ids.size))
        return [int(v) for v in ids[:n]]

    def admit_pages(self, page_tokens, free_pages):
        ids = np.zeros(4096, np.uint64)
        fp = C.c_uint64(int(free_pages))
        n = lib().fjo_sched_admit_pages(self.h, _u32(page_tokens), C.byref(fp), _p(ids), _sz(ids.size))
        return [int(v) for v in ids[:n]], fp.value

    def decode_bucket(self, slots):
        s = np.array(list(slots), np.uint32)
        v = lib().fjo_sched_decode_bucket(self.h, _p(s), _sz(s.size))
        return None if v < 0 else int(v)

    def ready_prompt(self, rid, tokens): lib().fjo_sched_ready_prompt(self.h, _u64(rid), _u32(tokens))

    def prompt_batch(self, decoding):
        ids, spend = np.zeros(1024, np.uint64), np.zeros(1024, np.uint32)
        n = lib().fjo_sched_prompt_batch(self.h, int(bool(decoding)), _p(ids), _p(spend), _sz(1024))
        return [(int(ids[i]), int(spend[i])) for i in range(n)]


def chunk_work(piece, remaining, allowance): return lib().fjo_chunk_work(_u32(piece), _u32(remaining), _u32(allowance))
def chunk_merged_work(piece, remaining, allowance): return lib().fjo_chunk_merged_work(_u32(piece), _u32(remaining), _u32(allowance))


def reservations_fit(page_tokens, max_context, reservations):
    r = np.array(list(reservations), np.uint64)
    return bool(lib().fjo_reservations_fit(_u32(page_tokens), _u32(max_context), _p(r), _sz(r.size)))


def prefill_plan(sequence, chunk, tail_chunk):
    out = np.zeros(4096, np.uint32)
    n = lib().fjo_prefill_plan(_u32(sequence), _u32(chunk), _u32(tail_chunk), _p(out), _sz(out.size))
    return [int(v) for v in out[:n]]


def pack_step(lanes_start, lanes_tokens, lanes_logical_len, tables, page_tokens):
    """tables [lanes, table_pages, 2]. Returns dict of the packed metadata arrays."""
    start, tokens, llen = (np.ascontiguousarray(a, np.uint32) for a in (lanes_start, lanes_tokens, lanes_logical_len))
    tables = np.ascontiguousarray(tables, np.uint32)
    lanes, table_pages = tables.shape[0], tables.shape[1]
    rows_cap = int(tokens.sum())
    out = {k: np.zeros(lanes, np.uint32) for k in ("logical_lengths", "query_starts", "absolute_positions", "activity")}
    out["cu_seqlens"] = np.zeros(lanes + 1, np.uint32)
    for k in ("positions", "slot_mapping", "row_lane"):
        out[k] = np.zeros(max(rows_cap, 1), np.uint32)
    rows = lib().fjo_pack_step(_p(start), _p(tokens), _p(llen), _sz(lanes), _p(tables), _sz(table_pages), _u32(page_tokens),
                               _p(out["logical_lengths"]), _p(out["query_starts"]), _p(out["absolute_positions"]), _p(out["activity"]),
                               _p(out["cu_seqlens"]), _p(out["positions"]), _p(out["slot_mapping"]), _p(out["row_lane"]), _sz(rows_cap))
    if rows < 0:
        raise OracleError(INVALID_INPUT)
    for k in ("positions", "slot_mapping", "row_lane"):
        out[k] = out[k][:rows]
    out["rows"] = int(rows)
    return out
