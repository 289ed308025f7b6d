"""Shared helpers of the GPU parity tests: one backend per process, upload/download with the
oracle's conversions, and the reference's tolerances (support/forja-testing/src/lib.rs:23-29,
483-533: normwise relative error with f64 accumulation; f32 1e-5, f16 2e-3, bf16 1e-2,
quantized 1e-2)."""
import numpy as np

import forja_b200 as fb
from oracle import fjo

TOL = {fb.F32: 1e-5, fb.F16: 2e-3, fb.BF16: 1e-2}
QUANT_TOL = 1e-2

_backend = None


def backend():
    global _backend
    if _backend is None:
        _backend = fb.CudaBackend(0)
    return _backend


def up(values_f32, dt):
    """f32 numpy values -> device tensor of dtype dt (rounded like the oracle); returns (tensor, host storage array)."""
    host = fjo.encode(np.asarray(values_f32, np.float32), dt)
    return backend().tensor_from(host, dt), host


def up_u32(values):
    host = np.ascontiguousarray(values, np.uint32)
    return backend().tensor_from(host, fb.U32), host


def down(tensor):
    """Device tensor -> f32 numpy values (u32 tensors are returned as they are)."""
    raw = backend().read(tensor)
    if tensor.dtype in (fb.U32, fb.I32):
        return raw
    return fjo.decode(raw, tensor.dtype)


def down_raw(tensor):
    return backend().read(tensor)


def normwise(actual, expected):
    a = np.asarray(actual, np.float64).ravel()
    e = np.asarray(expected, np.float64).ravel()
    assert a.shape == e.shape
    assert np.array_equal(np.isnan(a), np.isnan(e)) and np.array_equal(np.isinf(a), np.isinf(e)), "non-finite classes differ"
    finite = np.isfinite(e)
    den = np.sqrt(np.sum(e[finite] ** 2))
    num = np.sqrt(np.sum((a[finite] - e[finite]) ** 2))
    return num / den if den > 0 else num


def assert_close(actual, expected, tol):
    err = normwise(actual, expected)
    assert err <= tol, f"normwise relative error {err:.3e} > {tol:.1e}"


def max_abs_rel(actual, expected):
    """max |a - e| / max |e|: the 'max-abs rel' bound used for bf16 / 4-bit logits (2e-2)."""
    a = np.asarray(actual, np.float64).ravel()
    e = np.asarray(expected, np.float64).ravel()
    return float(np.max(np.abs(a - e)) / max(np.max(np.abs(e)), 1e-30))
