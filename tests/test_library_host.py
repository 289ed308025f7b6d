"""CPU-side checks of the product library: it loads, exports every symbol the header declares,
refuses to create a backend without a device, and its host logic (program recognition, layout
views) behaves like the reference's. No kernel runs here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import forja_b200 as fb
from forja_b200 import _lib
from tests import ir_programs as ir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "forja_cuda.h")).read()
    declared = sorted(set(re.findall(r"\b(fj_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 40
    lib = C.CDLL(_lib.library_path())
    missing = [name for name in declared if not hasattr(lib, name)]
    assert missing == []
    assert sorted(_lib.EXPORTS) == declared


def test_library_does_not_link_the_oracle_or_python():
    import subprocess
    out = subprocess.run(["ldd", _lib.library_path()], capture_output=True, text=True).stdout
    assert "fjo" not in out and "python" not in out and "torch" not in out


def _classify(prog):
    lib = _lib.load()
    insts, outs = prog.words()
    kernel = C.c_uint32(0)
    consts = (C.c_float * 4)()
    st = lib.fj_program_classify(prog.kind, insts.ctypes.data_as(C.c_void_p), len(insts), outs.ctypes.data_as(C.c_void_p), len(outs), C.byref(kernel), consts)
    return st, kernel.value, tuple(consts)


def test_program_recognition_captures_constants():
    assert _classify(ir.add())[:2] == (0, 1)
    assert _classify(ir.silu_mul())[:2] == (0, 2)
    st, k, c = _classify(ir.rms_norm(1e-6))
    assert (st, k) == (0, 3) and c[0] == np.float32(1e-6)
    st, k, c = _classify(ir.residual_norm(1e-5))
    assert (st, k) == (0, 4) and c[0] == np.float32(1e-5)
    st, k, c = _classify(ir.qk_norm_rope(1e-6, 1e6, 128.0))
    assert (st, k) == (0, 5)
    assert c[0] == np.float32(1e-6) and c[1] == np.float32(1e6) and c[2] == 128.0 and c[3] == np.float32(-2.0 / 128.0)
    st, k, c = _classify(ir.rope_pairs(1e5, 64.0))
    assert (st, k) == (0, 6) and c[1] == np.float32(1e5) and c[3] == np.float32(-2.0 / 64.0)


def test_unknown_programs_are_refused_not_interpreted():
    assert _classify(ir.softmax())[0] == fb.backend.UNSUPPORTED_OPERATION
    # a different association order is a different program: x * (inv * w)
    from oracle import fjo
    p = fjo.Program(fjo.ROW)
    v, w = p.input(0), p.input(1)
    s = p.reduce(fjo.R_SUM, p.binary(fjo.B_MUL, v, v))
    inv = p.unary(fjo.U_RSQRT, p.binary(fjo.B_ADD, p.binary(fjo.B_DIV, s, p.cast(fjo.V_F32, p.extent(1))), p.constant(1e-6)))
    p.output(0, p.binary(fjo.B_MUL, v, p.binary(fjo.B_MUL, inv, w)))
    assert _classify(p)[0] == fb.backend.UNSUPPORTED_OPERATION
    # forward references are rejected
    bad = fjo.Program(fjo.MAP)
    bad.insts.append((fjo.T_UNARY, fjo.U_NEG, 5, 0))
    bad.output(0, 0)
    assert _classify(bad)[0] == fb.backend.UNSUPPORTED_OPERATION


def test_commuted_operands_still_match():
    from oracle import fjo
    p = fjo.Program(fjo.MAP)
    g, u = p.input(0), p.input(1)
    p.output(0, p.binary(fjo.B_MUL, u, p.binary(fjo.B_MUL, p.unary(fjo.U_SIGMOID, g), g)))
    assert _classify(p)[:2] == (0, 2)


def test_backend_creation_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(fb.BackendError) as e:
        fb.CudaBackend(0)
    assert e.value.status == fb.backend.ALLOCATION_FAILED


def test_layout_views_match_reference_semantics():
    # crates/forja-core/src/layout.rs: slice / reshape / permute / broadcast are metadata only
    base = fb.Layout.contiguous(fb.F32, (4, 6, 8))
    assert base.strides == (48, 8, 1)
    s = base.slice([(1, 2, 1), (0, 3, 2), (4, 4, 1)])
    assert (s.offset, s.shape, s.strides) == (48 + 4, (2, 3, 4), (48, 16, 1))
    p = base.permute([1, 0, 2])
    assert (p.shape, p.strides) == ((6, 4, 8), (8, 48, 1)) and not p.is_contiguous()
    with pytest.raises(fb.BackendError):
        p.reshape((24, 8))
    b = fb.Layout.contiguous(fb.F32, (8,)).broadcast((4, 6, 8))
    assert b.strides == (0, 0, 1)
    with pytest.raises(fb.BackendError):
        base.slice([(0, 5, 1), (0, 6, 1), (0, 8, 1)])


def _span(offset, shape, strides, dtype=fb.F32):
    lib = _lib.load()
    t = _lib.FjTensor()
    t.buffer, t.dtype, t.rank, t.offset = 1, dtype, len(shape), offset
    for a, (n, s) in enumerate(zip(shape, strides)):
        t.shape[a], t.strides[a] = n, s
    lo, hi = C.c_uint64(0), C.c_uint64(0)
    st = lib.fj_tensor_byte_span(C.byref(t), C.byref(lo), C.byref(hi))
    return st, lo.value, hi.value


def test_tensor_byte_span_uses_checked_arithmetic():
    """The one memory-safety re-check at the boundary must not wrap: a view whose strides or offset
    overflow 64 bits addresses nothing valid and is refused (crates/forja-core/src/layout.rs uses
    checked_mul / checked_add for the same arithmetic)."""
    INVALID = fb.backend.INVALID_INPUT
    assert _span(3, (4, 5), (5, 1)) == (0, 12, (3 + 19 + 1) * 4)
    assert _span(0, (2, 3), (0, 1), fb.BF16) == (0, 0, 6)           # broadcast axis
    assert _span(7, (4, 0, 2), (1 << 62, 1, 1)) == (0, 28, 28)       # empty view: nothing is addressed
    assert _span(0, (3,), (1 << 63,))[0] == INVALID                  # 2 * 2^63 wraps to 0
    assert _span(0, (2, 2), ((1 << 64) - 1, 2))[0] == INVALID        # sum of steps wraps
    assert _span(1 << 62, (1,), (1,))[0] == INVALID                  # offset * 4 wraps
    assert _span((1 << 64) - 1, (1,), (1,), fb.U32)[0] == INVALID    # last + 1 wraps
    assert _span(0, (1 << 31, 1 << 31, 8), (1 << 33, 4, 1 << 60))[0] == INVALID
    st, lo, hi = _span(0, (1,), (1,), 9)
    assert st == INVALID                                              # dtype out of range


def test_bounded_exchange_wait_gives_up_at_its_deadline():
    """The host waits of the expert-parallel exchange poll with a deadline (a peer that never posts must not hang the other
    ranks' hosts). Exercised here against a simulated clock: no device, no NCCL."""
    lib = _lib.load()
    polls = C.c_uint64(0)
    # the condition turns true at the 5th poll, well inside the deadline
    assert lib.fj_ep_poll_selftest(1000, 5, 1, C.byref(polls)) == 1 and polls.value == 5
    # a condition that never turns true: the wait ends once the clock has passed the deadline
    assert lib.fj_ep_poll_selftest(100, 0, 7, C.byref(polls)) == 0
    assert 100 // 7 <= polls.value <= 100 // 7 + 2
    # true only after the deadline: not seen
    assert lib.fj_ep_poll_selftest(10, 50, 1, C.byref(polls)) == 0 and polls.value < 50
    # no deadline: waits as long as it takes
    assert lib.fj_ep_poll_selftest(0, 300, 1000, C.byref(polls)) == 1 and polls.value == 300
