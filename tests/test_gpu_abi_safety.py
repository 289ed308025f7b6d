"""GPU-side checks of the memory-safety re-check at the C ABI: tensors whose layout arithmetic
wraps 64 bits, or that reach past their allocation, are refused with InvalidInput before any
kernel is launched; quota arithmetic cannot wrap either."""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200.backend import CommandList, Layout, Op, Tensor
from tests.gpu_util import backend

pytestmark = pytest.mark.gpu


def raw_view(t, offset, shape, strides):
    layout = Layout(t.layout.dtype, offset, tuple(shape), tuple(strides))
    return Tensor(t.buffer, layout, t.byte_len, t.writable)


@pytest.mark.parametrize("offset,shape,strides", [
    (0, (3, 8), (1 << 63, 1)),            # (shape - 1) * stride wraps to 0
    (1 << 62, (1, 8), (8, 1)),            # offset * element size wraps
    ((1 << 64) - 8, (1, 8), (8, 1)),      # offset + extent wraps
    (0, (3, 8), (1 << 40, 1)),            # no wrap, simply far outside the allocation
])
def test_wrapping_or_out_of_range_views_are_refused_before_any_launch(offset, shape, strides):
    be = backend()
    a = be.tensor_from(np.ones((4, 8), np.float32), fb.F32)
    out = be.alloc(fb.F32, shape)
    bad = raw_view(a, offset, shape, strides)
    before = be.kernel_launch_count()
    for ins, outs in (([bad], [out]), ([a.slice([(0, shape[0], 1), (0, 8, 1)])], [raw_view(out, offset, shape, strides)])):
        cl = CommandList()
        cl.dispatch_many(Op.Copy(), ins, outs)
        with pytest.raises(fb.BackendError) as e:
            be.submit(cl).wait()
        assert e.value.status == fb.backend.INVALID_INPUT
    with pytest.raises(fb.BackendError):
        be.read(bad)
    assert be.kernel_launch_count() == before


def test_quota_arithmetic_does_not_wrap():
    be = fb.CudaBackend(0, memory_limit=1 << 20)
    be.alloc(fb.F32, (1024,))
    import ctypes as C
    buf = C.c_uint64(0)
    assert be._lib.fj_alloc(be._h, (1 << 64) - 1024, C.byref(buf)) == fb.backend.QUOTA_EXCEEDED
    be.close()
