"""Op::Sample / Op::SampleMasked on the GPU against the oracle's restatement of
crates/forja-cpu/src/lib.rs:1553-1700 (parameter words, top-k / top-p truncation, counter-based
Gumbel-max). Indices must be identical to the oracle's on every draw of the fixed seeds used here."""
import numpy as np
import pytest

import forja_b200 as fb
from forja_b200 import Op
from oracle import fjo
from tests.gpu_util import backend, down_raw, up, up_u32

pytestmark = pytest.mark.gpu


def bits(value):
    return int(np.array([value], np.float32).view(np.uint32)[0])


def run_sample(x, params, position, allow=None):
    be = backend()
    rows = int(np.prod(x.shape[:-1]))
    out = be.alloc(fb.U32, (rows,))
    p, _ = up_u32(np.array(params, np.uint32))
    inputs = [x, p]
    if allow is not None:
        a, _ = up_u32(allow)
        inputs.append(a)
    be.run(Op.Sample(position), inputs, [out])
    return down_raw(out)


CASES = [
    # temperature, top_k, top_p, spread of the logits, width
    (0.0, 0, 1.0, 3.0, 3000),      # greedy through temperature 0
    (0.7, 1, 0.9, 3.0, 3000),      # greedy through top_k 1
    (0.8, 40, 0.95, 3.0, 3000),    # the usual serving setting
    (1.0, 5, 1.0, 3.0, 3000),      # top-k only
    (1.3, 0, 1.0, 3.0, 3000),      # plain temperature sampling over the whole row
    (1.0, 0, 0.9, 3.0, 3000),      # nucleus over the whole row
    (1.0, 0, 0.97, 0.05, 10000),   # flat logits: more than 4096 weights matter, the sorted prefix takes several passes
    (0.6, 6000, 0.999, 0.2, 10000),  # top-k larger than one pass of the sort
    (1.0, 50, 0.5, 3.0, 151936),   # vocabulary width of the benchmark models
]


@pytest.mark.parametrize("dt", [fb.F32, fb.BF16])
def test_sampled_indices_equal_the_oracle(dt):
    total = different = 0
    for case, (temperature, top_k, top_p, spread, width) in enumerate(CASES):
        rng = np.random.default_rng(100 + case)
        rows = 24 if width > 20000 else 96
        values = (rng.standard_normal((rows, width)) * spread).astype(np.float32)
        values[0, 5] = values[0, 77] = values[0].max() + 1.0  # equal maxima
        values[1, :] = 0.25                                     # everything equal
        x, xh = up(values, dt)
        for position, seed in ((0, (1, 2)), (977, (0xDEADBEEF, 0x1234))):
            params = [bits(temperature), top_k, bits(top_p), seed[0], seed[1]]
            got = run_sample(x, params, position)
            fjo.set_threads(fjo.max_threads())
            want = fjo.sample(xh, dt, params, position)
            fjo.set_threads(1)
            total += rows
            different += int(np.count_nonzero(got != want))
            if temperature == 0.0 or top_k == 1:
                assert np.array_equal(got, want), f"greedy case {case} differs"
            assert np.array_equal(got, run_sample(x, params, position)), "same seed and position must reproduce"
    # Bit-exact given equal logits. A draw could only flip where the device's expf/logf and glibc's differ in the last place
    # of a deciding key; on these fixed seeds (3 168 draws per dtype) none does, so the test demands zero differences.
    assert different == 0, f"{different} of {total} sampled indices differ from the oracle"


def test_masked_sampling_and_non_finite_logits():
    rng = np.random.default_rng(9)
    width, rows = 1000, 64
    values = rng.standard_normal((rows, width)).astype(np.float32) * 2.0
    values[2, 10] = np.inf              # infinite maximum: the nucleus keeps one candidate
    values[3, 20] = -np.inf
    values.view(np.uint32)[4, 30] = 0x7FC00001  # +NaN is the greatest value
    values.view(np.uint32)[5, 40] = 0xFFC00001  # -NaN is the least value and poisons an untruncated nucleus
    values[6, :] = -np.inf
    allow = rng.integers(0, 2 ** 32, (width + 31) // 32, dtype=np.uint64).astype(np.uint32)
    allow[-1] &= (1 << (width % 32)) - 1
    x, xh = up(values, fb.F32)
    different = total = 0
    for params in ([bits(0.9), 0, bits(0.8), 7, 8], [bits(1.1), 30, bits(1.0), 7, 8], [bits(1.0), 0, bits(1.0), 3, 4], [bits(0.0), 0, bits(1.0), 0, 0]):
        for mask in (None, allow):
            got = run_sample(x, params, 12, mask)
            want = fjo.sample(xh, fb.F32, params, 12, allow=mask)
            total += rows
            different += int(np.count_nonzero(got != want))
            if mask is not None:
                assert all((allow[t // 32] >> (t % 32)) & 1 for t in got.tolist())
            assert got[2] == want[2] and got[4] == want[4] and got[6] == want[6]
    assert different == 0, f"{different} of {total} differ"
    only = np.zeros((width + 31) // 32, np.uint32)
    only[3] = 1 << 5
    assert set(run_sample(x, [bits(1.0), 0, bits(0.9), 1, 1], 0, only).tolist()) == {3 * 32 + 5}


def test_invalid_parameters_and_masks_are_refused():
    x, _ = up(np.zeros((2, 70), np.float32), fb.F32)
    for params in ([bits(-1.0), 0, bits(1.0), 0, 0], [bits(np.nan), 0, bits(1.0), 0, 0], [bits(1.0), 0, bits(0.0), 0, 0], [bits(1.0), 0, bits(1.5), 0, 0]):
        with pytest.raises(fb.BackendError) as e:
            run_sample(x, params, 0)
        assert "InvalidInput" in str(e.value)
    good = [bits(1.0), 0, bits(1.0), 0, 0]
    empty = np.zeros(3, np.uint32)
    stray = np.array([1, 0, 1 << 7], np.uint32)  # bit 71 of a 70-wide row
    for mask in (empty, stray):
        with pytest.raises(fb.BackendError):
            run_sample(x, good, 0, mask)
    wrong_length = np.ones(2, np.uint32)
    with pytest.raises(fb.BackendError):
        run_sample(x, good, 0, wrong_length)
