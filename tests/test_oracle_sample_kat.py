"""The sampler's own tests in the reference (crates/forja-cpu/src/lib.rs:2491-2700, helpers :3269-3306), restated against the
oracle: greedy selection at edge values and widths, counter determinism, the exact allowed sets of top-k / top-p / masks,
mask validation, the full candidate set beyond 1024 values, known distributions under a chi-squared bound, refused
parameters. Same rows, parameters, position ranges and bounds as the reference uses. CPU only."""
import struct

import numpy as np
import pytest

from oracle import fjo


def bits(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


def params(temperature, top_k, top_p, seed):
    return [bits(temperature), top_k, bits(top_p), seed & 0xFFFFFFFF, seed >> 32]


def sample_row(row, parameters, position, allow=None):
    return int(fjo.sample(np.asarray(row, np.float32).reshape(1, -1), fjo.F32, parameters, position=position, allow=allow)[0])


def total_order_key(value_bits):
    """Key of f32::total_cmp: negative values in reverse bit order below positive ones."""
    return (~value_bits & 0xFFFFFFFF) if value_bits >> 31 else (value_bits | 0x80000000)


def test_greedy_sampling_matches_argmax_for_edge_values_and_widths():  # lib.rs:2491-2520
    for width in (1, 7, 33, 4097, 151936):
        row = (np.arange(width) % 19).astype(np.float32) - 9.0
        if width >= 7:
            row[:7] = [-np.inf, -0.0, 0.0, np.inf, np.nan, np.nan, np.inf]
        keys = [total_order_key(int(b)) for b in row.view(np.uint32)]
        expected = max(range(width), key=lambda i: (keys[i], i))  # max_by keeps the last of equal maxima
        for parameters in (params(0.0, 0, 1.0, 7), params(0.7, 1, 0.9, 7)):
            assert sample_row(row, parameters, 33) == expected


def test_sampled_tokens_are_counter_deterministic():  # lib.rs:2523-2534
    row = [0.1, -0.3, 1.2, 0.7, 0.0, 0.9, -1.0]
    parameters = params(0.7, 0, 1.0, 0xFEEDBEEFDEADCAFE)
    first = [sample_row(row, parameters, position) for position in range(128)]
    second = [sample_row(row, parameters, position) for position in range(128)]
    assert first == second
    assert any(a != b for a, b in zip(first, first[1:]))


def test_top_k_and_top_p_keep_only_the_exact_allowed_set():  # lib.rs:2537-2547
    row = [10.0, 9.0, 8.0, 1.0, 0.0, -1.0, -2.0]
    top_k, top_p, combined = params(1.0, 3, 1.0, 11), params(1.0, 0, 0.7, 11), params(1.0, 2, 0.999, 11)
    for position in range(4096):
        assert sample_row(row, top_k, position) <= 2
        assert sample_row(row, top_p, position) <= 1
        assert sample_row(row, combined, position) <= 1


def test_masked_sampling_conditions_every_sampling_mode():  # lib.rs:2550-2566
    row = [10.0, 9.0, 8.0, 7.0, 6.0, 5.0, 4.0]
    allow = np.array([0b01010010], np.uint32)
    for parameters in (params(0.0, 0, 1.0, 11), params(1.0, 2, 1.0, 12), params(1.0, 0, 0.8, 13), params(0.7, 0, 1.0, 14)):
        for position in range(256):
            assert sample_row(row, parameters, position, allow) in (1, 4, 6)


def test_all_allowed_mask_preserves_unconstrained_sampling():  # lib.rs:2605-2617
    row = [index / 7.0 for index in range(33)]
    allow = np.array([0xFFFFFFFF, 1], np.uint32)
    parameters = params(0.7, 7, 0.9, 0xFEEDBEEF)
    for position in range(512):
        assert sample_row(row, parameters, position, allow) == sample_row(row, parameters, position)


def test_masked_sampling_refuses_empty_and_padding_bits():  # lib.rs:2620-2631
    row = [0.0] * 7
    parameters = params(1.0, 0, 1.0, 1)
    with pytest.raises(fjo.OracleError):
        sample_row(row, parameters, 0, np.array([0], np.uint32))
    with pytest.raises(fjo.OracleError):
        sample_row(row, parameters, 0, np.array([1 << 7], np.uint32))
    assert sample_row(row, parameters, 0, np.array([1 << 6], np.uint32)) == 6


def test_top_p_uses_the_full_candidate_set_beyond_1024_values():  # lib.rs:2634-2640
    """1025 equal logits at top_p 0.9995: the nucleus needs all 1025 candidates (1024 of them hold 0.99902). The reference
    asks its truncation helper directly; through the sampler the same fact shows as the last candidate being drawn."""
    row = [0.0] * 1025
    parameters = params(1.0, 0, 0.9995, 11)
    seen = {sample_row(row, parameters, position) for position in range(12000)}
    assert 1024 in seen and len(seen) > 1000


def chi_squared(row, parameters, expected, trials=20000):  # lib.rs:3283-3306
    counts = np.zeros(len(row), np.int64)
    for position in range(trials):
        counts[sample_row(row, parameters, position)] += 1
    statistic = sum((counts[i] - p * trials) ** 2 / (p * trials) for i, p in enumerate(expected) if p > 0.0)
    assert statistic < 16.3, f"chi-squared statistic was {statistic}"
    for i, p in enumerate(expected):
        if p == 0.0:
            assert counts[i] == 0


def test_sampling_distributions_match_known_probabilities():  # lib.rs:2642-2663
    chi_squared([0.0, 0.0, 0.0, 0.0], params(1.0, 0, 1.0, 91), [0.25] * 4)
    chi_squared([2.0, 1.0, 0.0], params(1.0, 2, 1.0, 92), [0.7310586, 0.2689414, 0.0])
    chi_squared([2.0, 1.0, 0.0], params(1.0, 0, 0.8, 93), [0.7310586, 0.2689414, 0.0])
    chi_squared([2.0, 1.0, 0.0, -1.0], params(1.0, 3, 0.95, 94), [0.66524094, 0.24472848, 0.09003057, 0.0])


def test_sample_refuses_invalid_live_parameters():  # lib.rs:2666-2700
    row = [0.0] * 7
    for bad in ([bits(float("nan")), 0, bits(1.0), 0, 0], [bits(-1.0), 0, bits(1.0), 0, 0], [bits(1.0), 0, bits(0.0), 0, 0],
                [bits(1.0), 0, bits(1.5), 0, 0], [bits(float("inf")), 0, bits(1.0), 0, 0]):
        with pytest.raises(fjo.OracleError):
            sample_row(row, bad, 0)
