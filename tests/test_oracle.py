"""The CPU oracle against the reference's known answers (no GPU needed)."""

import json
import math
import pathlib
import struct

import numpy as np
import pytest

import oracle

GOLDEN = pathlib.Path(__file__).parent / "golden"
KNOWN = json.loads((GOLDEN / "segmented_known_answers.json").read_text())


def from_bits(words):
    return np.array(words, dtype=np.uint32).view(np.float32)


def case_inputs(lengths):
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    index = np.arange(offsets[-1])
    values = (((index % 17) - 8) / 4).astype(np.float32)
    return values, offsets


def same_bits_or_both_nan(actual, expected):
    actual = np.asarray(actual, dtype=np.float32)
    expected = np.asarray(expected, dtype=np.float32)
    both_nan = np.isnan(actual) & np.isnan(expected)
    equal = actual.view(np.uint32) == expected.view(np.uint32)
    return bool(np.all(both_nan | equal))


@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("name", sorted(KNOWN["length_cases"]))
def test_c_oracle_matches_reference_length_cases(name, kind):
    case = KNOWN["length_cases"][name]
    values, offsets = case_inputs(case["lengths"])
    expected = from_bits(case[f"{kind}_bits"])
    assert same_bits_or_both_nan(
        oracle.segreduce_f32(values, offsets, kind), expected)
    # all-core run of the same arithmetic gives the same bits
    assert same_bits_or_both_nan(
        oracle.segreduce_f32(values, offsets, kind, threads=4), expected)


@pytest.mark.parametrize("name", sorted(KNOWN["literal_cases"]))
def test_c_oracle_matches_reference_literal_cases(name):
    case = KNOWN["literal_cases"][name]
    values = from_bits(case["values_bits"])
    expected = from_bits(case["expected_bits"])
    actual = oracle.segreduce_f32(values, case["offsets"], case["kind"])
    assert same_bits_or_both_nan(actual, expected)
    assert same_bits_or_both_nan(
        oracle.py_segreduce(values, case["offsets"], case["kind"]), expected)


@pytest.mark.parametrize("kind", ["sum", "max", "min"])
def test_c_and_python_restatements_agree_on_random_small_inputs(kind):
    rng = np.random.default_rng(11)
    for _ in range(20):
        lengths = rng.integers(0, 40, size=rng.integers(1, 12))
        offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
        values = rng.standard_normal(offsets[-1] + 3).astype(np.float32)
        assert same_bits_or_both_nan(
            oracle.segreduce_f32(values, offsets, kind),
            oracle.py_segreduce(values, offsets, kind))


def test_max_orders_negative_zero_below_positive_zero():
    values = np.array([-0.0, 0.0, 0.0, -0.0, -0.0], dtype=np.float32)
    result = oracle.segreduce_f32(values, [0, 2, 4, 5], "max")
    assert [struct.pack("<f", v) for v in result] == [
        struct.pack("<f", 0.0), struct.pack("<f", 0.0),
        struct.pack("<f", -0.0)]


def test_min_is_the_mirror_image_of_max():
    """kind<min> has no reference lowering; it is restated by symmetry:
    min(x) == -max(-x) bit for bit, NaN propagates, -0 below +0, +inf when
    empty."""
    rng = np.random.default_rng(12)
    lengths = rng.integers(0, 50, size=40)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    values = rng.standard_normal(offsets[-1]).astype(np.float32)
    values[rng.integers(0, values.size, size=5)] = np.nan
    low = oracle.segreduce_f32(values, offsets, "min")
    high = oracle.segreduce_f32(-values, offsets, "max")
    assert same_bits_or_both_nan(low, -high)
    zeros = np.array([-0.0, 0.0, 0.0, -0.0, 0.0], dtype=np.float32)
    result = oracle.segreduce_f32(zeros, [0, 2, 4, 5, 5], "min")
    assert [struct.pack("<f", v) for v in result] == [
        struct.pack("<f", -0.0), struct.pack("<f", -0.0),
        struct.pack("<f", 0.0), struct.pack("<f", np.inf)]


def test_sequential_sum_is_strictly_left_to_right():
    # 1e8 + 1 - 1e8 in fp32, left to right, loses the 1; any reassociation
    # that pairs the two large terms first would give 1.
    values = np.array([1e8, 1.0, -1e8], dtype=np.float32)
    assert oracle.segreduce_f32(values, [0, 3], "sum")[0] == 0.0


def test_fp64_references_and_tolerance():
    rng = np.random.default_rng(5)
    lengths = rng.integers(0, 3000, size=64)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    values = rng.standard_normal(offsets[-1]).astype(np.float32)
    exact = oracle.segsum_f64(values, offsets)
    expected = np.array([
        math.fsum(values[a:b].astype(np.float64))
        for a, b in zip(offsets[:-1], offsets[1:])])
    assert np.allclose(exact, expected, rtol=1e-13, atol=1e-12)
    sequential = oracle.segreduce_f32(values, offsets, "sum")
    bound = oracle.sum_tolerance(values, offsets)
    assert np.all(np.abs(sequential - exact) <= bound + 1e-30)


def test_element_map_rounds_the_product_and_the_sum_separately():
    """``fn(scale * x + shift)`` in fp32, no contraction: 0.1 * 10 rounds to
    1 before -1 is added (a fused multiply-add would leave 2^-26 behind);
    -0.0 is the neutral shift; |NaN| stays NaN."""
    x = np.array([10.0, -0.0, 3.0, np.nan, -np.inf], np.float32)
    got = oracle.map_f32(x, "identity", np.float32(0.1), -1.0)
    assert got[0] == 0.0
    assert np.float32(0.1).astype(np.float64) * 10.0 - 1.0 != 0.0
    unchanged = oracle.map_f32(x, "identity", 1.0, -0.0)
    assert np.array_equal(unchanged.view(np.uint32), x.view(np.uint32))
    assert oracle.map_f32(x, "identity", 1.0, 0.0)[1].view(np.uint32) == 0
    assert np.array_equal(oracle.map_f32(x, "abs")[[1, 2, 4]],
                          np.array([0.0, 3.0, np.inf], np.float32))
    assert np.isnan(oracle.map_f32(x, "abs")[3])
    assert np.array_equal(oracle.map_f32(x, "square", 2.0, 1.0)[[0, 2]],
                          np.array([441.0, 49.0], np.float32))
    expected = np.exp(np.float64(0.5) * 3.0 - 1.0)
    assert oracle.map_f32(x, "exp", 0.5, -1.0)[2] == np.float32(expected)
    assert oracle.map_f32(x, "exp")[4] == 0.0
    with pytest.raises(KeyError):
        oracle.map_f32(x, "sqrt")


def test_softmax_oracles():
    rng = np.random.default_rng(6)
    lengths = np.array([0, 1, 5, 0, 300, 33])
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    values = (2 * rng.standard_normal(offsets[-1] + 2)).astype(np.float32)
    out64 = oracle.segsoftmax_f64(values, offsets)
    out32 = oracle.segsoftmax_f32(values, offsets)
    assert np.isnan(out64[offsets[-1]:]).all()  # outside every segment
    for a, b in zip(offsets[:-1], offsets[1:]):
        if b > a:
            x = values[a:b].astype(np.float64)
            e = np.exp(x - x.max())
            assert np.allclose(out64[a:b], e / e.sum(), rtol=1e-14)
            assert abs(out64[a:b].sum() - 1) < 1e-12
    inside = slice(0, offsets[-1])
    assert np.allclose(out32[inside], out64[inside], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("n", [0, 1, 127, 128, 129, 4097, 1025])
def test_vector_add_oracle(n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    for block in (128, 1024):
        out = oracle.vadd_f32(x, y, n, block=block)
        assert np.array_equal(out.view(np.uint32), (x + y).view(np.uint32))


def test_cpu_oracle_has_the_reference_calling_convention():
    import torch

    values = torch.tensor([2.0, 3.0, 4.0, 5.0])
    offsets = torch.tensor([0, 0, 1, 4, 4], dtype=torch.int32)
    result = oracle.cpu_oracle(values, offsets, "sum")
    assert result.dtype == torch.float32 and result.device.type == "cpu"
    assert result.tolist() == [0.0, 2.0, 12.0, 0.0]
    with pytest.raises(ValueError, match="'sum' or 'max'"):
        oracle.cpu_oracle(values, offsets, "min")
