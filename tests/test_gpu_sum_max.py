"""Sum and max of every segment in one launch, against the CPU oracle.

``swg_segreduce_sum_max_f32`` reads every value once and writes both
reductions; max must be bit-exact, sum within ``1e-5 * sqrt(len) * max|x|`` of
the fp64 sum.  Cases: the reference's eight length cases
(``python/tests/mlir/test_segmented_runtime.py:15-36``, exactly representable,
so bit-exact for the sum too), its NaN / empty case (``:151-181``), boundary
lengths at every alignment, long segments (one CTA per segment) and the
canonical 4096-segment configuration.
"""

import json
import pathlib

import numpy as np
import pytest
import torch

import oracle
import workloads
from gpu_util import (
    bits_equal_or_both_nan,
    fixture_values,
    offsets_from_lengths,
)
from swage_b200 import _native
from swage_b200._segmented_qualification import launch_sum_max_gpu

pytestmark = pytest.mark.gpu

KNOWN = json.loads(
    (pathlib.Path(__file__).parent / "golden" /
     "segmented_known_answers.json").read_text())


def from_bits(words):
    return np.array(words, dtype=np.uint32).view(np.float32)


def run(values, offsets, extra=3):
    device_values = torch.as_tensor(np.asarray(values, np.float32)).cuda()
    device_offsets = torch.as_tensor(np.asarray(offsets, np.int32)).cuda()
    segments = len(offsets) - 1
    sums = torch.full((segments + extra,), float("nan"), device="cuda")
    maxima = torch.full((segments + extra,), float("nan"), device="cuda")
    launch_sum_max_gpu(device_values, device_offsets, sums, maxima)
    torch.cuda.synchronize()
    sums, maxima = sums.cpu().numpy(), maxima.cpu().numpy()
    assert np.isnan(sums[segments:]).all(), "wrote past the last segment"
    assert np.isnan(maxima[segments:]).all(), "wrote past the last segment"
    return sums[:segments], maxima[:segments]


def check(values, offsets):
    values = np.asarray(values, dtype=np.float32)
    offsets = np.asarray(offsets, dtype=np.int32)
    sums, maxima = run(values, offsets)
    expected = oracle.segreduce_f32(values, offsets, "max",
                                    threads=oracle.max_threads())
    assert bits_equal_or_both_nan(maxima, expected)
    exact = oracle.segsum_f64(values, offsets)
    bound = oracle.sum_tolerance(values, offsets)
    error = np.abs(sums.astype(np.float64) - exact)
    assert np.all(error <= bound)
    empty = np.diff(offsets) == 0
    assert np.all(sums[empty].view(np.uint32) == 0), "empty sum != +0.0"
    assert np.all(maxima[empty] == -np.inf), "empty max != -inf"


@pytest.mark.parametrize("name", sorted(KNOWN["length_cases"]))
def test_reference_length_cases_bit_exact(name):
    case = KNOWN["length_cases"][name]
    offsets = offsets_from_lengths(case["lengths"])
    values = fixture_values(offsets[-1])
    sums, maxima = run(values, offsets)
    assert bits_equal_or_both_nan(sums, from_bits(case["sum_bits"]))
    assert bits_equal_or_both_nan(maxima, from_bits(case["max_bits"]))


def test_reference_nan_and_empty_case():
    values = np.array([1.0, np.nan, 3.0, 4.0, 5.0], dtype=np.float32)
    offsets = np.array([0, 3, 3, 5], dtype=np.int32)
    sums, maxima = run(values, offsets)
    assert np.isnan(maxima[0]) and maxima[1] == -np.inf and maxima[2] == 5.0
    assert np.isnan(sums[0]) and sums[1] == 0.0 and sums[2] == 9.0


def test_boundary_lengths_at_every_alignment():
    grid = [0, 1, 2, 3, 4, 5, 7, 8, 31, 32, 33, 127, 128, 129, 255, 256, 257,
            1023, 1024, 1025, 2047, 2048, 2049, 4095, 4096, 4097, 8193, 40000]
    rng = np.random.default_rng(23)
    for order in (grid, grid[::-1], list(rng.permutation(grid))):
        offsets = offsets_from_lengths(order)
        check(rng.standard_normal(offsets[-1]).astype(np.float32), offsets)


@pytest.mark.parametrize("shift", [1, 2, 3])
def test_misaligned_value_pointer(shift):
    rng = np.random.default_rng(shift)
    lengths = list(rng.integers(0, 300, size=100)) + [9000, 3, 20000, 0, 5]
    offsets = offsets_from_lengths(lengths)
    host = rng.standard_normal(offsets[-1] + shift).astype(np.float32)
    base = torch.as_tensor(host).cuda()
    values = base[shift:]
    assert values.data_ptr() % 16 == 4 * shift
    segments = len(lengths)
    sums = torch.empty(segments, device="cuda")
    maxima = torch.empty(segments, device="cuda")
    launch_sum_max_gpu(values, torch.as_tensor(offsets).cuda(), sums, maxima)
    torch.cuda.synchronize()
    view = host[shift:]
    expected = oracle.segreduce_f32(view, offsets, "max")
    assert bits_equal_or_both_nan(maxima.cpu().numpy(), expected)
    error = np.abs(sums.cpu().numpy() - oracle.segsum_f64(view, offsets))
    assert np.all(error <= oracle.sum_tolerance(view, offsets))


def test_long_segments_take_the_cta_mapping():
    lengths = [70000, 0, 123457, 2048 * 40, 1]
    offsets = offsets_from_lengths(lengths)
    rng = np.random.default_rng(5)
    check(rng.standard_normal(offsets[-1]).astype(np.float32), offsets)


def test_canonical_configuration_full():
    """4096 segments, lengths U{0..2048}, values N(0, 1): both outputs of the
    one launch against the oracle, and the maximum against the single-kind
    entry point bit for bit."""
    offsets = workloads.c1_offsets()
    values = workloads.normal_values(int(offsets[-1]), "cuda",
                                     workloads.SEEDS["c1"])
    check(values.cpu().numpy(), offsets)
    segments = len(offsets) - 1
    device_offsets = torch.as_tensor(offsets).cuda()
    sums = torch.empty(segments, device="cuda")
    maxima = torch.empty(segments, device="cuda")
    launch_sum_max_gpu(values, device_offsets, sums, maxima)
    alone = torch.empty(segments, device="cuda")
    _native.segreduce(_native.KIND_MAX, values.data_ptr(),
                      device_offsets.data_ptr(), alone.data_ptr(),
                      values.numel(), segments, None, _native.SCHED_WARP, 0,
                      torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(alone.view(torch.int32), maxima.view(torch.int32))


def test_validation_is_the_reference_runner_s():
    values = torch.zeros(8, device="cuda")
    offsets = torch.tensor([0, 4, 8], dtype=torch.int32, device="cuda")
    out = torch.zeros(2, device="cuda")
    with pytest.raises(ValueError, match="output has 1 elements"):
        launch_sum_max_gpu(values, offsets, out, torch.zeros(1, device="cuda"))
    with pytest.raises(ValueError, match="must not alias"):
        launch_sum_max_gpu(values, offsets, out, out)
    with pytest.raises(ValueError, match="nondecreasing"):
        bad = torch.tensor([0, 5, 4], dtype=torch.int32, device="cuda")
        launch_sum_max_gpu(values, bad, out, torch.zeros(2, device="cuda"))
    with pytest.raises(TypeError, match="torch.float32"):
        launch_sum_max_gpu(values, offsets, out,
                           torch.zeros(2, device="cuda", dtype=torch.float64))
