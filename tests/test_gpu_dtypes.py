"""Segmented sum / max / min over f16, bf16 and i32 values.

The reference's dialect admits these element types
(``include/swage/Dialect/Swage/IR/SwageOps.td:101-105``) and its lowering
rejects everything but f32
(``lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:110-119``), so
there is no reference result to pin; the checker is the CPU oracle:

* f16 / bf16 values are widened exactly to fp32 and reduced in fp32: max / min
  must be bit-exact against the fp32 oracle on the widened values, sum within
  ``1e-5 * sqrt(len) * max|x|`` of the fp64 sum -- the f32 rules;
* i32: wrap-around sum, signed max / min, bit-exact against the sequential
  integer oracle (integer addition is associative).

The reference's eight length cases use values ``((i % 17) - 8) / 4``, exact in
f16 and bf16 too, so their known sums must come out bit for bit.
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
from swage_b200._segmented_qualification import launch_gpu, plan_segments

pytestmark = pytest.mark.gpu

KNOWN = json.loads(
    (pathlib.Path(__file__).parent / "golden" /
     "segmented_known_answers.json").read_text())
FLOATS = [torch.float16, torch.bfloat16]
SCHEDULES = ["auto", "warp", "cta", "split", "persistent", "resident"]
INT_IDENTITY = {"sum": 0, "max": -(1 << 31), "min": (1 << 31) - 1}


def from_bits(words):
    return np.array(words, dtype=np.uint32).view(np.float32)


def run(values, offsets, kind, schedule, extra=3):
    """``values``: a CUDA tensor of the element type under test."""
    device_offsets = torch.as_tensor(np.asarray(offsets, np.int32)).cuda()
    segments = len(offsets) - 1
    if values.dtype == torch.int32:
        output = torch.full((segments + extra,), 12345, dtype=torch.int32,
                            device="cuda")
    else:
        output = torch.full((segments + extra,), float("nan"), device="cuda")
    launch_gpu(values, device_offsets, output, kind, schedule=schedule,
               extensions=True)
    torch.cuda.synchronize()
    host = output.cpu().numpy()
    if values.dtype == torch.int32:
        assert np.all(host[segments:] == 12345), "wrote past the last segment"
    else:
        assert np.isnan(host[segments:]).all(), "wrote past the last segment"
    return host[:segments]


def check_float(values, offsets, kind, schedule):
    result = run(values, offsets, kind, schedule)
    wide = values.float().cpu().numpy()  # exact widening
    offsets = np.asarray(offsets, np.int32)
    if kind == "sum":
        exact = oracle.segsum_f64(wide, offsets)
        bound = oracle.sum_tolerance(wide, offsets)
        assert np.all(np.abs(result.astype(np.float64) - exact) <= bound)
        empty = np.diff(offsets) == 0
        assert np.all(result[empty].view(np.uint32) == 0)
    else:
        expected = oracle.segreduce_f32(wide, offsets, kind)
        assert bits_equal_or_both_nan(result, expected)


def check_int(values, offsets, kind, schedule):
    result = run(values, offsets, kind, schedule)
    expected = oracle.segreduce_i32(values.cpu().numpy(),
                                    np.asarray(offsets, np.int32), kind)
    assert np.array_equal(result, expected)
    empty = np.diff(np.asarray(offsets)) == 0
    assert np.all(result[empty] == INT_IDENTITY[kind])


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("dtype", FLOATS, ids=str)
@pytest.mark.parametrize("name", sorted(KNOWN["length_cases"]))
def test_reference_length_cases_in_half_precision_inputs(name, dtype, kind,
                                                         schedule):
    case = KNOWN["length_cases"][name]
    offsets = offsets_from_lengths(case["lengths"])
    values = torch.as_tensor(fixture_values(offsets[-1])).cuda().to(dtype)
    assert torch.equal(values.float().cpu(),
                       torch.as_tensor(fixture_values(offsets[-1])))
    result = run(values, offsets, kind, schedule)
    assert bits_equal_or_both_nan(result, from_bits(case[f"{kind}_bits"]))


GRID = [0, 1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 32, 33, 127, 128, 129, 255,
        256, 257, 1023, 1024, 1025, 2047, 2048, 2049, 4095, 4096, 4097, 8193,
        40000]


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max", "min"])
@pytest.mark.parametrize("dtype", FLOATS, ids=str)
def test_half_precision_boundary_lengths(dtype, kind, schedule):
    rng = np.random.default_rng(41)
    for order in (GRID, GRID[::-1], list(rng.permutation(GRID))):
        offsets = offsets_from_lengths(order)
        values = torch.as_tensor(
            rng.standard_normal(offsets[-1]).astype(np.float32)
        ).cuda().to(dtype)
        check_float(values, offsets, kind, schedule)


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max", "min"])
def test_int32_boundary_lengths_with_wrap_around(kind, schedule):
    rng = np.random.default_rng(43)
    for order in (GRID, GRID[::-1], list(rng.permutation(GRID))):
        offsets = offsets_from_lengths(order)
        # the full int32 range: sums wrap around many times
        values = torch.as_tensor(rng.integers(
            -(1 << 31), 1 << 31, size=int(offsets[-1]),
            dtype=np.int64).astype(np.int32)).cuda()
        check_int(values, offsets, kind, schedule)


@pytest.mark.parametrize("schedule", ["warp", "split", "resident"])
@pytest.mark.parametrize("shift", [1, 3, 5, 7])
@pytest.mark.parametrize("dtype", FLOATS, ids=str)
def test_half_precision_values_at_every_phase_of_a_16_byte_line(dtype, shift,
                                                                schedule):
    rng = np.random.default_rng(shift)
    lengths = list(rng.integers(0, 300, size=150)) + [9000, 3, 20000, 0, 5]
    offsets = offsets_from_lengths(lengths)
    base = torch.as_tensor(rng.standard_normal(
        offsets[-1] + shift + 9).astype(np.float32)).cuda().to(dtype)
    values = base[shift:shift + int(offsets[-1]) + 2]
    assert values.data_ptr() % 16 == 2 * shift
    check_float(values, offsets, "sum", schedule)
    check_float(values, offsets, "max", schedule)


@pytest.mark.parametrize("shift", [1, 2, 3])
def test_int32_values_at_every_phase(shift):
    rng = np.random.default_rng(shift + 10)
    lengths = list(rng.integers(0, 300, size=150)) + [9000, 3, 20000, 0, 5]
    offsets = offsets_from_lengths(lengths)
    base = torch.as_tensor(rng.integers(
        -1000, 1000, size=int(offsets[-1]) + shift).astype(np.int32)).cuda()
    values = base[shift:]
    assert values.data_ptr() % 16 == 4 * shift
    for schedule in ("split", "resident", "warp"):
        check_int(values, offsets, "sum", schedule)
        check_int(values, offsets, "min", schedule)


@pytest.mark.parametrize("dtype", FLOATS + [torch.int32], ids=str)
def test_extreme_skew_shape_through_the_device_planner(dtype):
    """The extreme-skew shape at 1/64 of its size, planned on the GPU (the
    path a large launch takes by itself)."""
    offsets = workloads.c5_offsets(segments=1 << 16, total=1 << 24, giants=4,
                                   giant_length=1 << 21)
    count = int(offsets[-1])
    if dtype == torch.int32:
        rng = np.random.default_rng(3)
        values = torch.as_tensor(rng.integers(
            -(1 << 31), 1 << 31, size=count, dtype=np.int64
        ).astype(np.int32)).cuda()
        for kind in ("sum", "max"):
            check_int(values, offsets, kind, "auto")
    else:
        values = workloads.normal_values(count, "cuda", 5).to(dtype)
        for kind in ("sum", "max"):
            check_float(values, offsets, kind, "auto")


def test_a_plan_serves_every_element_type():
    offsets = workloads.c3_offsets(segments=1 << 13)
    count = int(offsets[-1])
    device_offsets = torch.as_tensor(offsets).cuda()
    plan = plan_segments(device_offsets, count)
    try:
        base = workloads.normal_values(count, "cuda", 9)
        for values in (base, base.half(), base.bfloat16(),
                       (base * 1000).to(torch.int32)):
            out_dtype = (torch.int32 if values.dtype == torch.int32
                         else torch.float32)
            output = torch.empty(len(offsets) - 1, dtype=out_dtype,
                                 device="cuda")
            launch_gpu(values, device_offsets, output, "max", plan=plan,
                       extensions=True)
            torch.cuda.synchronize()
            if values.dtype == torch.int32:
                expected = oracle.segreduce_i32(values.cpu().numpy(), offsets,
                                                "max")
                assert np.array_equal(output.cpu().numpy(), expected)
            else:
                expected = oracle.segreduce_f32(
                    values.float().cpu().numpy(), offsets, "max")
                assert bits_equal_or_both_nan(output.cpu().numpy(), expected)
        plan.check()
    finally:
        plan.close()


def test_the_reference_s_type_errors_are_kept_without_extensions():
    offsets = torch.tensor([0, 4, 8], dtype=torch.int32, device="cuda")
    out = torch.zeros(2, device="cuda")
    with pytest.raises(TypeError, match="values must have dtype torch.float32"):
        launch_gpu(torch.zeros(8, device="cuda", dtype=torch.float16), offsets,
                   out, "sum")
    with pytest.raises(TypeError, match="values must have dtype torch.float32"):
        launch_gpu(torch.zeros(8, device="cuda", dtype=torch.int32), offsets,
                   out, "sum")
    with pytest.raises(TypeError, match="torch.int32 for int32 values"):
        launch_gpu(torch.zeros(8, device="cuda", dtype=torch.int32), offsets,
                   out, "sum", extensions=True)
    with pytest.raises(TypeError, match="output must have dtype torch.float32"):
        launch_gpu(torch.zeros(8, device="cuda", dtype=torch.float16), offsets,
                   torch.zeros(2, device="cuda", dtype=torch.float16), "sum",
                   extensions=True)
