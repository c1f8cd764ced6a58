"""Segmented sum / max on the GPU against the CPU oracle, every schedule."""

import json
import pathlib

import numpy as np
import pytest
import torch

import oracle
import workloads
from gpu_util import (
    bits_equal_or_both_nan,
    check_reduce,
    fixture_values,
    make_plan,
    offsets_from_lengths,
    run_reduce,
)
from swage_b200._segmented_qualification import launch_gpu, plan_segments

pytestmark = pytest.mark.gpu

KNOWN = json.loads(
    (pathlib.Path(__file__).parent / "golden" /
     "segmented_known_answers.json").read_text())
SCHEDULES = ["auto", "warp", "cta", "split", "persistent", "resident"]


def from_bits(words):
    return np.array(words, dtype=np.uint32).view(np.float32)


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("name", sorted(KNOWN["length_cases"]))
def test_reference_length_cases_bit_exact(name, kind, schedule):
    """The reference's eight cases: exactly representable, so every
    summation order must give these bits."""
    case = KNOWN["length_cases"][name]
    offsets = offsets_from_lengths(case["lengths"])
    values = fixture_values(offsets[-1])
    result, tail = run_reduce(values, offsets, kind, schedule)
    assert bits_equal_or_both_nan(result, from_bits(case[f"{kind}_bits"]))
    assert np.isnan(tail).all()
    assert bits_equal_or_both_nan(
        result, oracle.segreduce_f32(values, offsets, kind))


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("name", sorted(KNOWN["literal_cases"]))
def test_reference_literal_cases(name, schedule):
    case = KNOWN["literal_cases"][name]
    values = from_bits(case["values_bits"])
    result, _ = run_reduce(values, case["offsets"], case["kind"], schedule)
    assert bits_equal_or_both_nan(result, from_bits(case["expected_bits"]))


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max"])
def test_repeatable_without_stale_state(kind, schedule):
    offsets = offsets_from_lengths([0, 2, 0, 129])
    values = torch.as_tensor(fixture_values(offsets[-1])).cuda()
    device_offsets = torch.as_tensor(offsets).cuda()
    output = torch.empty(4, device="cuda")
    launch_gpu(values, device_offsets, output, kind, schedule=schedule)
    first = output.clone()
    output.fill_(float("nan"))
    launch_gpu(values, device_offsets, output, kind, schedule=schedule)
    torch.cuda.synchronize()
    assert torch.equal(output.view(torch.int32), first.view(torch.int32))


@pytest.mark.parametrize("schedule", SCHEDULES)
def test_max_signed_zero_and_nan_rules(schedule):
    values = np.array([-0.0, 0.0, 0.0, -0.0, -0.0, np.nan, 1.0, -np.inf],
                      dtype=np.float32)
    offsets = np.array([0, 2, 4, 5, 7, 8, 8], dtype=np.int32)
    result, _ = run_reduce(values, offsets, "max", schedule)
    expected = oracle.segreduce_f32(values, offsets, "max")
    assert bits_equal_or_both_nan(result, expected)
    assert result[0].tobytes() == np.float32(0.0).tobytes()
    assert result[2].tobytes() == np.float32(-0.0).tobytes()
    assert np.isnan(result[3]) and result[5] == -np.inf


LENGTH_GRID = [0, 1, 2, 3, 4, 5, 7, 8, 31, 32, 33, 63, 64, 65, 127, 128, 129,
               255, 256, 257, 1023, 1024, 1025, 2047, 2048, 2049, 4095, 4096,
               4097, 8191, 8192, 8193, 16385, 40000]


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max"])
def test_boundary_lengths_in_every_position(kind, schedule):
    """Lengths around every internal boundary, in three different orders so
    each one starts at many different alignments."""
    rng = np.random.default_rng(17)
    for order in (LENGTH_GRID, LENGTH_GRID[::-1],
                  list(rng.permutation(LENGTH_GRID))):
        offsets = offsets_from_lengths(order)
        values = rng.standard_normal(offsets[-1]).astype(np.float32)
        check_reduce(values, offsets, kind, schedule)


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("shift", [1, 2, 3])
def test_misaligned_value_pointers(kind, schedule, shift):
    rng = np.random.default_rng(shift)
    lengths = list(rng.integers(0, 300, size=200)) + [9000, 3, 20000, 0, 5]
    offsets = offsets_from_lengths(lengths)
    host = rng.standard_normal(offsets[-1] + shift + 5).astype(np.float32)
    base = torch.as_tensor(host).cuda()
    values = base[shift:shift + int(offsets[-1])]
    assert values.data_ptr() % 16 == 4 * shift
    device_offsets = torch.as_tensor(offsets).cuda()
    output = torch.full((len(lengths),), float("nan"), device="cuda")
    launch_gpu(values, device_offsets, output, kind, schedule=schedule)
    torch.cuda.synchronize()
    view = host[shift:shift + int(offsets[-1])]
    if kind == "max":
        assert bits_equal_or_both_nan(
            output.cpu().numpy(), oracle.segreduce_f32(view, offsets, "max"))
    else:
        error = np.abs(output.cpu().numpy() - oracle.segsum_f64(view, offsets))
        assert np.all(error <= oracle.sum_tolerance(view, offsets))


@pytest.mark.parametrize("schedule", SCHEDULES)
def test_trailing_values_and_oversized_output(schedule):
    """offsets[-1] < value_count and output longer than S are both legal."""
    rng = np.random.default_rng(23)
    offsets = offsets_from_lengths([5, 0, 700, 9001])
    values = rng.standard_normal(offsets[-1] + 1234).astype(np.float32)
    for kind in ("sum", "max"):
        check_reduce(values, offsets, kind, schedule)


@pytest.mark.parametrize("schedule", SCHEDULES)
def test_many_empty_segments(schedule):
    lengths = [0] * 7000 + [3] + [0] * 5000 + [10000] + [0] * 3000
    offsets = offsets_from_lengths(lengths)
    values = np.random.default_rng(2).standard_normal(
        offsets[-1]).astype(np.float32)
    for kind in ("sum", "max"):
        check_reduce(values, offsets, kind, schedule)


def test_zero_segments_is_a_no_op():
    values = torch.randn(8, device="cuda")
    offsets = torch.zeros(1, dtype=torch.int32, device="cuda")
    output = torch.full((2,), float("nan"), device="cuda")
    assert launch_gpu(values, offsets, output, "sum") is None
    torch.cuda.synchronize()
    assert torch.isnan(output).all()


def test_validation_errors_reach_the_caller():
    values = torch.randn(8, device="cuda")
    output = torch.empty(2, device="cuda")
    good = torch.tensor([0, 3, 8], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="nondecreasing"):
        launch_gpu(values, torch.tensor([0, 5, 3], dtype=torch.int32,
                                        device="cuda"), output, "sum")
    with pytest.raises(ValueError, match="exceeds value count"):
        launch_gpu(values, torch.tensor([0, 3, 9], dtype=torch.int32,
                                        device="cuda"), output, "sum")
    with pytest.raises(ValueError, match="'sum' or 'max'"):
        launch_gpu(values, good, output, "min")
    with pytest.raises(ValueError, match="exceeds device limit"):
        launch_gpu(values, good, output, "sum", block_size=4096)
    with pytest.raises(TypeError, match="must be a CUDA tensor"):
        launch_gpu(values.cpu(), good, output, "sum")
    with pytest.raises(ValueError, match="schedule must be one of"):
        launch_gpu(values, good, output, "sum", schedule="fastest")


def test_plan_mismatch_is_reported():
    plan = make_plan(offsets_from_lengths([3, 4]))
    values = torch.randn(20, device="cuda")
    offsets = torch.tensor([0, 3, 7, 9], dtype=torch.int32, device="cuda")
    output = torch.empty(3, device="cuda")
    with pytest.raises(RuntimeError, match="SWG_ERR_PLAN_MISMATCH"):
        launch_gpu(values, offsets, output, "sum", plan=plan)
    plan.close()
    with pytest.raises(RuntimeError, match="closed"):
        plan.handle


def test_plan_description_reports_histogram_and_schedule():
    offsets = workloads.c5_offsets(segments=1 << 16, total=1 << 22, giants=4,
                                   giant_length=1 << 19)
    plan = make_plan(offsets)
    info = plan.describe()
    assert info["segments"] == 1 << 16 and info["values"] == 1 << 22
    lengths = np.diff(offsets)
    assert info["max_length"] == int(lengths.max())
    assert info["split_segments"] >= int((lengths > info["tile_values"]).sum())
    assert sum(info["histogram"]) == 1 << 16
    assert info["schedule"] in (3, 4)
    plan.check()
    plan.close()


# ---- the benchmark configurations, at sizes the oracle finishes quickly ----

@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max"])
def test_config_canonical(kind, schedule):
    """4096 segments, lengths uniform in {0..2048}, N(0,1): the full size."""
    offsets = workloads.c1_offsets()
    values = workloads.normal_values(int(offsets[-1]), "cuda",
                                     workloads.SEEDS["c1"]).cpu().numpy()
    check_reduce(values, offsets, kind, schedule)


@pytest.mark.parametrize(
    "schedule", ["auto", "warp", "split", "persistent", "resident"])
def test_config_lognormal_max_reduced(schedule):
    offsets = workloads.c3_offsets(segments=1 << 15, cap=1 << 30)
    values = workloads.c3_values(offsets, "cuda").cpu().numpy()
    result = check_reduce(values, offsets, "max", schedule)
    # the planted duplicates really are ties for the maximum
    first = int(np.argmax(np.diff(offsets) > 200))
    piece = values[offsets[first]:offsets[first + 1]]
    assert (piece == result[first]).sum() >= 2


@pytest.mark.parametrize(
    "schedule", ["auto", "split", "persistent", "resident"])
@pytest.mark.parametrize("kind", ["sum", "max"])
def test_config_extreme_skew_reduced(kind, schedule):
    offsets = workloads.c5_offsets(segments=1 << 17, total=1 << 24, giants=8,
                                   giant_length=1 << 20)
    values = workloads.normal_values(int(offsets[-1]), "cuda",
                                     workloads.SEEDS["c5"]).cpu().numpy()
    check_reduce(values, offsets, kind, schedule)


def test_sum_is_bit_reproducible_and_plan_independent_of_launch_order():
    offsets = workloads.c5_offsets(segments=1 << 16, total=1 << 23, giants=4,
                                   giant_length=1 << 20)
    values = workloads.normal_values(int(offsets[-1]), "cuda", 99)
    device_offsets = torch.as_tensor(offsets).cuda()
    plan = make_plan(offsets)
    outputs = []
    for _ in range(3):
        output = torch.empty(len(offsets) - 1, device="cuda")
        launch_gpu(values, device_offsets, output, "sum", plan=plan,
                   schedule="persistent")
        outputs.append(output)
    torch.cuda.synchronize()
    plan.check()
    assert torch.equal(outputs[0].view(torch.int32),
                       outputs[1].view(torch.int32))
    assert torch.equal(outputs[0].view(torch.int32),
                       outputs[2].view(torch.int32))
    # split and persistent run the same tasks with the same combine tree
    output = torch.empty(len(offsets) - 1, device="cuda")
    launch_gpu(values, device_offsets, output, "sum", plan=plan,
               schedule="split")
    torch.cuda.synchronize()
    assert torch.equal(outputs[0].view(torch.int32), output.view(torch.int32))
    plan.close()


# ---- full-size configurations: oracle on all host cores + properties ----

def full_size_check(offsets, values, kind, planner):
    """``planner`` "host": the plan is built by the host planner from a CPU
    copy of the offsets; "device": by the GPU planner from the device-resident
    offsets, with the schedule it picks -- the path a large ``launch_gpu`` call
    takes by itself, and the one the benchmark times."""
    device_offsets = torch.as_tensor(offsets).cuda()
    if planner == "host":
        plan = make_plan(offsets)
    else:
        plan = plan_segments(device_offsets, int(values.numel()))
    segments = len(offsets) - 1
    output = torch.empty(segments, device="cuda")
    launch_gpu(values, device_offsets, output, kind, plan=plan)
    torch.cuda.synchronize()
    plan.check()
    host_values = values.cpu().numpy()
    result = output.cpu().numpy()
    threads = oracle.max_threads()
    if kind == "max":
        expected = oracle.segreduce_f32(host_values, offsets, "max",
                                        threads=threads)
        assert bits_equal_or_both_nan(result, expected)
        # idempotence: the max of per-segment maxima over singleton segments
        again = torch.empty(segments, device="cuda")
        singles = torch.arange(segments + 1, dtype=torch.int32, device="cuda")
        launch_gpu(output, singles, again, "max")
        torch.cuda.synchronize()
        assert torch.equal(again.view(torch.int32), output.view(torch.int32))
    else:
        exact = oracle.segsum_f64(host_values, offsets, threads=threads)
        bound = oracle.sum_tolerance(host_values, offsets)
        assert np.all(np.abs(result - exact) <= bound)
        # The reference's strictly sequential fp32 order is reported beside
        # it, not held to the bound: over 2**23 elements its rounding error
        # grows past 1e-5*sqrt(len)*max|x| while the GPU's tree order stays
        # well inside.
        sequential = oracle.segreduce_f32(host_values, offsets, "sum",
                                          threads=threads)
        nonempty = bound > 0
        gpu_ratio = float(np.max(np.abs(result - exact)[nonempty]
                                 / bound[nonempty]))
        cpu_ratio = float(np.max(np.abs(sequential - exact)[nonempty]
                                 / bound[nonempty]))
        print(f"worst |err|/bound: gpu {gpu_ratio:.3g}, "
              f"sequential fp32 oracle {cpu_ratio:.3g}")
        assert gpu_ratio <= 1.0 and np.isfinite(cpu_ratio)
        short = nonempty & (np.diff(offsets) <= 4096)
        assert np.all(np.abs(sequential - exact)[short] <= bound[short])
        # linearity: scaling by two is exact in fp32, so sums double exactly
        doubled = torch.empty(segments, device="cuda")
        launch_gpu(values * 2, device_offsets, doubled, "sum", plan=plan)
        torch.cuda.synchronize()
        assert torch.equal((output * 2).view(torch.int32),
                           doubled.view(torch.int32))
        # a checksum of checksums: the sum of segment sums is the grand total
        total = float(exact.sum())
        assert abs(float(output.double().sum()) - total) <= float(bound.sum())
    plan.close()


@pytest.mark.parametrize("planner", ["host", "device"])
def test_full_size_lognormal_max(planner):
    """2**20 segments, lognormal lengths, about 4.8e8 values."""
    offsets = workloads.c3_offsets()
    values = workloads.c3_values(offsets, "cuda")
    full_size_check(offsets, values, "max", planner)


@pytest.mark.parametrize("planner", ["host", "device"])
def test_full_size_extreme_skew_sum(planner):
    """2**22 segments, 2**30 values, 64 segments of 2**23."""
    offsets = workloads.c5_offsets()
    values = workloads.normal_values(int(offsets[-1]), "cuda",
                                     workloads.SEEDS["c5"])
    full_size_check(offsets, values, "sum", planner)
