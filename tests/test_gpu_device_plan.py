"""Offsets validation and planning on the GPU: same verdicts as the host
pass, same results as the host-built plans."""

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
    offsets_from_lengths,
)
from swage_b200 import _native
from swage_b200 import _segmented_qualification as runner
from swage_b200._segmented_qualification import (
    launch_gpu,
    launch_softmax_gpu,
    plan_segments,
)

pytestmark = pytest.mark.gpu

KNOWN = json.loads(
    (pathlib.Path(__file__).parent / "golden" /
     "segmented_known_answers.json").read_text())


def device_verdict(offsets, value_count, output_count=None):
    offsets = np.asarray(offsets, dtype=np.int32)
    tensor = torch.as_tensor(offsets).cuda()
    segments = len(offsets) - 1
    if output_count is None:
        output_count = segments
    stream = torch.cuda.current_stream().cuda_stream
    return _native.validate_offsets_device(
        tensor.data_ptr(), segments, value_count, output_count, stream)


def host_verdict(offsets, value_count, output_count=None):
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    if output_count is None:
        output_count = len(offsets) - 1
    return _native.validate_offsets(offsets.ctypes.data, len(offsets),
                                    value_count, output_count)


BAD_OFFSETS = {
    "nonzero_start": ([1, 2, 3], 3),
    "nonzero_start_and_negative": ([5, -1, 3], 3),
    "negative": ([0, -1, 3], 3),
    "negative_then_decreasing": ([0, 4, -2, 1], 4),
    "decreasing": ([0, 3, 2, 4], 4),
    "decreasing_before_negative": ([0, 3, 2, -4], 4),
    "exceeds": ([0, 2, 5], 4),
    "decreasing_at_the_end": ([0, 2, 1], 4),
    "output_small": ([0, 1, 2, 3], 3),
}


@pytest.mark.parametrize("name", sorted(BAD_OFFSETS))
def test_device_verdict_equals_host_verdict(name):
    offsets, value_count = BAD_OFFSETS[name]
    output_count = 2 if name == "output_small" else None
    reason, index, _, _ = device_verdict(offsets, value_count, output_count)
    assert (reason, index) == host_verdict(offsets, value_count, output_count)
    assert reason != "ok"


def test_first_violation_deep_inside_a_large_array():
    rng = np.random.default_rng(11)
    lengths = rng.integers(0, 9, size=1 << 20)
    offsets = offsets_from_lengths(lengths)
    total = int(offsets[-1])
    assert device_verdict(offsets, total)[:2] == ("ok", -1)
    for where, value in ((777_777, -5), (123_456, None), (1 << 20, None)):
        broken = offsets.copy()
        if value is None:
            broken[where] = broken[where - 1] - 1   # one step down
        else:
            broken[where] = value
        # a later violation must not win over the first one
        broken[900_000] = -1
        reason, index, _, _ = device_verdict(broken, total)
        assert (reason, index) == host_verdict(broken, total)
    reason, index, _, last = device_verdict(offsets, total - 1)
    assert (reason, index, last) == ("exceeds_values", 1 << 20, total)


def test_digest_depends_on_content_and_order():
    base = offsets_from_lengths([3, 0, 5, 2, 2])
    swapped = offsets_from_lengths([0, 3, 5, 2, 2])
    other = offsets_from_lengths([3, 0, 5, 2, 3])
    digests = {device_verdict(o, int(o[-1]))[2] for o in (base, swapped, other)}
    assert len(digests) == 3
    assert device_verdict(base, 12)[2] == device_verdict(base.copy(), 12)[2]


def test_launch_raises_the_reference_messages_without_a_host_copy():
    """A launch large enough to be planned validates on the device."""
    rng = np.random.default_rng(5)
    lengths = rng.integers(0, 64, size=4096)
    offsets = offsets_from_lengths(lengths)
    total = int(offsets[-1])
    assert total + 4096 >= runner._PLAN_THRESHOLD
    values = torch.zeros(total, device="cuda")
    output = torch.empty(4096, device="cuda")
    cases = (
        (lambda o: o.__setitem__(0, 1), "start at zero"),
        (lambda o: o.__setitem__(100, -3), "must not be negative"),
        (lambda o: o.__setitem__(200, o[199] - 1), "nondecreasing"),
        (lambda o: o.__setitem__(4096, total + 7),
         f"final offset {total + 7} exceeds value count {total}"),
    )
    for damage, message in cases:
        broken = offsets.copy()
        damage(broken)
        with pytest.raises(ValueError, match=message):
            launch_gpu(values, torch.as_tensor(broken).cuda(), output, "sum")
    with pytest.raises(ValueError, match="output has 4000 elements"):
        launch_gpu(values, torch.as_tensor(offsets).cuda(), output[:4000],
                   "sum")


LENGTH_MIXES = {
    "one_value": [1],
    "one_empty": [0],
    "all_empty": [0] * 5000,
    "empties_around": [0, 0, 7, 0, 0, 0, 3000, 0],
    "exact_tile": [2030],
    "tile_plus_header": [2031],
    "two_tiles": [2030, 2030],
    "straddle": [2029, 5, 2025, 1, 1, 4000],
    "long_then_short": [100000, 1, 2, 3],
    "short_then_long": [1, 2, 3, 100000, 5],
    "three_long": [50000, 60000, 70000],
    "cut_at_last_value": [2030, 1, 2029, 2, 2031 * 3 - 2],
    "header_last_in_tile": [2030, 10, 2020, 10],
    "many_tiny": [3] * 40000,
    "single_giant": [3_000_000],
}


def device_plan(offsets, value_count=None, op="reduce"):
    offsets = np.asarray(offsets, dtype=np.int32)
    if value_count is None:
        value_count = int(offsets[-1])
    return plan_segments(torch.as_tensor(offsets).cuda(), value_count, op)


@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("name", sorted(LENGTH_MIXES))
def test_device_planned_reduce_matches_the_oracle(name, kind):
    offsets = offsets_from_lengths(LENGTH_MIXES[name])
    rng = np.random.default_rng(len(name))
    values = rng.standard_normal(int(offsets[-1]) + 3).astype(np.float32)
    plan = device_plan(offsets)
    try:
        for schedule in ("split", "persistent", "resident"):
            check_reduce(values, offsets, kind, schedule, plan=plan)
        plan.check()
    finally:
        plan.close()


@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("name", sorted(KNOWN["length_cases"]))
def test_reference_length_cases_with_a_device_plan(name, kind):
    case = KNOWN["length_cases"][name]
    offsets = offsets_from_lengths(case["lengths"])
    values = fixture_values(offsets[-1])
    plan = device_plan(offsets)
    try:
        result = check_reduce(values, offsets, kind, "split", plan=plan)
    finally:
        plan.close()
    expected = np.array(case[f"{kind}_bits"], dtype=np.uint32).view(np.float32)
    assert bits_equal_or_both_nan(result, expected)


def test_device_plan_statistics_equal_the_host_plan():
    offsets = workloads.c3_offsets(segments=1 << 16)
    host = plan_segments(torch.as_tensor(offsets))
    device = device_plan(offsets)
    try:
        a, b = host.describe(), device.describe()
        for key in ("segments", "values", "max_length", "histogram",
                    "elements_in_bin", "schedule"):
            assert a[key] == b[key], key
        assert abs(a["mean_length"] - b["mean_length"]) < 1e-6
        # a segment counts for its values plus four header items
        items = int(offsets[-1]) + 4 * (len(offsets) - 1)
        assert b["tasks"] == -(-items // 2031)
        # two partial slots per tile; the cut segments are those longer than
        # a tile plus the shorter ones a boundary happens to fall in
        assert b["partial_slots"] == 2 * b["tasks"]
        assert b["pack_tasks"] + b["chunk_tasks"] == b["tasks"]
        assert b["split_segments"] >= int((np.diff(offsets) > 2031).sum())
    finally:
        host.close()
        device.close()


@pytest.mark.parametrize("workload", ["c1", "c3", "c5"])
@pytest.mark.parametrize("kind", ["sum", "max"])
def test_workload_shapes_with_a_device_plan(workload, kind):
    offsets = {
        "c1": lambda: workloads.c1_offsets(segments=20000),
        "c3": lambda: workloads.c3_offsets(segments=1 << 15),
        "c5": lambda: workloads.c5_offsets(
            segments=1 << 16, total=1 << 24, giants=2, giant_length=1 << 22),
    }[workload]()
    rng = np.random.default_rng(3)
    values = rng.standard_normal(int(offsets[-1])).astype(np.float32)
    plan = device_plan(offsets)
    try:
        check_reduce(values, offsets, kind, "auto", plan=plan)
        check_reduce(values, offsets, kind, "split", plan=plan)
        plan.check()
    finally:
        plan.close()


def test_trailing_unused_values_are_legal():
    offsets = offsets_from_lengths([5000, 0, 70000, 33])
    rng = np.random.default_rng(9)
    values = rng.standard_normal(int(offsets[-1]) + 4099).astype(np.float32)
    plan = device_plan(offsets, value_count=values.size)
    try:
        check_reduce(values, offsets, "sum", "split", plan=plan)
    finally:
        plan.close()


def test_device_plan_rejects_bad_offsets():
    with pytest.raises(ValueError, match="nondecreasing"):
        device_plan([0, 5, 4, 9], value_count=9)
    with pytest.raises(ValueError, match="exceeds value count"):
        device_plan([0, 5, 9], value_count=8)


def test_automatic_launch_plans_on_the_device_and_caches_by_content():
    runner.clear_plan_cache()
    offsets = workloads.c3_offsets(segments=1 << 14)
    rng = np.random.default_rng(1)
    values_host = rng.standard_normal(int(offsets[-1])).astype(np.float32)
    values = torch.as_tensor(values_host).cuda()
    device_offsets = torch.as_tensor(offsets).cuda()
    output = torch.empty(len(offsets) - 1, device="cuda")
    launch_gpu(values, device_offsets, output, "max")
    assert len(runner._device_plan_cache) == 1
    assert len(runner._plan_cache) == 0, "the offsets were copied to the host"
    launch_gpu(values, device_offsets.clone(), output, "max")
    assert len(runner._device_plan_cache) == 1, "same content, same plan"
    torch.cuda.synchronize()
    expected = oracle.segreduce_f32(values_host, offsets, "max",
                                    threads=oracle.max_threads())
    assert bits_equal_or_both_nan(output.cpu().numpy(), expected)
    shifted = offsets.copy()
    shifted[1] += 1 if shifted[2] > shifted[1] else 0
    launch_gpu(values, torch.as_tensor(shifted).cuda(), output, "max")
    assert len(runner._device_plan_cache) == (
        2 if not np.array_equal(shifted, offsets) else 1)
    runner.clear_plan_cache()


def test_status_can_be_read_without_synchronising():
    """``peek`` reads the kernels' error word from pinned host memory: no CUDA
    call, so the launch functions can afford it before every launch.  After
    clean launches both it and the synchronising ``check`` stay silent."""
    offsets = workloads.c5_offsets(segments=1 << 14, total=1 << 22, giants=2,
                                   giant_length=1 << 20)
    values = torch.randn(int(offsets[-1]), device="cuda")
    output = torch.empty(len(offsets) - 1, device="cuda")
    plan = device_plan(offsets)
    try:
        for schedule in ("split", "persistent", "resident"):
            launch_gpu(values, torch.as_tensor(offsets).cuda(), output, "sum",
                       plan=plan, schedule=schedule)
            plan.peek()
        torch.cuda.synchronize()
        plan.peek()
        plan.check()
    finally:
        plan.close()


def test_a_wait_that_runs_out_is_reported_and_the_plan_stays_usable():
    """Every device-side wait is bounded.  The self-test kernel waits a
    millisecond for a copy nobody issues, gives up and returns; the error
    reaches the host both ways (without a CUDA call through ``peek``, with a
    synchronisation through ``check``), the NEXT drop-in launch raises instead
    of passing silently, and after that the plan works as before."""
    offsets = workloads.c5_offsets(segments=1 << 14, total=1 << 22, giants=2,
                                   giant_length=1 << 20)
    host_values = np.random.default_rng(6).standard_normal(
        int(offsets[-1])).astype(np.float32)
    values = torch.as_tensor(host_values).cuda()
    device_offsets = torch.as_tensor(offsets).cuda()
    output = torch.empty(len(offsets) - 1, device="cuda")
    plan = device_plan(offsets)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        _native.plan_selftest_timeout(plan.handle, 1000, stream)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="SWG_ERR_DEVICE_TIMEOUT"):
            launch_gpu(values, device_offsets, output, "sum", plan=plan)
        with pytest.raises(RuntimeError, match="SWG_ERR_DEVICE_TIMEOUT"):
            plan.check()
        plan.check()  # reported and cleared
        plan.peek()
        check_reduce(host_values, offsets, "sum", "split", plan=plan)
        check_reduce(host_values, offsets, "max", "persistent", plan=plan)
        plan.check()
    finally:
        plan.close()


def test_two_streams_over_the_same_offsets_get_a_plan_each():
    """Launches that share a plan share its merge scratch; the drop-in call
    therefore caches plans per stream.  Two streams reducing over the same CSR
    structure at the same time must both match the oracle."""
    runner.clear_plan_cache()
    offsets = workloads.c5_offsets(segments=1 << 16, total=1 << 24, giants=4,
                                   giant_length=1 << 21)
    segments = len(offsets) - 1
    device_offsets = torch.as_tensor(offsets).cuda()
    host_values = [np.random.default_rng(s).standard_normal(
        int(offsets[-1])).astype(np.float32) for s in (1, 2)]
    values = [torch.as_tensor(v).cuda() for v in host_values]
    outputs = [torch.empty(segments, device="cuda") for _ in range(2)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for _ in range(4):
        for stream, v, out in zip(streams, values, outputs):
            with torch.cuda.stream(stream):
                launch_gpu(v, device_offsets, out, "sum")
    torch.cuda.synchronize()
    assert len(runner._device_plan_cache) == 2
    for v, out in zip(host_values, outputs):
        exact = oracle.segsum_f64(v, offsets)
        bound = oracle.sum_tolerance(v, offsets)
        assert np.all(np.abs(out.cpu().numpy() - exact) <= bound)
    runner.clear_plan_cache()


def softmax_check(values, offsets, plan):
    device_values = torch.as_tensor(values).cuda()
    output = torch.full((values.size,), float("nan"), device="cuda")
    launch_softmax_gpu(device_values, torch.as_tensor(offsets).cuda(), output,
                       plan=plan)
    torch.cuda.synchronize()
    result = output.cpu().numpy().astype(np.float64)
    exact = oracle.segsoftmax_f64(values, offsets)
    inside = ~np.isnan(exact)
    assert np.isnan(result[~inside]).all()
    covered = slice(0, int(offsets[-1]))
    error = np.abs(result[covered] - exact[covered])
    assert np.all(error <= 4e-6 * exact[covered] + 1e-10)


def test_device_planned_softmax():
    offsets = workloads.c4_offsets(segments=4096)
    values = (2 * np.random.default_rng(4).standard_normal(
        int(offsets[-1]))).astype(np.float32)
    host = plan_segments(torch.as_tensor(offsets), op="softmax")
    device = device_plan(offsets, op="softmax")
    try:
        assert (host.describe()["softmax_buckets"] ==
                device.describe()["softmax_buckets"])
        softmax_check(values, offsets, device)
        device.check()
    finally:
        host.close()
        device.close()
    small = offsets_from_lengths([0, 1, 64, 65, 0, 513, 2049, 9000, 0, 30000])
    values = np.random.default_rng(2).standard_normal(
        int(small[-1])).astype(np.float32)
    plan = device_plan(small, op="softmax")
    try:
        softmax_check(values, small, plan)
    finally:
        plan.close()


def test_dump_plan_variable(monkeypatch, capfd):
    """SWAGE_DUMP_PLAN: every new plan is described on stderr."""
    monkeypatch.setenv("SWAGE_DUMP_PLAN", "1")
    offsets = offsets_from_lengths([5, 0, 4000, 17])
    for plan in (device_plan(offsets),
                 plan_segments(torch.as_tensor(offsets))):
        plan.close()
    lines = [line for line in capfd.readouterr().err.splitlines()
             if line.startswith("swage plan: ")]
    assert len(lines) == 2
    for line in lines:
        described = json.loads(line[len("swage plan: "):])
        assert described["segments"] == 4 and described["values"] == 4022
