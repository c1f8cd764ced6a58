"""Element maps fused into a segmented reduction.

``out[s] = reduce(fn(scale * x + shift) for x in segment s)`` in one pass: the
dialect's ``swage.map`` region in front of a ``swage.reduce``
(``test/Dialect/Swage/roundtrip.mlir:43-52``; the composition of
``test/Dialect/Swage/softmax.mlir:17-24``).  The reference's lowering accepts
the identity region only
(``lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:106-119``), so no
reference result exists; the checker is the CPU oracle: ``oracle.map_f32``
applies the map element by element in fp32 (product and sum rounded
separately) and the pinned sequential / fp64 reductions reduce what it gives.

* identity / abs / square: every mapped element is exact, so max / min must be
  bit-exact against the oracle, and sum within ``1e-5 * sqrt(len) * max|m| +
  1e-6 * sum|m|`` of the fp64 sum of the mapped elements ``m``.  The first
  term is the f32 rule; the second is there because mapped elements are
  often all of one sign (squares, magnitudes, exponentials): their sum grows
  like ``len`` while the first term grows like ``sqrt(len)``, and fp32
  rounding of the running total alone is ``6e-8 * sum`` per level of the
  combine tree;
* exp: the kernels use one multiply and ``ex2.approx`` (as the softmax does):
  max / min within ``4e-6`` relative, sum within the bound above plus
  ``4e-6 * sum|m|``.
"""

import numpy as np
import pytest
import torch

import oracle
import swage_b200 as sw
import workloads
from gpu_util import bits_equal_or_both_nan, offsets_from_lengths
from swage_b200 import language as sl
from swage_b200._segmented_qualification import (
    ElementMap,
    launch_gpu,
    plan_segments,
)

pytestmark = pytest.mark.gpu

SCHEDULES = ["auto", "warp", "cta", "split", "persistent", "resident"]
MAPS = [
    ElementMap("identity", 1.0, -0.0),
    ElementMap("identity", -2.5, 0.75),
    ElementMap("abs", 1.0, -0.0),
    ElementMap("abs", 0.5, -1.0),
    ElementMap("square", 1.0, -0.0),
    ElementMap("square", 3.0, 0.125),
    ElementMap("exp", 1.0, -0.0),
    ElementMap("exp", -0.5, 1.0),
]
EXP_RELATIVE = 4e-6
SUM_RELATIVE = 1e-6
GRID = [0, 1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 32, 33, 127, 128, 129, 255,
        256, 257, 1023, 1024, 1025, 2047, 2048, 2049, 4095, 4096, 4097, 8193,
        40000]
IDENTITY = {"sum": 0.0, "max": -np.inf, "min": np.inf}


def run(values, offsets, kind, element_map, schedule, plan=None, extra=3):
    device_offsets = torch.as_tensor(np.asarray(offsets, np.int32)).cuda()
    segments = len(offsets) - 1
    output = torch.full((segments + extra,), float("nan"), device="cuda")
    launch_gpu(values, device_offsets, output, kind, schedule=schedule,
               plan=plan, extensions=True, map=element_map)
    torch.cuda.synchronize()
    host = output.cpu().numpy()
    assert np.isnan(host[segments:]).all(), "wrote past the last segment"
    return host[:segments]


def sum_bound(mapped, offsets, exp):
    total = oracle.segsum_f64(np.abs(mapped), offsets)
    relative = SUM_RELATIVE + (EXP_RELATIVE if exp else 0.0)
    return oracle.sum_tolerance(mapped, offsets) + relative * total


def check(values, offsets, kind, element_map, schedule, plan=None):
    """``values``: a CUDA tensor of any floating element type."""
    offsets = np.asarray(offsets, np.int32)
    result = run(values, offsets, kind, element_map, schedule, plan)
    wide = values.float().cpu().numpy()  # exact widening
    mapped = wide if element_map is None else oracle.map_f32(
        wide, *element_map)
    empty = np.diff(offsets) == 0
    assert bits_equal_or_both_nan(
        result[empty], np.full(int(empty.sum()), IDENTITY[kind], np.float32))
    exp = element_map is not None and element_map.fn == "exp"
    if kind == "sum":
        exact = oracle.segsum_f64(mapped, offsets)
        bound = sum_bound(mapped, offsets, exp)
        finite = np.isfinite(exact)
        error = np.abs(result.astype(np.float64) - exact)
        assert np.all(error[finite] <= bound[finite])
        assert np.all(np.isnan(result[~finite]) == np.isnan(exact[~finite]))
    else:
        expected = oracle.segreduce_f32(mapped, offsets, kind)
        if exp:
            both_nan = np.isnan(result) & np.isnan(expected)
            close = np.abs(result - expected) <= EXP_RELATIVE * np.abs(expected)
            assert np.all(both_nan | close | (result == expected))
        else:
            assert bits_equal_or_both_nan(result, expected)


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("kind", ["sum", "max", "min"])
@pytest.mark.parametrize("element_map", MAPS, ids=lambda m: "%s_%g_%g" % m)
def test_mapped_boundary_lengths(element_map, kind, schedule):
    rng = np.random.default_rng(51)
    for order in (GRID, list(rng.permutation(GRID))):
        offsets = offsets_from_lengths(order)
        values = torch.as_tensor(
            (2.0 * rng.standard_normal(offsets[-1])).astype(np.float32)).cuda()
        check(values, offsets, kind, element_map, schedule)


@pytest.mark.parametrize("schedule", ["warp", "split", "resident"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("element_map", MAPS[1::2], ids=lambda m: "%s_%g_%g" % m)
def test_mapped_half_precision_inputs(element_map, dtype, schedule):
    rng = np.random.default_rng(53)
    offsets = offsets_from_lengths(list(rng.permutation(GRID)))
    values = torch.as_tensor(
        rng.standard_normal(offsets[-1]).astype(np.float32)).cuda().to(dtype)
    for kind in ("sum", "max"):
        check(values, offsets, kind, element_map, schedule)


@pytest.mark.parametrize("schedule", ["warp", "split", "resident"])
def test_special_values_go_through_the_map(schedule):
    """NaN, infinities and signed zeros: |NaN| is NaN and wins every max,
    (-inf)^2 = +inf, exp(-inf) = 0; the identity map with the default shift of
    -0.0 leaves -0.0 as it is (max(-0, -0) = -0 bit for bit)."""
    lengths = [5, 0, 3, 700, 4, 2500, 2]
    offsets = offsets_from_lengths(lengths)
    host = np.linspace(-3, 3, offsets[-1]).astype(np.float32)
    host[1] = np.nan
    host[5:8] = -0.0
    host[20] = -np.inf
    host[8 + 700 + 1] = np.inf
    host[-2:] = -0.0
    values = torch.as_tensor(host).cuda()
    for element_map in MAPS:
        for kind in ("sum", "max", "min"):
            check(values, offsets, kind, element_map, schedule)
    got = run(values, offsets, "max", ElementMap(), schedule)
    assert got[2].view(np.uint32) == np.float32(-0.0).view(np.uint32)
    assert got[6].view(np.uint32) == np.float32(-0.0).view(np.uint32)


@pytest.mark.parametrize("shift", [1, 2, 3])
def test_mapped_values_at_every_phase_of_a_16_byte_line(shift):
    rng = np.random.default_rng(shift + 60)
    lengths = list(rng.integers(0, 300, size=150)) + [9000, 3, 20000, 0, 5]
    offsets = offsets_from_lengths(lengths)
    base = torch.as_tensor(rng.standard_normal(
        offsets[-1] + shift + 5).astype(np.float32)).cuda()
    values = base[shift:shift + int(offsets[-1]) + 2]
    assert values.data_ptr() % 16 == 4 * shift
    for schedule in ("split", "resident", "warp"):
        check(values, offsets, "sum", ElementMap("square", 0.5, 0.25), schedule)
        check(values, offsets, "max", ElementMap("abs", -1.0, 0.5), schedule)


def test_extreme_skew_shape_through_the_device_planner():
    """Sum of squares and max of |x| on the extreme-skew shape at 1/64 of its
    size, planned on the GPU (what a large launch does by itself), and the
    same plan reused for an unmapped launch."""
    offsets = workloads.c5_offsets(segments=1 << 16, total=1 << 24, giants=4,
                                   giant_length=1 << 21)
    count = int(offsets[-1])
    values = workloads.normal_values(count, "cuda", 7)
    check(values, offsets, "sum", ElementMap("square"), "auto")
    check(values, offsets, "max", ElementMap("abs"), "auto")
    check(values, offsets, "sum", ElementMap("exp", 0.25, -1.0), "auto")
    device_offsets = torch.as_tensor(offsets).cuda()
    plan = plan_segments(device_offsets, count)
    try:
        for schedule in ("split", "resident"):
            check(values, offsets, "sum", ElementMap("abs", 2.0, 0.5),
                  schedule, plan)
            check(values, offsets, "sum", None, schedule, plan)
        plan.check()
    finally:
        plan.close()


def test_log_sum_exp_composed_from_two_launches():
    """max, then the sum of exp(x - m) with m a captured scalar: the two
    reductions of a log-sum-exp with one global shift."""
    offsets = workloads.c3_offsets(segments=1 << 12)
    count = int(offsets[-1])
    values = workloads.normal_values(count, "cuda", 11, scale=3.0)
    top = float(values.max())
    got = run(values, offsets, "sum", ElementMap("exp", 1.0, -top), "auto")
    host = values.cpu().numpy().astype(np.float64)
    exact = np.array([np.exp(host[a:b] - np.float64(np.float32(top))).sum()
                      for a, b in zip(offsets[:-1], offsets[1:])])
    assert np.all(np.abs(got - exact) <= 1e-5 * np.maximum(exact, 1e-30))


@sw.jit
def sum_of_squares(values_ptr, offsets_ptr, output_ptr, SCALE: sl.constexpr):
    sid = sl.segment_id(0)
    seg = sl.segment(values_ptr, offsets_ptr, sid)
    x = sl.load_segment(seg)
    y = x * SCALE - 1.5
    sl.store(output_ptr + sid, sl.sum(y * y))


@sw.jit
def max_magnitude(values_ptr, offsets_ptr, output_ptr):
    sid = sl.segment_id(0)
    seg = sl.segment(values_ptr, offsets_ptr, sid)
    x = sl.load_segment(seg)
    sl.store(output_ptr + sid, sl.max(sl.abs(x)))


@sw.jit
def sum_of_exponentials(values_ptr, offsets_ptr, output_ptr,
                        SHIFT: sl.constexpr):
    sid = sl.segment_id(0)
    seg = sl.segment(values_ptr, offsets_ptr, sid)
    x = sl.load_segment(seg)
    sl.store(output_ptr + sid, sl.sum(sl.exp(0.5 * x + SHIFT)))


def test_mapped_kernels_through_kernel_launch():
    offsets = workloads.c1_offsets(segments=512)
    count = int(offsets[-1])
    segments = len(offsets) - 1
    values = workloads.normal_values(count, "cuda", 13)
    device_offsets = torch.as_tensor(offsets).cuda()
    host = values.cpu().numpy()
    cases = (
        (sum_of_squares, {"SCALE": 3}, "sum", ("square", 3.0, -1.5)),
        (sum_of_squares, {"SCALE": 0.25}, "sum", ("square", 0.25, -1.5)),
        (max_magnitude, {}, "max", ("abs", 1.0, -0.0)),
        (sum_of_exponentials, {"SHIFT": -2.0}, "sum", ("exp", 0.5, -2.0)),
    )
    for kernel, constexprs, kind, spec in cases:
        output = torch.full((segments,), float("nan"), device="cuda")
        kernel.launch(
            arguments={"values_ptr": values, "offsets_ptr": device_offsets,
                       "output_ptr": output},
            constexprs=constexprs, grid=(segments,))
        torch.cuda.synchronize()
        got = output.cpu().numpy()
        mapped = oracle.map_f32(host, *spec)
        if kind == "max":
            assert bits_equal_or_both_nan(
                got, oracle.segreduce_f32(mapped, offsets, "max"))
        else:
            bound = sum_bound(mapped, offsets, spec[0] == "exp")
            error = np.abs(got - oracle.segsum_f64(mapped, offsets))
            assert np.all(error <= bound)
    output = torch.zeros(segments, device="cuda")
    arguments = {"values_ptr": values, "offsets_ptr": device_offsets,
                 "output_ptr": output}
    with pytest.raises(ValueError, match="exactly the kernel's constexpr"):
        sum_of_squares.launch(arguments=arguments, constexprs={},
                              grid=(segments,))
    with pytest.raises(TypeError, match="must be an int or a float"):
        sum_of_squares.launch(arguments=arguments, constexprs={"SCALE": "2"},
                              grid=(segments,))
    with pytest.raises(ValueError, match="take no constexprs"):
        max_magnitude.launch(arguments=arguments, constexprs={"SCALE": 2},
                             grid=(segments,))


def test_maps_are_an_extension_and_floating_only():
    offsets = torch.tensor([0, 4, 8], dtype=torch.int32, device="cuda")
    values = torch.ones(8, device="cuda")
    out = torch.zeros(2, device="cuda")
    with pytest.raises(ValueError, match="needs extensions=True"):
        launch_gpu(values, offsets, out, "sum", map=ElementMap("abs"))
    with pytest.raises(TypeError, match="must be an ElementMap"):
        launch_gpu(values, offsets, out, "sum", extensions=True,
                   map=("abs", 1.0, 0.0))
    with pytest.raises(ValueError, match="map function must be"):
        launch_gpu(values, offsets, out, "sum", extensions=True,
                   map=ElementMap("sqrt"))
    with pytest.raises(TypeError, match="integer segments are not mapped"):
        launch_gpu(values.to(torch.int32), offsets,
                   torch.zeros(2, dtype=torch.int32, device="cuda"), "sum",
                   extensions=True, map=ElementMap("abs"))
