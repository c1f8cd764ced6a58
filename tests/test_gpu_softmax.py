"""Segmented softmax on the GPU against the fp64 oracle."""

import numpy as np
import pytest
import torch

import oracle
import workloads
from gpu_util import launch_softmax_gpu, offsets_from_lengths

pytestmark = pytest.mark.gpu

SCHEDULES = ["auto", "warp", "cta", "split"]


def check_softmax(values, offsets, schedule, poison=True):
    """|err| <= 1e-5 * sqrt(len) * max|x| per element against fp64, and a
    much tighter relative bound where the probability is not tiny."""
    values = np.asarray(values, dtype=np.float32)
    offsets = np.asarray(offsets, dtype=np.int32)
    device_values = torch.as_tensor(values).cuda()
    output = torch.full((values.size,), float("nan"), device="cuda")
    launch_softmax_gpu(device_values, torch.as_tensor(offsets).cuda(), output,
                       schedule=schedule)
    torch.cuda.synchronize()
    result = output.cpu().numpy().astype(np.float64)
    exact = oracle.segsoftmax_f64(values, offsets)
    inside = ~np.isnan(exact)
    assert np.isnan(result[~inside]).all(), "wrote outside every segment"
    lengths = np.diff(offsets)
    per_segment = 1e-5 * np.sqrt(lengths) * oracle.segabsmax_f64(values,
                                                                 offsets)
    bound = np.repeat(per_segment, lengths)
    covered = slice(0, int(offsets[-1]))
    error = np.abs(result[covered] - exact[covered])
    assert np.all(error <= bound + 1e-12)
    assert np.all(error <= 4e-6 * exact[covered] + 1e-10)
    return result


@pytest.mark.parametrize("schedule", SCHEDULES)
def test_small_cases(schedule):
    rng = np.random.default_rng(4)
    for lengths in ([1], [0], [0, 2, 0, 0, 3], [33, 33, 33, 33],
                    [1, 257, 2, 3837], [4097], [129, 0, 128, 127, 1],
                    [511, 512, 513], [2047, 2048, 2049], [8191, 8192, 8193],
                    [16384, 3, 20000], [8192, 8193, 8200, 65535, 65536, 65537],
                    [9001, 30011, 12345], [63, 64, 65, 1, 8, 9, 7, 0, 64],
                    [16383, 16384, 16385, 28671, 28672, 28673, 57343, 57344,
                     57345]):
        offsets = offsets_from_lengths(lengths)
        values = (2 * rng.standard_normal(offsets[-1] + 2)).astype(np.float32)
        result = check_softmax(values, offsets, schedule)
        for a, b in zip(offsets[:-1], offsets[1:]):
            if b > a:
                assert abs(result[a:b].sum() - 1) < 1e-5


@pytest.mark.parametrize("schedule", SCHEDULES)
def test_large_magnitudes_do_not_overflow(schedule):
    values = np.array([1000.0, 999.0, -1000.0, 88.0, 89.0, -5000.0, -5001.0],
                      dtype=np.float32)
    check_softmax(values, np.array([0, 3, 5, 7], dtype=np.int32), schedule)


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("shift", [0, 1, 3])
def test_misaligned_pointers(schedule, shift):
    rng = np.random.default_rng(8)
    lengths = list(rng.integers(0, 400, size=100)) + [70000, 2, 5000]
    offsets = offsets_from_lengths(lengths)
    host = (2 * rng.standard_normal(offsets[-1] + 8)).astype(np.float32)
    base = torch.as_tensor(host).cuda()
    values = base[shift:shift + int(offsets[-1])]
    out_base = torch.full((int(offsets[-1]) + 8,), float("nan"),
                          device="cuda")
    output = out_base[(shift * 2) % 4:(shift * 2) % 4 + int(offsets[-1])]
    launch_softmax_gpu(values, torch.as_tensor(offsets).cuda(), output,
                       schedule=schedule)
    torch.cuda.synchronize()
    exact = oracle.segsoftmax_f64(host[shift:shift + int(offsets[-1])],
                                  offsets)
    assert np.allclose(output.cpu().numpy(), exact, rtol=4e-6, atol=1e-10)


@pytest.mark.parametrize("schedule", SCHEDULES)
def test_nan_and_empty_semantics(schedule):
    values = torch.tensor([1.0, float("nan"), 3.0, 4.0, 5.0], device="cuda")
    offsets = torch.tensor([0, 3, 3, 5], dtype=torch.int32, device="cuda")
    output = torch.zeros(5, device="cuda")
    launch_softmax_gpu(values, offsets, output, schedule=schedule)
    torch.cuda.synchronize()
    host = output.cpu().numpy()
    assert np.isnan(host[:3]).all()
    assert np.allclose(host[3:], [1 / (1 + np.e), np.e / (1 + np.e)],
                       rtol=1e-6)


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("length", [5, 700, 1024, 1025, 5000, 30001, 70000])
def test_infinities_follow_the_oracle(schedule, length):
    """-inf entries get probability 0; a NaN or +inf poisons its segment."""
    rng = np.random.default_rng(length)
    base = (2 * rng.standard_normal(length)).astype(np.float32)
    cases = []
    minus = base.copy()
    minus[rng.choice(length, size=max(1, length // 3), replace=False)] = -np.inf
    cases.append(minus)
    front = base.copy()
    front[: length - 1] = -np.inf          # one finite value at the very end
    cases.append(front)
    nan = base.copy()
    nan[length // 2] = np.nan
    cases.append(nan)
    plus = base.copy()
    plus[length // 3] = np.inf
    cases.append(plus)
    cases.append(np.full(length, -np.inf, dtype=np.float32))
    values = np.concatenate(cases)
    offsets = (np.arange(len(cases) + 1) * length).astype(np.int32)
    output = torch.full((values.size,), 7.0, device="cuda")
    launch_softmax_gpu(torch.as_tensor(values).cuda(),
                       torch.as_tensor(offsets).cuda(), output,
                       schedule=schedule)
    torch.cuda.synchronize()
    got = output.cpu().numpy().astype(np.float64)
    with np.errstate(invalid="ignore"):
        exact = oracle.segsoftmax_f64(values, offsets)
    assert np.array_equal(np.isnan(got), np.isnan(exact))
    finite = ~np.isnan(exact)
    assert np.allclose(got[finite], exact[finite], rtol=4e-6, atol=1e-10)


def test_rejects_aliasing_and_short_output():
    values = torch.randn(8, device="cuda")
    offsets = torch.tensor([0, 8], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="must not alias"):
        launch_softmax_gpu(values, offsets, values)
    with pytest.raises(ValueError, match="output has 4 elements"):
        launch_softmax_gpu(values, offsets, torch.empty(4, device="cuda"))


@pytest.mark.parametrize("schedule", SCHEDULES)
def test_config_softmax_reduced(schedule):
    """The softmax configuration's length mix at 1/64 of its segment count."""
    offsets = workloads.c4_offsets(segments=4096)
    values = workloads.normal_values(int(offsets[-1]), "cuda",
                                     workloads.SEEDS["c4"], scale=2.0)
    check_softmax(values.cpu().numpy(), offsets, schedule)


def test_softmax_is_reproducible_run_to_run():
    """The same launch repeated gives the same bits.  (A stage of the ring
    kernel handed back to the copy engine before every lane had its values
    showed up as one 128-value row differing in about every second run.)"""
    offsets = workloads.c4_offsets(segments=4096)
    values = workloads.normal_values(int(offsets[-1]), "cuda",
                                     workloads.SEEDS["c4"], scale=2.0)
    device_offsets = torch.as_tensor(offsets).cuda()
    first = None
    for _ in range(6):
        output = torch.full((values.numel(),), float("nan"), device="cuda")
        launch_softmax_gpu(values, device_offsets, output)
        torch.cuda.synchronize()
        if first is None:
            first = output
        else:
            assert torch.equal(first, output)


def test_full_size_softmax_every_segment():
    """262144 segments, about 1.13e9 values, planned on the GPU from the
    device-resident offsets (what a launch of this size does by itself and
    what the benchmark times): EVERY segment is compared with the fp64
    oracle, in slices of whole segments; besides, every segment sums to one
    and the output is a valid probability everywhere."""
    offsets = workloads.c4_offsets()
    count = int(offsets[-1])
    values = workloads.normal_values(count, "cuda", workloads.SEEDS["c4"],
                                     scale=2.0)
    device_offsets = torch.as_tensor(offsets).cuda()
    output = torch.full((count,), float("nan"), device="cuda")
    launch_softmax_gpu(values, device_offsets, output)
    torch.cuda.synchronize()
    assert bool(((output >= 0) & (output <= 1)).all())
    lengths = torch.as_tensor(np.diff(offsets).astype(np.int64)).cuda()
    sums = torch.segment_reduce(output.double(), "sum", lengths=lengths)
    assert float((sums - 1).abs().max()) < 1e-4
    del sums
    host_values = values.cpu().numpy()
    host_output = output.cpu().numpy()
    segments = len(offsets) - 1
    threads = oracle.max_threads()
    worst_relative = 0.0
    longest_checked = 0
    first = 0
    while first < segments:
        # a slice of whole segments holding about 2**26 values
        last = int(np.searchsorted(offsets, int(offsets[first]) + (1 << 26),
                                   side="right")) - 1
        last = min(segments, max(last, first + 1))
        a, b = int(offsets[first]), int(offsets[last])
        local = (offsets[first:last + 1] - a).astype(np.int32)
        exact = oracle.segsoftmax_f64(host_values[a:b], local,
                                      threads=threads)
        got = host_output[a:b].astype(np.float64)
        error = np.abs(got - exact)
        # the stated bound, per segment: 1e-5 * sqrt(len) * max|x|
        bound = np.repeat(oracle.sum_tolerance(host_values[a:b], local),
                          np.diff(local))
        assert np.all(error <= bound)
        # and the tighter one this library holds itself to
        close = error <= 1e-10 + 4e-6 * np.abs(exact)
        assert np.all(close), (
            f"segment slice {first}..{last}: "
            f"{int((~close).sum())} values off, worst relative "
            f"{float(np.max(error / np.maximum(exact, 1e-300)))}")
        visible = exact > 1e-30
        worst_relative = max(worst_relative,
                             float(np.max(error[visible] / exact[visible])))
        longest_checked = max(longest_checked, int(np.diff(local).max()))
        first = last
    print(f"worst relative error {worst_relative:.3g}; longest segment "
          f"checked {longest_checked}")
    # every length class ran, the one that re-reads its head included
    assert longest_checked > 57344
