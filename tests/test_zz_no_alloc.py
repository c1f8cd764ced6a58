"""The allocation-free reduce entry point against the planned one.

Some callers cannot allocate device memory when they call this library: their
framework's memory pool already owns the GPU, or the implicit synchronisation
of ``cudaMalloc`` is not acceptable in their serving loop.  For them
``swg_segreduce_f32_noalloc`` runs the split schedule out of a fixed array in
the library image.  This file checks, through the C ABI, that it gives the
same bits as ``swg_segreduce_f32`` with a plan and the split schedule (both run
the same tile tasks with the same combine tree), on two calls in a row --
the second call sees the first call's leftovers in the shared array -- and
that both agree with the CPU oracle (max bit for bit, sum within
``1e-5 * sqrt(len) * max|x|`` of the fp64 sum).

Collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import numpy as np
import pytest
import torch

import oracle
import workloads
from swage_b200 import _native

pytestmark = pytest.mark.gpu


def planned(kind, values, offsets, segments):
    plan = _native.plan_create(offsets.ctypes.data, segments, values.numel(),
                               _native.OP_REDUCE)
    device_offsets = torch.from_numpy(offsets).cuda()
    out = torch.full((segments,), float("nan"), device="cuda")
    _native.segreduce(kind, values.data_ptr(), device_offsets.data_ptr(),
                      out.data_ptr(), values.numel(), segments, plan,
                      _native.SCHED_SPLIT, 0,
                      torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    _native.plan_destroy(plan)
    return out


def no_alloc(kind, values, offsets, segments):
    out = torch.full((segments,), float("nan"), device="cuda")
    _native.segreduce_noalloc(kind, values.data_ptr(), offsets.ctypes.data,
                              out.data_ptr(), values.numel(), segments,
                              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out


def same_bits(a, b):
    return torch.equal(a.view(torch.int32), b.view(torch.int32))


def agrees_with_oracle(kind, result, values, offsets):
    host_values = values.cpu().numpy()
    result = result.cpu().numpy()
    if kind == _native.KIND_MAX:
        expected = oracle.segreduce_f32(host_values, offsets, "max")
        return np.array_equal(result.view(np.uint32),
                              expected.view(np.uint32))
    exact = oracle.segsum_f64(host_values, offsets)
    bound = oracle.sum_tolerance(host_values, offsets)
    return bool(np.all(np.abs(result - exact) <= bound))


def test_two_calls_in_a_row_match_the_planned_entry_point():
    # first a skewed input with split segments, then a different, smaller one
    # that leaves most of the previous call's data behind in the shared array
    skewed = workloads.c5_offsets(segments=1 << 16, total=1 << 23, giants=4,
                                  giant_length=1 << 20)
    canonical = workloads.c1_offsets(segments=3000)
    for kind in (_native.KIND_SUM, _native.KIND_MAX):
        for offsets in (skewed, canonical):
            segments = len(offsets) - 1
            values = workloads.normal_values(int(offsets[-1]) + 5, "cuda", 77)
            expected = planned(kind, values, offsets, segments)
            assert not torch.isnan(expected).any()
            first = no_alloc(kind, values, offsets, segments)
            second = no_alloc(kind, values, offsets, segments)
            assert same_bits(first, expected)
            assert same_bits(second, expected)
            assert agrees_with_oracle(kind, first, values, offsets)
            assert agrees_with_oracle(kind, second, values, offsets)


def test_sizes_beyond_the_fixed_array_are_rejected_clearly():
    segments = (1 << 18) + 1
    offsets = np.zeros(segments + 1, dtype=np.int32)
    values = torch.zeros(4, device="cuda")
    out = torch.zeros(segments, device="cuda")
    with pytest.raises(RuntimeError, match="exceed the fixed scratch"):
        _native.segreduce_noalloc(_native.KIND_SUM, values.data_ptr(),
                                  offsets.ctypes.data, out.data_ptr(), 4,
                                  segments, 0)
    # too many tile tasks: 40000 segments of 2049 values -> 40000 chunk tasks
    lengths = np.full(40000, 2049, dtype=np.int64)
    big = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    with pytest.raises(RuntimeError, match="tile tasks"):
        _native.segreduce_noalloc(_native.KIND_SUM, values.data_ptr(),
                                  big.ctypes.data, out.data_ptr(),
                                  int(big[-1]), 40000, 0)
    with pytest.raises(RuntimeError, match="SWG_ERR_INVALID_OFFSETS"):
        bad = np.array([0, 3, 2], dtype=np.int32)
        _native.segreduce_noalloc(_native.KIND_SUM, values.data_ptr(),
                                  bad.ctypes.data, out.data_ptr(), 4, 2, 0)
