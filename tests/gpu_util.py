"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

import oracle
from swage_b200._segmented_qualification import (
    launch_gpu,
    launch_softmax_gpu,
    plan_segments,
)


def offsets_from_lengths(lengths):
    return np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)


def fixture_values(count):
    index = np.arange(count)
    return (((index % 17) - 8) / 4).astype(np.float32)


def bits_equal_or_both_nan(actual, expected):
    actual = np.asarray(actual, dtype=np.float32)
    expected = np.asarray(expected, dtype=np.float32)
    both_nan = np.isnan(actual) & np.isnan(expected)
    return bool(np.all(both_nan |
                       (actual.view(np.uint32) == expected.view(np.uint32))))


def run_reduce(values, offsets, kind, schedule="auto", plan=None, extra=3,
               block_size=128):
    """Launch on the GPU; return the first S outputs and the untouched tail."""
    device_values = torch.as_tensor(
        np.asarray(values, dtype=np.float32)).cuda()
    device_offsets = torch.as_tensor(
        np.asarray(offsets, dtype=np.int32)).cuda()
    segments = len(offsets) - 1
    output = torch.full((segments + extra,), float("nan"), device="cuda")
    launch_gpu(device_values, device_offsets, output, kind, block_size,
               plan=plan, schedule=schedule)
    torch.cuda.synchronize()
    host = output.cpu().numpy()
    return host[:segments], host[segments:]


def check_reduce(values, offsets, kind, schedule, plan=None):
    """Bit-exact for max; within 1e-5*sqrt(len)*max|x| of fp64 for sum."""
    values = np.asarray(values, dtype=np.float32)
    offsets = np.asarray(offsets, dtype=np.int32)
    result, tail = run_reduce(values, offsets, kind, schedule, plan)
    assert np.isnan(tail).all(), "wrote past the last segment"
    if kind == "max":
        expected = oracle.segreduce_f32(values, offsets, "max",
                                        threads=oracle.max_threads())
        assert bits_equal_or_both_nan(result, expected)
    else:
        exact = oracle.segsum_f64(values, offsets)
        bound = oracle.sum_tolerance(values, offsets)
        error = np.abs(result.astype(np.float64) - exact)
        worst = int(np.argmax(error - bound))
        assert np.all(error <= bound), (
            f"segment {worst}: |err| {error[worst]} > bound {bound[worst]}")
        empty = np.diff(offsets) == 0
        assert np.all(result[empty].view(np.uint32) == 0), "empty sum != +0.0"
    return result


def make_plan(offsets, op="reduce"):
    return plan_segments(torch.as_tensor(np.asarray(offsets, dtype=np.int32)),
                         op=op)


__all__ = [
    "bits_equal_or_both_nan", "check_reduce", "fixture_values",
    "launch_softmax_gpu", "make_plan", "offsets_from_lengths", "run_reduce",
]
