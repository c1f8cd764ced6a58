"""Segment kernels written against the kernel language and launched through
the public ``kernel.launch`` surface (the reference's README sketch)."""

import numpy as np
import pytest
import torch

import oracle
import swage_b200 as sw
import swage_b200.language as sl
import workloads

pytestmark = pytest.mark.gpu


@sw.jit
def segmented_sum(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    segment = sl.segment(values_ptr, offsets_ptr, sid)
    x = sl.load_segment(segment)
    sl.store(output_ptr + sid, sl.sum(x))


@sw.jit
def segmented_max(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    sl.store(output_ptr + sid, sl.max(x))


@sw.jit
def segmented_min(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    sl.store(output_ptr + sid, sl.min(x))


@sw.jit
def segmented_softmax(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    segment = sl.segment(values_ptr, offsets_ptr, sid)

    x = sl.load_segment(segment)
    maximum = sl.max(x)
    numerator = sl.exp(x - maximum)
    denominator = sl.sum(numerator)

    sl.store_segment(output_ptr, segment, numerator / denominator)


def inputs():
    offsets = workloads.c5_offsets(segments=1 << 13, total=1 << 20, giants=2,
                                   giant_length=1 << 18)
    values = workloads.normal_values(int(offsets[-1]), "cuda", 21)
    return offsets, values, torch.as_tensor(offsets).cuda()


def test_sum_and_max_through_kernel_launch():
    offsets, values, device_offsets = inputs()
    segments = len(offsets) - 1
    host = values.cpu().numpy()
    for kernel, kind in ((segmented_sum, "sum"), (segmented_max, "max")):
        output = torch.full((segments,), float("nan"), device="cuda")
        result = kernel.launch(
            arguments={"values_ptr": values, "offsets_ptr": device_offsets,
                       "output_ptr": output},
            constexprs={}, grid=(segments,))
        assert result is None
        torch.cuda.synchronize()
        got = output.cpu().numpy()
        if kind == "max":
            expected = oracle.segreduce_f32(host, offsets, "max")
            assert np.array_equal(got.view(np.uint32),
                                  expected.view(np.uint32))
        else:
            error = np.abs(got - oracle.segsum_f64(host, offsets))
            assert np.all(error <= oracle.sum_tolerance(host, offsets))


def test_min_kind_every_schedule():
    """kind<min> (an extension: the reference's lowering rejects it): bit-exact
    against the oracle's mirror image of max, through kernel.launch and
    through every schedule of launch_gpu; the plain launch_gpu call keeps the
    reference's error."""
    from swage_b200._segmented_qualification import launch_gpu, plan_segments

    offsets, values, device_offsets = inputs()
    segments = len(offsets) - 1
    host = values.cpu().numpy().copy()
    host[12345] = np.nan
    values = torch.as_tensor(host).cuda()
    expected = oracle.segreduce_f32(host, offsets, "min")
    output = torch.full((segments,), float("nan"), device="cuda")
    segmented_min.launch(
        arguments={"values_ptr": values, "offsets_ptr": device_offsets,
                   "output_ptr": output},
        constexprs={}, grid=(segments,))
    torch.cuda.synchronize()
    got = output.cpu().numpy()
    both_nan = np.isnan(got) & np.isnan(expected)
    assert np.all(both_nan | (got.view(np.uint32) == expected.view(np.uint32)))
    assert np.isnan(expected).sum() == 1
    plans = (plan_segments(torch.as_tensor(offsets)),
             plan_segments(device_offsets, int(offsets[-1])))
    for plan in plans:
        for schedule in ("warp", "cta", "split", "persistent", "resident"):
            output.fill_(float("nan"))
            launch_gpu(values, device_offsets, output, "min", plan=plan,
                       schedule=schedule, extensions=True)
            torch.cuda.synchronize()
            got = output.cpu().numpy()
            both_nan = np.isnan(got) & np.isnan(expected)
            assert np.all(both_nan | (got.view(np.uint32) ==
                                      expected.view(np.uint32))), schedule
        plan.close()
    empty = torch.full((3,), float("nan"), device="cuda")
    launch_gpu(values, torch.zeros(4, dtype=torch.int32, device="cuda"),
               empty, "min", extensions=True)
    torch.cuda.synchronize()
    assert torch.isinf(empty).all() and (empty > 0).all()
    with pytest.raises(ValueError, match="must be 'sum' or 'max'"):
        launch_gpu(values, device_offsets, output, "min")


def test_softmax_through_kernel_launch():
    offsets = workloads.c4_offsets(segments=2048)
    values = workloads.normal_values(int(offsets[-1]), "cuda", 22, scale=2.0)
    output = torch.empty_like(values)
    segmented_softmax.launch(
        arguments={"values_ptr": values,
                   "offsets_ptr": torch.as_tensor(offsets).cuda(),
                   "output_ptr": output},
        constexprs={}, grid=(len(offsets) - 1,))
    torch.cuda.synchronize()
    exact = oracle.segsoftmax_f64(values.cpu().numpy(), offsets)
    assert np.allclose(output.cpu().numpy(), exact, rtol=4e-6, atol=1e-10)


def test_launch_validation_for_segment_kernels():
    offsets, values, device_offsets = inputs()
    segments = len(offsets) - 1
    output = torch.empty(segments, device="cuda")
    good = {"values_ptr": values, "offsets_ptr": device_offsets,
            "output_ptr": output}
    with pytest.raises(ValueError, match="grid must equal"):
        segmented_sum.launch(arguments=good, constexprs={},
                             grid=(segments + 1,))
    with pytest.raises(ValueError, match="take no constexprs"):
        segmented_sum.launch(arguments=good, constexprs={"BLOCK": 128},
                             grid=(segments,))
    with pytest.raises(ValueError, match="exactly the kernel's three"):
        segmented_sum.launch(arguments={"values_ptr": values}, constexprs={},
                             grid=(segments,))
    with pytest.raises(TypeError, match="offsets must have dtype"):
        segmented_sum.launch(
            arguments={**good, "offsets_ptr": device_offsets.long()},
            constexprs={}, grid=(segments,))
    with pytest.raises(ValueError, match="output has"):
        segmented_sum.launch(
            arguments={**good, "output_ptr": output[: segments - 1]},
            constexprs={}, grid=(segments,))

    @sw.jit
    def not_a_segment_kernel(values_ptr, offsets_ptr, output_ptr):
        sid = sl.segment_id(0)
        x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
        sl.store(output_ptr + sid, sl.exp(x))

    with pytest.raises(sw.CompilationError, match="not one of the supported"):
        not_a_segment_kernel.launch(arguments=good, constexprs={},
                                    grid=(segments,))
