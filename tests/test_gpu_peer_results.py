"""Result exchange of a sharded reduction by peer stores.

``swg_scatter_results_f32`` stores one rank's results into every rank's copy of
the full result array (plain stores; the copies of other ranks are mapped
through CUDA IPC).  No reference counterpart: the reference is single-GPU
(``python/swage/_runtime.py:146-151``).  The checker is the CPU oracle on the
whole, unsharded problem.
"""

import os
import pathlib
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from swage_b200 import _native

pytestmark = pytest.mark.gpu
WORKER = pathlib.Path(__file__).with_name("peer_results_worker.py")


@pytest.mark.parametrize("offset", [0, 1, 2, 3, 4, 1023])
@pytest.mark.parametrize("count", [0, 1, 2, 3, 4, 5, 7, 8, 9, 1000, 70001])
def test_scatter_places_every_element_in_every_destination(count, offset):
    """Same-process form: the destinations are buffers on this GPU.  Every
    alignment of the destination range (scalar head, 128-bit body, scalar
    tail), guard elements on both sides untouched, bit for bit."""
    rng = np.random.default_rng(count * 7 + offset)
    source = torch.as_tensor(
        rng.standard_normal(count + 3).astype(np.float32)).cuda()
    total = offset + count + 5
    destinations = [torch.full((total,), float("nan"), device="cuda")
                    for _ in range(3)]
    stream = torch.cuda.current_stream().cuda_stream
    _native.scatter_results(source.data_ptr(), count,
                            [d.data_ptr() for d in destinations], offset,
                            stream)
    torch.cuda.synchronize()
    expected = source[:count].cpu().numpy().view(np.uint32)
    for destination in destinations:
        host = destination.cpu().numpy()
        assert np.array_equal(host[offset:offset + count].view(np.uint32),
                              expected)
        assert np.isnan(host[:offset]).all()
        assert np.isnan(host[offset + count:]).all()


def test_scatter_rejects_bad_arguments():
    buffer = torch.zeros(64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    with pytest.raises(RuntimeError, match="not 16-byte aligned"):
        _native.scatter_results(buffer.data_ptr(), 4,
                                [buffer.data_ptr() + 4], 0, stream)
    with pytest.raises(RuntimeError, match="more than 16 destinations"):
        _native.scatter_results(buffer.data_ptr(), 4,
                                [buffer.data_ptr()] * 17, 0, stream)
    with pytest.raises(RuntimeError, match="negative count or offset"):
        _native.scatter_results(buffer.data_ptr(), 4, [buffer.data_ptr()], -1,
                                stream)


@pytest.mark.parametrize("schedule", ["split", "resident"])
@pytest.mark.parametrize("kind", ["sum", "max", "min"])
def test_fused_launch_stores_every_result_in_every_destination(kind, schedule):
    """Same-process form of the fused reduce + exchange: three destination
    arrays on this GPU, results at an odd offset.  Bit for bit what the plain
    launch with the same plan and schedule writes (so parity with the oracle
    carries over), guard elements untouched."""
    import workloads
    from swage_b200._segmented_qualification import launch_gpu, plan_segments

    offsets = workloads.c5_offsets(segments=(1 << 13) + 5, total=1 << 21,
                                   giants=3, giant_length=1 << 18)
    segments = len(offsets) - 1
    count = int(offsets[-1])
    values = workloads.normal_values(count, "cuda", 17)
    device_offsets = torch.as_tensor(offsets).cuda()
    plan = plan_segments(device_offsets, count)
    try:
        plain = torch.empty(segments, device="cuda")
        launch_gpu(values, device_offsets, plain, kind, plan=plan,
                   schedule=schedule, extensions=True)
        shift = 37
        destinations = [
            torch.full((shift + segments + 9,), float("nan"), device="cuda")
            for _ in range(3)]
        _native.segreduce_peers(
            {"sum": 0, "max": 1, "min": 2}[kind], values.data_ptr(),
            device_offsets.data_ptr(), [d.data_ptr() for d in destinations],
            shift, count, segments, plan.handle, _native.SCHEDULES[schedule],
            torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        plan.check()
        expected = plain.cpu().numpy().view(np.uint32)
        for destination in destinations:
            host = destination.cpu().numpy()
            assert np.array_equal(
                host[shift:shift + segments].view(np.uint32), expected)
            assert np.isnan(host[:shift]).all()
            assert np.isnan(host[shift + segments:]).all()
    finally:
        plan.close()


def test_fused_launch_needs_a_plan():
    values = torch.ones(8, device="cuda")
    offsets = torch.tensor([0, 4, 8], dtype=torch.int32, device="cuda")
    out = torch.zeros(2, device="cuda")
    with pytest.raises(RuntimeError, match="needs a plan"):
        _native.segreduce_peers(0, values.data_ptr(), offsets.data_ptr(),
                                [out.data_ptr()], 0, 8, 2, None, 0,
                                torch.cuda.current_stream().cuda_stream)


def free_port():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_ranks_publish_their_shards_into_every_copy(world):
    """``world`` processes (one GPU each where the box has that many, else all
    on GPU 0), gloo for the host side: every rank reduces its shard, publishes
    it, and finds the oracle's full result in its own copy."""
    environment = dict(os.environ, WORLD_SIZE=str(world),
                       MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
    ranks = [
        subprocess.Popen([sys.executable, str(WORKER)],
                         env=dict(environment, RANK=str(rank)),
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True)
        for rank in range(world)
    ]
    outputs = []
    try:
        for process in ranks:
            text, _ = process.communicate(timeout=240)
            outputs.append(text)
    finally:
        for process in ranks:
            if process.poll() is None:
                process.kill()
    for rank, (process, text) in enumerate(zip(ranks, outputs)):
        assert process.returncode == 0, f"rank {rank}:\n{text[-3000:]}"
        assert f"rank {rank} ok" in text
