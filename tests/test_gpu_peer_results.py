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
