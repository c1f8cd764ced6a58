"""The N > 1 path on CPU: two gloo ranks shard, reduce (with the oracle
standing in for the kernels) and all-gather; results equal the unsharded run."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
import workloads
from swage_b200 import multi_gpu


def free_port():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        offsets = torch.from_numpy(workloads.c5_offsets(
            segments=1 << 12, total=1 << 18, giants=3, giant_length=1 << 15))
        values = np.random.default_rng(7).standard_normal(
            int(offsets[-1])).astype(np.float32)
        cuts = multi_gpu.shard_cuts(offsets, world)
        local, begin, end = multi_gpu.local_shard(offsets, cuts, rank)
        assert int(local[0]) == 0 and int(local[-1]) == end - begin
        # each rank reduces only its own slice
        mine = torch.from_numpy(
            oracle.segreduce_f32(values[begin:end], local.numpy(), "max"))
        everything = multi_gpu.gather_results(mine, cuts)
        expected = oracle.segreduce_f32(values, offsets.numpy(), "max")
        assert np.array_equal(everything.numpy().view(np.uint32),
                              expected.view(np.uint32))
        sizes = [int(offsets[cuts[g + 1]] - offsets[cuts[g]])
                 for g in range(world)]
        longest = int((offsets[1:] - offsets[:-1]).max())
        results[rank] = (cuts, sizes, longest)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_reduce_and_gather_match_the_unsharded_result(world):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), results), nprocs=world,
             join=True)
    assert len(results) == world
    cuts, sizes, longest = results[0]
    assert all(results[r][0] == cuts for r in range(world))
    assert cuts[0] == 0 and cuts[-1] == 1 << 12
    assert sum(sizes) == 1 << 18
    # element-balanced: a segment is never split, so no shard is further from
    # the ideal size than the longest segment
    ideal = (1 << 18) / world
    assert max(abs(size - ideal) for size in sizes) <= longest


def test_shard_helpers_validate_their_inputs():
    offsets = torch.tensor([0, 3, 3, 10], dtype=torch.int32)
    assert multi_gpu.shard_cuts(offsets, 1) == [0, 3]
    with pytest.raises(TypeError, match="CPU int32"):
        multi_gpu.shard_cuts(offsets.long(), 2)
    with pytest.raises(ValueError, match="positive integer"):
        multi_gpu.shard_cuts(offsets, 0)
    local, begin, end = multi_gpu.local_shard(offsets, [0, 1, 3], 1)
    assert local.tolist() == [0, 0, 7] and (begin, end) == (3, 10)
