"""One rank of tests/test_gpu_peer_results.py (run as a child process).

Reduces its shard of a small extreme-skew problem, publishes the results into
every rank's copy through ``PeerResults`` -- once with the scatter kernel
behind the reduction, once with the reduction's own warps storing into every
copy -- and checks the full array against the CPU oracle.  RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT come from the
environment; the ranks talk over gloo, and share GPU 0 when the box has fewer
GPUs than ranks (CUDA IPC works between processes on one device too).
"""

import os
import pathlib
import sys

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import oracle  # noqa: E402
import workloads  # noqa: E402
from swage_b200 import multi_gpu  # noqa: E402
from swage_b200._segmented_qualification import (  # noqa: E402
    launch_gpu,
    plan_segments,
)


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    device = rank if torch.cuda.device_count() >= world else 0
    torch.cuda.set_device(device)
    offsets = workloads.c5_offsets(segments=(1 << 12) + 3, total=1 << 20,
                                   giants=2, giant_length=1 << 18)
    host_values = workloads.normal_values(int(offsets[-1]), "cpu", 5).numpy()
    cuts = multi_gpu.shard_cuts(torch.from_numpy(offsets), world)
    local, begin, end = multi_gpu.local_shard(torch.from_numpy(offsets), cuts,
                                              rank)
    values = torch.from_numpy(host_values[begin:end]).cuda()
    device_offsets = local.cuda()
    exchange = multi_gpu.PeerResults(cuts)
    try:
        for kind in ("max", "sum"):
            output = torch.empty(local.numel() - 1, device="cuda")
            launch_gpu(values, device_offsets, output, kind)
            exchange.publish(output)
            exchange.wait()
            got = exchange.results.cpu().numpy()
            if kind == "max":
                expected = oracle.segreduce_f32(host_values, offsets, "max")
                assert np.array_equal(got.view(np.uint32),
                                      expected.view(np.uint32)), "max differs"
            else:
                exact = oracle.segsum_f64(host_values, offsets)
                bound = oracle.sum_tolerance(host_values, offsets)
                assert np.all(np.abs(got - exact) <= bound), "sum out of bound"
            dist.barrier()  # everyone has read before the next kind overwrites
        # the fused form: the reduction's own warps store into every copy
        plan = plan_segments(device_offsets, int(values.numel()))
        try:
            for kind, schedule in (("max", "split"), ("max", "resident"),
                                   ("sum", "auto")):
                exchange.results.fill_(float("nan"))
                torch.cuda.synchronize()
                dist.barrier()
                exchange.reduce(values, device_offsets, kind, plan,
                                schedule=schedule)
                exchange.wait()
                got = exchange.results.cpu().numpy()
                if kind == "max":
                    expected = oracle.segreduce_f32(host_values, offsets,
                                                    "max")
                    assert np.array_equal(got.view(np.uint32),
                                          expected.view(np.uint32)), schedule
                else:
                    exact = oracle.segsum_f64(host_values, offsets)
                    bound = oracle.sum_tolerance(host_values, offsets)
                    assert np.all(np.abs(got - exact) <= bound), schedule
                dist.barrier()
            plan.check()
        finally:
            plan.close()
    finally:
        exchange.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
