"""Benchmark of the segmented-reduction hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
                    [--impl ours|reference] [--schedule NAME] [--allgather]

One "step" is one pass of the hot path over one batch of synthetic input.
Default workload ``c5``: extreme-skew segmented sum, 2**30 fp32 values in 2**22
segments (64 of them 2**23 long), the configuration the multi-GPU metric is
quoted on.  With N > 1 (launched by torchrun, one rank per GPU) the SAME 2**30
values are cut into N element-balanced contiguous segment ranges -- strong
scaling, no data-path collective (``--allgather`` adds the optional NCCL
all-gather of the per-segment results to every step).

Rank 0 prints ONE JSON line.  ``value`` is whole-job throughput with inputs
resident in HBM; ``e2e`` is the same metric through the public
``launch_gpu`` / ``kernel.launch`` call with the inputs copied from pinned host
memory and the result read back inside the timed region; ``roofline`` is the
dominant kernel against the measured HBM copy bandwidth; ``cpu_baseline`` is
the CPU oracle timed on this host; ``plan`` gives the one-off cost of building
the schedule (on the GPU from device-resident offsets, and by the host
planner from a host copy) and of validating the offsets on the GPU, none of
which is inside ``value``'s timed region (``e2e`` pays validation every step
and finds the plan by the offsets' content digest).

``--impl reference`` times the reference's CPU path -- the sequential lowering
restated in ``oracle/`` (the reference's own executable path needs an LLVM
toolchain that is not in its tree) -- on all host threads, same workload.
"""

import argparse
import json
import os
import pathlib
import subprocess
import sys
import tempfile
import time

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

import workloads  # noqa: E402

NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per launch of the dominant kernel divided by its algorithmic
# bytes, from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum).
# c5: capture of the workload shrunk 4x, 1.090 GB for 1.082 GB (traffic grows
# in proportion to the units processed); c4: the kernels of a full-size call,
# 8.75 GB for 9.055 GB (reads 4.562 GB for 4.528 GB of input; the writes
# counted are short of the output because the last lines of each kernel are
# still in L2 when it ends).  Workloads without a capture report null.
TRAFFIC_RATIO = {"c5": 1.0074, "c4": 0.966}


def parse_arguments():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=400)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="c5",
                        choices=["c1", "c1x256", "c2", "c3", "c4", "c5"])
    parser.add_argument("--schedule", default="auto")
    parser.add_argument("--block", type=int, default=128)
    parser.add_argument("--allgather", action="store_true")
    parser.add_argument("--planner", default="device",
                        choices=["device", "host"],
                        help="where the plan of the timed region is built "
                             "(both are built once and timed)")
    parser.add_argument("--e2e-steps", type=int, default=None)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-probe", action="store_true",
                        help="do not record per-kernel events in the timed "
                             "region (roofline.achieved is then null)")
    parser.add_argument("--shrink", type=int, default=1,
                        help="divide the c5 workload by this power of two "
                             "(profiling captures only; not a bench value)")
    return parser.parse_args()


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------
# workload description
# ---------------------------------------------------------------------------

def describe_workload(name, shrink=1):
    """(operation, kind, offsets or None, description)."""
    if name == "c5" and shrink > 1:
        offsets = workloads.c5_offsets(
            segments=(1 << 22) // shrink, total=(1 << 30) // shrink,
            giants=max(1, 64 // shrink))
        return "reduce", "sum", offsets, \
            f"extreme skew shrunk {shrink}x (profiling only)"
    if name == "c4" and shrink > 1:
        return "softmax", None, \
            workloads.c4_offsets(segments=262144 // shrink), \
            f"softmax shrunk {shrink}x (profiling only)"
    if name == "c1":
        offsets = workloads.c1_offsets()
        return "reduce", "sum", offsets, "canonical 4096 segments U{0..2048}"
    if name == "c1x256":
        offsets = workloads.c1_offsets(segments=1 << 20)
        return "reduce", "sum", offsets, "canonical x256: 2^20 segments U{0..2048}"
    if name == "c3":
        return "reduce", "max", workloads.c3_offsets(), \
            "lognormal(5,1.5) lengths, 2^20 segments, max"
    if name == "c4":
        return "softmax", None, workloads.c4_offsets(), \
            "softmax 262144 segments, 50/40/10 % length mix"
    if name == "c5":
        return "reduce", "sum", workloads.c5_offsets(), \
            "extreme skew: 2^22 segments, 2^30 values, 64 x 2^23"
    return "vadd", None, None, "vector add n = 2^28 - 37"


def make_values(name, offsets, device):
    if name == "c3":
        return workloads.c3_values(offsets, device)
    scale = 2.0 if name == "c4" else 1.0
    return workloads.normal_values(int(offsets[-1]), device,
                                   workloads.SEEDS[name[:2]], scale=scale)


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------

class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,"
             "clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv",
                                                delete=False)
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self):
        result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [],
                  "samples": 0}
        if self.process is None:
            return result
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, max_clocks, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                 "sw_power_cap")
        for line in self.file.read().splitlines():
            cells = [cell.strip() for cell in line.split(",")]
            if len(cells) < 7:
                continue
            try:
                clocks.append(float(cells[0]))
                max_clocks.append(float(cells[1]))
                power.append(float(cells[2]))
            except ValueError:
                continue
            for name, cell in zip(names, cells[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if clocks:
            # "under load" = the upper half of the power samples
            order = np.argsort(power)
            loaded = [clocks[i] for i in order[len(order) // 2:]]
            result.update(sm_mhz=float(np.median(loaded)),
                          sm_max_mhz=float(max(max_clocks)),
                          reasons=sorted(reasons), samples=len(clocks),
                          power_w_max=float(max(power)))
        return result


# ---------------------------------------------------------------------------
# reference arm: the CPU path on all host threads
# ---------------------------------------------------------------------------

def cpu_sample(name, offsets, limit_elements):
    """A prefix of whole segments holding at most ``limit_elements``."""
    if offsets is None:
        return None
    last = int(np.searchsorted(offsets, limit_elements, side="right")) - 1
    last = max(1, min(last, len(offsets) - 1))
    return offsets[:last + 1]


def cpu_pass(operation, kind, values, offsets, threads, block):
    import oracle

    start = time.perf_counter()
    if operation == "reduce":
        oracle.segreduce_f32(values, offsets, kind, threads=threads)
    elif operation == "softmax":
        oracle.segsoftmax_f32(values, offsets, threads=threads)
    else:
        oracle.vadd_f32(values[0], values[1], len(values[0]), block=block,
                        threads=threads)
    return time.perf_counter() - start


def host_inputs(name, operation, offsets, count):
    """Host arrays with the workload's distribution (numpy, seeded)."""
    rng = np.random.default_rng(workloads.SEEDS[name[:2]])
    if operation == "vadd":
        return (rng.standard_normal(count, dtype=np.float32),
                rng.standard_normal(count, dtype=np.float32))
    if name == "c3":
        return rng.uniform(-1e3, 1e3, size=count).astype(np.float32)
    values = rng.standard_normal(count, dtype=np.float32)
    if name == "c4":
        values *= 2.0
    return values


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    oracle.build()
    operation, kind, offsets, text = describe_workload(args.workload,
                                                       args.shrink)
    threads = oracle.max_threads()
    full_count = int(offsets[-1]) if offsets is not None else (1 << 28) - 37
    # probe the throughput on a small sample, then size the timed sample so
    # that steps + warm-up stay within about two minutes
    probe_offsets = cpu_sample(args.workload, offsets, 1 << 24)
    probe_count = int(probe_offsets[-1]) if offsets is not None else 1 << 24
    probe_values = host_inputs(args.workload, operation, probe_offsets,
                               probe_count)
    cpu_pass(operation, kind, probe_values, probe_offsets, threads, args.block)
    rate = probe_count / cpu_pass(operation, kind, probe_values,
                                  probe_offsets, threads, args.block)
    seconds_per_step = 120.0 / max(1, args.steps + args.warmup)
    sample_count = int(min(full_count, max(1 << 22, rate * seconds_per_step)))
    sample_offsets = cpu_sample(args.workload, offsets, sample_count)
    if offsets is not None:
        sample_count = int(sample_offsets[-1])
    values = host_inputs(args.workload, operation, sample_offsets,
                         sample_count)
    for _ in range(args.warmup):
        cpu_pass(operation, kind, values, sample_offsets, threads, args.block)
    elapsed = 0.0
    for _ in range(args.steps):
        elapsed += cpu_pass(operation, kind, values, sample_offsets, threads,
                            args.block)
    value = sample_count * args.steps / elapsed / 1e9
    sample = (f"{sample_count} of {full_count} elements "
              f"({'whole workload' if sample_count == full_count else 'prefix of whole segments'})")
    line = {
        "impl": "reference",
        "metric": metric_name(operation), "value": value, "unit": "Gelem/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {text}",
                   "device": "host CPU", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "Gelem/s", "cores": threads,
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "Gelem/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def metric_name(operation):
    return {"reduce": "segmented_reduce_throughput",
            "softmax": "segmented_softmax_throughput",
            "vadd": "vector_add_throughput"}[operation]


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist

    import swage_b200 as sw
    import swage_b200.language as sl
    from swage_b200 import _native, multi_gpu
    from swage_b200._segmented_qualification import (
        launch_gpu,
        launch_softmax_gpu,
        plan_segments,
    )

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL announces its version on stdout when its communicator comes
        # up; stdout carries the one JSON line only, so the communicator is
        # created here with descriptor 1 pointing at stderr
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    operation, kind, offsets, text = describe_workload(args.workload,
                                                       args.shrink)
    peak, peak_source = measured_peak()
    plan_info = {}

    @sw.jit
    def add_kernel(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):
        pid = sl.program_id(0)
        offsets = pid * BLOCK + sl.arange(0, BLOCK)
        mask = offsets < n
        x = sl.load(x_ptr + offsets, mask=mask, other=0.0)
        y = sl.load(y_ptr + offsets, mask=mask, other=0.0)
        sl.store(output_ptr + offsets, x + y, mask=mask)

    # ---- this rank's share ----
    if operation == "vadd":
        total = (1 << 28) - 37
        per = -(-total // world)
        per += (-per) % 32  # 128-byte boundaries between ranks
        begin = min(total, rank * per)
        count = min(total, begin + per) - begin
        generator = torch.Generator(device=device).manual_seed(
            workloads.SEEDS["c2"] + rank)
        x = torch.randn(count, generator=generator, device=device)
        y = torch.randn(count, generator=generator, device=device)
        out = torch.empty(count, device=device)
        segments = 0
        bytes_per_step = workloads.vadd_bytes(count)
        total_elements = total
        plan = None
        local_offsets = None
    else:
        total_elements = int(offsets[-1])
        host_offsets = torch.from_numpy(offsets)
        cuts = multi_gpu.shard_cuts(host_offsets, world)
        local, begin, end = multi_gpu.local_shard(host_offsets, cuts, rank)
        local_offsets = local.numpy()
        full = make_values(args.workload, offsets, device)
        values = full[begin:end].clone() if world > 1 else full
        del full
        torch.cuda.empty_cache()
        count = end - begin
        segments = len(local_offsets) - 1
        device_offsets = torch.from_numpy(local_offsets).to(device)
        if operation == "reduce":
            out = torch.empty(segments, device=device)
            bytes_per_step = workloads.reduce_bytes(count, segments)
            plan_op = "reduce"
        else:
            out = torch.empty(count, device=device)
            bytes_per_step = workloads.softmax_bytes(count, segments)
            plan_op = "softmax"
        # both planners once, outside the timed region: the host walk over a
        # host copy of the offsets, and the GPU planner over the device copy
        # (each twice; the second build is reported: the first one also pays
        # for loading the planner's kernels)
        plans = {}
        for where, source in (("host", torch.from_numpy(local_offsets)),
                              ("device", device_offsets)):
            for attempt in range(2):
                if attempt:
                    plans[where].close()
                torch.cuda.synchronize()
                began = time.perf_counter()
                plans[where] = plan_segments(source, count, op=plan_op)
                torch.cuda.synchronize()
                plan_info[where + "_build_ms"] = (
                    1e3 * (time.perf_counter() - began))
        plan = plans.pop(args.planner)
        for other in plans.values():
            other.close()
        plan_info["planner"] = args.planner
        began = time.perf_counter()
        _native.validate_offsets_device(
            device_offsets.data_ptr(), segments, count, segments,
            torch.cuda.current_stream().cuda_stream)
        plan_info["validate_on_device_us"] = 1e6 * (time.perf_counter() - began)
    gather = args.allgather and world > 1 and operation == "reduce"

    launches_per_step = [0]

    def step():
        if operation == "vadd":
            add_kernel.launch(
                arguments={"x_ptr": x, "y_ptr": y, "output_ptr": out,
                           "n": count},
                constexprs={"BLOCK": args.block},
                grid=(-(-count // args.block),))
        elif operation == "reduce":
            launch_gpu(values, device_offsets, out, kind, args.block,
                       plan=plan, schedule=args.schedule,
                       _validated=(count, segments))
            if gather:
                multi_gpu.gather_results(out, cuts)
        else:
            launch_softmax_gpu(values, device_offsets, out, plan=plan,
                               schedule=args.schedule,
                               _validated=(count, segments))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    barrier()
    # the dominant kernel of every probe_stride-th step is timed with its own
    # pair of events; a sparse sample keeps the event records (about 5 us of
    # stream time per pair) from inflating the step time
    probe_stride = 8 if args.steps >= 64 else 1
    if not args.no_probe:
        _native.profile_start(args.steps, probe_stride)
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    kernel_ms = [] if args.no_probe else _native.profile_stop(args.steps)
    if plan is not None:
        plan.check()
    times = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms = float(times.item())

    # kernels per step: planned reduce = tile kernel + combine pass (when any
    # segment is split); everything else = one kernel
    per_step = 1
    if plan is not None and operation == "reduce":
        info = plan.describe()
        uses_tiles = (args.schedule in ("split", "persistent")
                      or (args.schedule == "auto" and info["schedule"] >= 3))
        if uses_tiles and info["split_segments"] > 0:
            per_step = 2
    if plan is not None and operation == "softmax":
        info = plan.describe()
        per_step = sum(1 for n in info["softmax_buckets"] if n > 0)
    launches_per_step[0] = per_step

    # ---- end to end through the public call, host buffers ----
    e2e_steps = args.e2e_steps or max(1, min(args.steps, 5))
    if operation == "vadd":
        host_inputs_ = [x.cpu().pin_memory(), y.cpu().pin_memory()]
        host_out = torch.empty(count, dtype=torch.float32).pin_memory()
        h2d = 8 * count
        d2h = 4 * count
    else:
        host_inputs_ = [values.cpu().pin_memory(),
                        torch.from_numpy(local_offsets).pin_memory()]
        host_out = torch.empty(out.numel(), dtype=torch.float32).pin_memory()
        h2d = 4 * count + 4 * (segments + 1)
        d2h = 4 * out.numel()

    def e2e_step():
        if operation == "vadd":
            x.copy_(host_inputs_[0], non_blocking=True)
            y.copy_(host_inputs_[1], non_blocking=True)
            add_kernel.launch(
                arguments={"x_ptr": x, "y_ptr": y, "output_ptr": out,
                           "n": count},
                constexprs={"BLOCK": args.block},
                grid=(-(-count // args.block),))
        else:
            values.copy_(host_inputs_[0], non_blocking=True)
            device_offsets.copy_(host_inputs_[1], non_blocking=True)
            if operation == "reduce":
                # the drop-in call: validates the offsets, finds the plan
                launch_gpu(values, device_offsets, out, kind, args.block,
                           schedule=args.schedule)
            else:
                launch_softmax_gpu(values, device_offsets, out,
                                   schedule=args.schedule)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    barrier()
    e2e_start = torch.cuda.Event(enable_timing=True)
    e2e_stop = torch.cuda.Event(enable_timing=True)
    e2e_start.record()
    wall = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_stop.record()
    barrier()
    e2e_ms = max(e2e_start.elapsed_time(e2e_stop),
                 1e3 * (time.perf_counter() - wall))
    times = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    e2e_ms = float(times.item())
    clocks = sampler.stop() if sampler is not None else None

    # ---- CPU baseline on this host (rank 0, single GPU runs only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle

        oracle.build()
        threads = oracle.max_threads()
        if operation == "vadd":
            sample_offsets = None
            sample_values = (host_inputs_[0].numpy(), host_inputs_[1].numpy())
            sample_count = count
        else:
            # bounded sample: a prefix of whole segments, at most 2**29 values
            sample_offsets = cpu_sample(args.workload, local_offsets, 1 << 29)
            sample_count = int(sample_offsets[-1])
            sample_values = host_inputs_[0].numpy()[:sample_count]
        single = cpu_pass(operation, kind, sample_values, sample_offsets, 1,
                          args.block)
        cpu_pass(operation, kind, sample_values, sample_offsets, threads,
                 args.block)
        parallel = min(
            cpu_pass(operation, kind, sample_values, sample_offsets, threads,
                     args.block) for _ in range(3))
        cpu = {
            "value": sample_count / parallel / 1e9, "unit": "Gelem/s",
            "cores": threads, "kind": "port",
            "sample": f"{sample_count} of {count} elements, best of 3",
            "single_thread_value": sample_count / single / 1e9,
        }

    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        gelems = total_elements / (ms_per_step * 1e-3) / 1e9
        kernel_avg_ms = float(np.mean(kernel_ms)) if kernel_ms else None
        achieved = (bytes_per_step / (kernel_avg_ms * 1e-3) / 1e9
                    if kernel_avg_ms else None)
        step_gbs = bytes_per_step / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": metric_name(operation), "value": gelems,
            "unit": "Gelem/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": f"{args.workload}: {text}",
                "elements_total": total_elements,
                "elements_rank0": count, "segments_rank0": segments,
                "schedule": args.schedule,
                "sharding": f"{world} element-balanced contiguous segment "
                            "ranges, no collective"
                            + (" + NCCL all-gather of results"
                               if gather else ""),
                "l2": "inputs larger than L2" if bytes_per_step > 3e8
                      else "inputs fit in L2 (warm)",
            },
            "hbm_gbs_per_gpu": step_gbs,
            "pct_of_8tbs_per_gpu": 100.0 * step_gbs / NOMINAL_HBM_GBS,
            "clocks": clocks,
            "e2e": {"value": total_elements / (e2e_ms / e2e_steps * 1e-3) / 1e9,
                    "unit": "Gelem/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps * launches_per_step[0],
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak,
                "unit": "GB/s",
                "frac": achieved / peak if achieved else None,
                "traffic": (TRAFFIC_RATIO[args.workload] * bytes_per_step
                            if args.workload in TRAFFIC_RATIO
                            and args.shrink == 1 else None),
                "traffic_source": "ncu capture, scaled by algorithmic bytes"
                if args.workload in TRAFFIC_RATIO else None,
                "peak_source": peak_source,
                "kernel_ms": kernel_avg_ms,
                "kernel_launches_timed": len(kernel_ms),
                "algorithmic_bytes_per_launch": bytes_per_step,
                "pct_of_8tbs": 100.0 * achieved / NOMINAL_HBM_GBS
                if achieved else None,
            },
            "cpu_baseline": cpu,
            "plan": plan_info or None,
        }
        print(json.dumps(line))
    if plan is not None:
        plan.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_arguments()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
