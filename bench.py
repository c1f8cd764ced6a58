"""Benchmark of the segmented-reduction hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
                    [--impl ours|reference] [--schedule NAME]
                    [--allgather | --peer-results [fused|scatter]]

One "step" is one pass of the hot path over one batch of synthetic input.
Default workload ``c5``: extreme-skew segmented sum, 2**30 fp32 values in 2**22
segments (64 of them 2**23 long), the configuration the multi-GPU metric is
quoted on.  With N > 1 (launched by torchrun, one rank per GPU) the SAME 2**30
values are cut into N element-balanced contiguous segment ranges -- strong
scaling, no data-path collective (``--allgather`` adds the optional NCCL
all-gather of the per-segment results to every step; ``--peer-results`` the
same exchange without a collective: every rank stores its results into every
rank's copy through peer-mapped memory -- ``fused``, the default: by the
reducing warps themselves; ``scatter``: by one small kernel behind the
reduction).

Rank 0 prints ONE JSON line.

``value``      whole-job throughput with inputs resident in HBM and the plan
               built: K steps between two CUDA events, nothing else recorded
               on the stream inside that region.
``roofline``   the dominant kernel against the measured HBM copy bandwidth;
               its duration comes from a SEPARATE short loop in which the
               library records a pair of events around that kernel.
``cold``       the drop-in call on offsets the plan cache has not seen:
               validation + planning + launch, device-resident inputs.
``e2e``        the drop-in call with the inputs copied from pinned host
               memory and the result read back, every step.
``workloads``  (1 GPU) the other configurations measured the same way in the
               same process, each with its parity status against the CPU
               oracle at full size.
``cpu_baseline`` the CPU restatement of the reference's sequential lowering
               timed on this host's cores.

``--impl reference`` times that CPU restatement (the reference's own
executable path needs an LLVM toolchain that is not in its tree) on all host
cores, on the same seeded inputs as the GPU arm.
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
# bytes, from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum) of
# shrunk cases; traffic grows in proportion to the units processed.
# Softmax: the reads were measured (1.0077 x the input on a case shrunk 8x);
# the writes are counted as algorithmic, because at that size much of the
# output is still dirty in L2 when a kernel ends and the counter misses it.
# Workloads without a capture report null.
TRAFFIC_RATIO = {"c5": 1.0091, "c4": 1.004}
ALL_WORKLOADS = ("c1", "c1x256", "c2", "c3", "c4", "c5")
VADD_COUNT = (1 << 28) - 37


def parse_arguments():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=400)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="c5", choices=ALL_WORKLOADS)
    parser.add_argument("--schedule", default="auto")
    parser.add_argument("--block", type=int, default=128)
    parser.add_argument("--allgather", action="store_true")
    parser.add_argument("--peer-results", nargs="?", const="fused",
                        default=None, choices=["fused", "scatter"],
                        help="every step also stores this rank's results "
                             "into every rank's copy (peer-mapped memory)")
    parser.add_argument("--planner", default="device",
                        choices=["device", "host"],
                        help="where the plan of the timed region is built "
                             "(both are built once and timed)")
    parser.add_argument("--e2e-steps", type=int, default=None)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-others", action="store_true",
                        help="skip the `workloads` entry (the other "
                             "configurations)")
    parser.add_argument("--no-parity", action="store_true",
                        help="skip the oracle comparison of the measured "
                             "workloads")
    parser.add_argument("--shrink", type=int, default=1,
                        help="divide the c5 / c4 workload by this power of "
                             "two (profiling captures only; not a bench "
                             "value)")
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
        return "reduce", "sum+max", offsets, \
            "canonical 4096 segments U{0..2048}, sum and max"
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
    """The workload's seeded values, drawn on ``device``."""
    if name == "c3":
        return workloads.c3_values(offsets, device)
    scale = 2.0 if name == "c4" else 1.0
    return workloads.normal_values(int(offsets[-1]), device,
                                   workloads.SEEDS[name[:2]], scale=scale)


def vadd_inputs(count, device, rank=0):
    import torch

    generator = torch.Generator(device=device).manual_seed(
        workloads.SEEDS["c2"] + rank)
    x = torch.randn(count, generator=generator, device=device)
    y = torch.randn(count, generator=generator, device=device)
    return x, y


def algorithmic_bytes(operation, kind, count, segments):
    if operation == "vadd":
        return workloads.vadd_bytes(count)
    if operation == "softmax":
        return workloads.softmax_bytes(count, segments)
    if kind == "sum+max":
        return workloads.reduce_bytes(count, segments) + 4 * segments
    return workloads.reduce_bytes(count, segments)


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
# the CPU path (reference arm and cpu_baseline)
# ---------------------------------------------------------------------------

def cpu_sample(offsets, limit_elements):
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
        for one in kind.split("+"):
            oracle.segreduce_f32(values, offsets, one, threads=threads)
    elif operation == "softmax":
        oracle.segsoftmax_f32(values, offsets, threads=threads)
    else:
        oracle.vadd_f32(values[0], values[1], len(values[0]), block=block,
                        threads=threads)
    return time.perf_counter() - start


def host_inputs(name, operation, offsets, count):
    """Host arrays holding the first ``count`` values of the workload.

    The same seeded values as the GPU arm: drawn by the same device generator
    and copied to the host when a CUDA device is there; a numpy draw with the
    workload's distribution otherwise (no GPU arm can run then either).
    """
    try:
        import torch

        on_device = torch.cuda.is_available()
    except Exception:
        on_device = False
    if on_device:
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        if operation == "vadd":
            x, y = vadd_inputs(VADD_COUNT, device)
            return x[:count].cpu().numpy(), y[:count].cpu().numpy()
        full = make_values(name, offsets, device)
        return full[:count].cpu().numpy()
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
    # every core this process may use, whatever OMP_NUM_THREADS a launcher
    # exported for its ranks
    threads = oracle.host_threads()
    full_count = int(offsets[-1]) if offsets is not None else VADD_COUNT
    everything = host_inputs(args.workload, operation, offsets, full_count)

    def prefix(sample_offsets, count):
        if operation == "vadd":
            return everything[0][:count], everything[1][:count]
        return everything[:count]

    # probe the throughput on a small sample, then size the timed sample so
    # that steps + warm-up stay within about two minutes
    probe_offsets = cpu_sample(offsets, 1 << 24)
    probe_count = int(probe_offsets[-1]) if offsets is not None else 1 << 24
    probe_values = prefix(probe_offsets, probe_count)
    cpu_pass(operation, kind, probe_values, probe_offsets, threads, args.block)
    rate = probe_count / cpu_pass(operation, kind, probe_values,
                                  probe_offsets, threads, args.block)
    seconds_per_step = 120.0 / max(1, args.steps + args.warmup)
    sample_count = int(min(full_count, max(1 << 22, rate * seconds_per_step)))
    sample_offsets = cpu_sample(offsets, sample_count)
    if offsets is not None:
        sample_count = int(sample_offsets[-1])
    values = prefix(sample_offsets, sample_count)
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
        "config": workload_config(args, text, operation, kind, offsets),
        "run": {"device": "host CPU", "sample": sample, "threads": threads},
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


def workload_config(args, text, operation, kind, offsets):
    """The ``config`` object: identical on both arms for one workload."""
    if offsets is None:
        elements, segments = VADD_COUNT, 0
    else:
        elements, segments = int(offsets[-1]), len(offsets) - 1
    fits = algorithmic_bytes(operation, kind, elements, segments) < 3e8
    return {
        "workload": f"{args.workload}: {text}",
        "elements_total": elements, "segments_total": segments,
        "l2": ("inputs fit in L2: the kernel is timed after a 256 MiB write "
               "(cold); back-to-back steps are L2-warm") if fits
        else "inputs larger than L2",
    }


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------

class Problem:
    """One workload's share on this rank, resident on the device."""

    def __init__(self, name, args, world, rank, device, shrink=1):
        import torch

        from swage_b200 import multi_gpu

        self.name = name
        self.args = args
        self.device = device
        (self.operation, self.kind, offsets,
         self.text) = describe_workload(name, shrink)
        self.full_offsets = offsets
        self.plan = None
        self._bound_step = None
        self.plan_info = {}
        self.cuts = None
        if self.operation == "vadd":
            total = VADD_COUNT
            per = -(-total // world)
            per += (-per) % 32  # 128-byte boundaries between ranks
            begin = min(total, rank * per)
            self.count = min(total, begin + per) - begin
            if world == 1:
                self.x, self.y = vadd_inputs(self.count, device)
            else:
                self.x, self.y = vadd_inputs(self.count, device, rank)
            self.out = torch.empty(self.count, device=device)
            self.segments = 0
            self.total_elements = total
            self.local_offsets = None
        else:
            self.total_elements = int(offsets[-1])
            host_offsets = torch.from_numpy(offsets)
            self.cuts = multi_gpu.shard_cuts(host_offsets, world)
            local, begin, end = multi_gpu.local_shard(host_offsets, self.cuts,
                                                      rank)
            self.local_offsets = local.numpy()
            full = make_values(name, offsets, device)
            self.values = full[begin:end].clone() if world > 1 else full
            del full
            torch.cuda.empty_cache()
            self.count = end - begin
            self.segments = len(self.local_offsets) - 1
            self.device_offsets = torch.from_numpy(
                self.local_offsets).to(device)
            if self.operation == "softmax":
                self.out = torch.empty(self.count, device=device)
            else:
                self.out = torch.empty(self.segments, device=device)
                if self.kind == "sum+max":
                    self.out2 = torch.empty(self.segments, device=device)
        self.bytes_per_step = algorithmic_bytes(self.operation, self.kind,
                                                self.count, self.segments)

    def build_plans(self):
        """Both planners once, outside every timed region (each twice; the
        second build is reported: the first also loads the planner's
        kernels)."""
        import torch

        from swage_b200 import _native
        from swage_b200._segmented_qualification import plan_segments

        if self.operation == "vadd" or self.kind == "sum+max":
            return
        plan_op = "softmax" if self.operation == "softmax" else "reduce"
        plans = {}
        for where, source in (("host", torch.from_numpy(self.local_offsets)),
                              ("device", self.device_offsets)):
            for attempt in range(2):
                if attempt:
                    plans[where].close()
                torch.cuda.synchronize()
                began = time.perf_counter()
                plans[where] = plan_segments(source, self.count, op=plan_op)
                torch.cuda.synchronize()
                self.plan_info[where + "_build_ms"] = (
                    1e3 * (time.perf_counter() - began))
        self.plan = plans.pop(self.args.planner)
        self._bound_step = None
        for other in plans.values():
            other.close()
        self.plan_info["planner"] = self.args.planner
        began = time.perf_counter()
        _native.validate_offsets_device(
            self.device_offsets.data_ptr(), self.segments, self.count,
            self.segments, torch.cuda.current_stream().cuda_stream)
        self.plan_info["validate_on_device_us"] = (
            1e6 * (time.perf_counter() - began))

    def step(self):
        """One pass with the inputs where they are and the plan built.  The
        call is bound once (``bound_step``): for the 12 us step of the
        canonical configuration the look-ups of a generic dispatch would be a
        tenth of what is measured."""
        if self._bound_step is None:
            self._bound_step = self.bound_step()
        self._bound_step()

    def bound_step(self):
        """A closure over this problem's tensors that makes the one call."""
        from swage_b200._segmented_qualification import (
            launch_gpu,
            launch_softmax_gpu,
            launch_sum_max_gpu,
        )

        args = self.args
        validated = (self.count, self.segments)
        if self.operation == "vadd":
            kernel = add_kernel()
            arguments = {"x_ptr": self.x, "y_ptr": self.y,
                         "output_ptr": self.out, "n": self.count}
            constexprs = {"BLOCK": args.block}
            grid = (-(-self.count // args.block),)

            def step():
                kernel.launch(arguments=arguments, constexprs=constexprs,
                              grid=grid)
        elif self.kind == "sum+max":
            values, offsets = self.values, self.device_offsets
            out, out2 = self.out, self.out2

            def step():
                launch_sum_max_gpu(values, offsets, out, out2,
                                   _validated=validated)
        elif self.operation == "reduce":
            values, offsets, out = self.values, self.device_offsets, self.out
            kind, block, plan = self.kind, args.block, self.plan
            schedule = args.schedule

            def step():
                launch_gpu(values, offsets, out, kind, block, plan=plan,
                           schedule=schedule, _validated=validated)
        else:
            values, offsets, out = self.values, self.device_offsets, self.out
            plan, schedule = self.plan, args.schedule

            def step():
                launch_softmax_gpu(values, offsets, out, plan=plan,
                                   schedule=schedule, _validated=validated)
        return step

    def drop_in_call(self):
        """The call a user makes: validates, finds or builds the plan."""
        from swage_b200._segmented_qualification import (
            launch_gpu,
            launch_softmax_gpu,
            launch_sum_max_gpu,
        )

        args = self.args
        if self.operation == "vadd":
            self.step()
        elif self.kind == "sum+max":
            launch_sum_max_gpu(self.values, self.device_offsets, self.out,
                               self.out2)
        elif self.operation == "reduce":
            launch_gpu(self.values, self.device_offsets, self.out, self.kind,
                       args.block, schedule=args.schedule)
        else:
            launch_softmax_gpu(self.values, self.device_offsets, self.out,
                               schedule=args.schedule)

    def launches_per_step(self):
        """Kernels of this library launched by one step."""
        if self.plan is None:
            return 1
        if self.operation == "softmax":
            info = self.plan.describe()
            return sum(1 for n in info["softmax_buckets"] if n > 0)
        info = self.plan.describe()
        schedule = self.args.schedule
        tiles = (schedule in ("split", "persistent", "resident")
                 or (schedule == "auto" and info["schedule"] >= 3))
        # the tile kernel and, when any segment is cut, the merge pass
        return 2 if tiles and info["split_segments"] > 0 else 1

    def parity(self):
        """The device result of one step against the CPU oracle, full size."""
        import torch

        import oracle

        self.step()
        torch.cuda.synchronize()
        if self.plan is not None:
            self.plan.check()
        threads = oracle.host_threads()
        if self.operation == "vadd":
            expected = oracle.vadd_f32(self.x.cpu().numpy(),
                                       self.y.cpu().numpy(), self.count,
                                       threads=threads)
            same = np.array_equal(self.out.cpu().numpy().view(np.uint32),
                                  expected.view(np.uint32))
            return "bit-exact vs x + y" if same else "MISMATCH"
        host_values = self.values.cpu().numpy()
        offsets = self.local_offsets
        if self.operation == "softmax":
            got = self.out.cpu().numpy()
            worst = 0.0
            first = 0
            while first < self.segments:
                last = int(np.searchsorted(
                    offsets, int(offsets[first]) + (1 << 26),
                    side="right")) - 1
                last = min(self.segments, max(last, first + 1))
                a, b = int(offsets[first]), int(offsets[last])
                local = (offsets[first:last + 1] - a).astype(np.int32)
                exact = oracle.segsoftmax_f64(host_values[a:b], local,
                                              threads=threads)
                error = np.abs(got[a:b] - exact)
                if not np.all(error <= 1e-10 + 4e-6 * exact):
                    return f"MISMATCH in segments {first}..{last}"
                seen = exact > 1e-30
                worst = max(worst, float(np.max(error[seen] / exact[seen])))
                first = last
            return (f"every segment within 4e-6 relative of fp64 "
                    f"(worst {worst:.2e})")
        notes = []
        if self.kind == "sum+max":
            outputs = (("sum", self.out), ("max", self.out2))
        else:
            outputs = ((self.kind, self.out),)
        for kind, tensor in outputs:
            result = tensor.cpu().numpy()
            if kind == "max":
                expected = oracle.segreduce_f32(host_values, offsets, "max",
                                                threads=threads)
                same = np.array_equal(result.view(np.uint32),
                                      expected.view(np.uint32))
                if not same:
                    return "MISMATCH (max)"
                notes.append("max bit-exact")
            else:
                exact = oracle.segsum_f64(host_values, offsets,
                                          threads=threads)
                bound = oracle.sum_tolerance(host_values, offsets)
                error = np.abs(result - exact)
                if not np.all(error <= bound):
                    return "MISMATCH (sum)"
                nonempty = bound > 0
                ratio = float(np.max(error[nonempty] / bound[nonempty]))
                notes.append(f"sum within {ratio:.2g} x bound of fp64")
        return ", ".join(notes)

    def close(self):
        if self.plan is not None:
            self.plan.close()
            self.plan = None


_ADD_KERNEL = []


def add_kernel():
    """The reference's example kernel through the public decorator."""
    if not _ADD_KERNEL:
        import swage_b200 as sw
        import swage_b200.language as sl

        @sw.jit
        def kernel(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):
            pid = sl.program_id(0)
            offsets = pid * BLOCK + sl.arange(0, BLOCK)
            mask = offsets < n
            x = sl.load(x_ptr + offsets, mask=mask, other=0.0)
            y = sl.load(y_ptr + offsets, mask=mask, other=0.0)
            sl.store(output_ptr + offsets, x + y, mask=mask)

        _ADD_KERNEL.append(kernel)
    return _ADD_KERNEL[0]


def timed_steps(step, steps, barrier):
    """Device time of ``steps`` calls, nothing else on the stream between."""
    import torch

    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    barrier()
    return start.elapsed_time(stop)


def dominant_kernel_ms(step, launches):
    """Mean duration of the dominant kernel over a separate loop in which the
    library records one pair of events around it per call."""
    import torch

    from swage_b200 import _native

    torch.cuda.synchronize()
    _native.profile_start(launches, 1)
    for _ in range(launches):
        step()
    torch.cuda.synchronize()
    return [float(ms) for ms in _native.profile_stop(launches)]


def l2_flusher(device):
    """Writes a buffer larger than L2 (for workloads that fit in it)."""
    import torch

    scratch = torch.empty(1 << 28, dtype=torch.uint8, device=device)

    def flush():
        scratch.fill_(1)
    return flush


def measure(problem, steps, warmup, barrier, peak):
    """value-style and roofline-style numbers of one resident problem."""
    import torch

    for _ in range(max(3, warmup)):
        problem.step()
    elapsed_ms = timed_steps(problem.step, steps, barrier)
    fits_l2 = problem.bytes_per_step < 3e8
    flush = l2_flusher(problem.device) if fits_l2 else None
    probes = max(5, min(steps, 40))
    if fits_l2:
        # cold: a write larger than L2 before every timed launch
        kernel_ms = []
        for _ in range(probes):
            flush()
            kernel_ms += dominant_kernel_ms(problem.step, 1)
        warm_ms = dominant_kernel_ms(problem.step, probes)
    else:
        kernel_ms = dominant_kernel_ms(problem.step, probes)
        warm_ms = None
    del flush
    torch.cuda.empty_cache()
    mean_ms = float(np.mean(kernel_ms))
    achieved = problem.bytes_per_step / (mean_ms * 1e-3) / 1e9
    result = {
        "elapsed_ms": elapsed_ms,
        "ms_per_step": elapsed_ms / steps,
        "kernel_ms": mean_ms,
        "kernel_launches_timed": len(kernel_ms),
        "achieved_gbs": achieved,
        "frac": achieved / peak,
        "l2": ("fits in L2: kernel timed after a 256 MiB write (cold); "
               "back-to-back steps and kernel_warm_ms are L2-warm")
        if fits_l2 else "inputs larger than L2",
    }
    if warm_ms is not None:
        result["kernel_warm_ms"] = float(np.mean(warm_ms))
    if fits_l2 and problem.kind == "sum+max":
        result["launch_interval_ms"] = launch_interval_ms(problem)
    return result


def launch_interval_ms(problem, launches=200):
    """Device time per launch when the fused sum+max kernel of a small input
    is issued back to back straight through the C ABI (two CUDA events around
    ``launches`` calls, L2-warm).  An event pair around ONE launch of a kernel
    this short measures mostly the events; the interval between launches in a
    saturated stream -- each launch placed while the one before drains -- is
    what a caller issuing many small reductions gets."""
    import torch

    from swage_b200 import _native

    pointers = (problem.values.data_ptr(), problem.device_offsets.data_ptr(),
                problem.out.data_ptr(), problem.out2.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream

    def issue(count):
        for _ in range(count):
            _native.segreduce_sum_max(*pointers, problem.count,
                                      problem.segments, stream)
    issue(20)
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    issue(launches)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / launches


def measure_mapped(problem, check):
    """The same reduction with an element map fused in front of it (sum of
    squares, sum of exponentials), same plan, same bytes: the dominant
    kernel's rate, and -- with ``check`` -- the sum of squares against the
    fp64 sum of the oracle's mapped elements at full size."""
    import torch

    from swage_b200._segmented_qualification import ElementMap, launch_gpu

    if (problem.operation != "reduce" or problem.kind == "sum+max"
            or problem.plan is None):
        return None
    result = {}
    for label, element_map in (("square", ElementMap("square")),
                               ("exp", ElementMap("exp", 0.5, -1.0))):
        def step():
            launch_gpu(problem.values, problem.device_offsets, problem.out,
                       problem.kind, problem.args.block, plan=problem.plan,
                       schedule=problem.args.schedule, extensions=True,
                       map=element_map,
                       _validated=(problem.count, problem.segments))
        for _ in range(3):
            step()
        kernel_ms = float(np.mean(dominant_kernel_ms(step, 10)))
        result[label] = {
            "map": f"{element_map.fn}({element_map.scale:g} * x + "
                   f"{element_map.shift:g})",
            "kernel_ms": kernel_ms,
            "kernel_gbs": problem.bytes_per_step / (kernel_ms * 1e-3) / 1e9,
        }
        if check and label == "square":
            import oracle

            torch.cuda.synchronize()
            got = problem.out.cpu().numpy()[:problem.segments]
            mapped = oracle.map_f32(problem.values.cpu().numpy(), "square")
            offsets = problem.local_offsets
            threads = oracle.host_threads()
            if problem.kind == "sum":
                exact = oracle.segsum_f64(mapped, offsets, threads=threads)
                bound = (oracle.sum_tolerance(mapped, offsets)
                         + 1e-6 * np.abs(exact))
                live = bound > 0
                worst = float(np.max(np.abs(got - exact)[live] / bound[live],
                                     initial=0.0))
                same = bool(np.all(np.abs(got - exact) <= bound))
                verdict = (f"sum of squares within {worst:.3f} x (1e-5 * "
                           "sqrt(len) * max + 1e-6 * sum) of fp64")
            else:
                expected = oracle.segreduce_f32(mapped, offsets, problem.kind,
                                                threads=threads)
                same = bool(np.array_equal(got.view(np.uint32),
                                           expected.view(np.uint32)))
                verdict = f"{problem.kind} of squares bit-exact"
            result[label]["parity"] = verdict if same else "MISMATCH"
            del mapped
    problem.plan.check()
    return result


def measure_vadd_misaligned(device, block):
    """The vector add on views whose three pointers disagree on their phase
    inside a 16-byte line (element offsets 1, 2 and 3): the element-wise
    kernel the library falls back to, against the 256-bit kernel of aligned
    inputs.  CUDA events around twenty launches, inputs larger than L2."""
    import torch

    from swage_b200 import _native

    n = VADD_COUNT
    base = [torch.empty(n + 4, device=device).normal_() for _ in range(2)]
    base.append(torch.empty(n + 4, device=device))
    x, y, out = (tensor[shift:shift + n]
                 for shift, tensor in zip((1, 2, 3), base))
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        _native.vadd(x.data_ptr(), y.data_ptr(), out.data_ptr(), n, block,
                     stream)
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(20):
        _native.vadd(x.data_ptr(), y.data_ptr(), out.data_ptr(), n, block,
                     stream)
    stop.record()
    torch.cuda.synchronize()
    same = bool(torch.equal(out, x + y))
    kernel_ms = start.elapsed_time(stop) / 20
    return {"what": "views at element offsets 1, 2, 3 (scalar kernel)",
            "kernel_us": 1e3 * kernel_ms,
            "kernel_gbs": 12.0 * n / (kernel_ms * 1e-3) / 1e9,
            "parity": "bit-exact vs x + y" if same else "MISMATCH"}


def measure_cold(problem, barrier):
    """The drop-in call on offsets no cache has seen: validation, planning
    and launch, inputs resident on the device.  Fourteen different offsets
    arrays (one boundary moved by one each), wall clock around call + stream
    synchronisation.  The first six calls are this measurement's warm-up and
    are reported apart (``first_calls_ms``): a process's first plans also grow
    the library's memory pool until it holds the plan cache's working set, a
    cost per process, not per call.  ``ms`` is the median of the other eight,
    ``all_ms`` those eight in order."""
    import torch

    if problem.operation == "vadd" or problem.kind == "sum+max":
        return None
    keep = problem.device_offsets
    offsets = problem.local_offsets
    movable = np.nonzero(offsets[1:-1] > offsets[:-2])[0] + 1
    if movable.size < 3:
        return None
    warm_up, timed = 6, 8
    calls = warm_up + timed
    times = []
    picks = [movable[(2 * i + 1) * movable.size // (2 * calls)]
             for i in range(calls)]
    for pick in picks:
        changed = offsets.copy()
        changed[pick] -= 1
        problem.device_offsets = torch.from_numpy(changed).to(problem.device)
        barrier()
        began = time.perf_counter()
        problem.drop_in_call()
        torch.cuda.current_stream().synchronize()
        times.append(1e3 * (time.perf_counter() - began))
    problem.device_offsets = keep
    return {"ms": float(np.median(times[warm_up:])),
            "all_ms": times[warm_up:], "first_calls_ms": times[:warm_up],
            "what": "validate + plan + launch through the drop-in call on "
                    "offsets not seen before, device-resident inputs, wall "
                    "clock to stream completion; the first six calls (also "
                    "growing the memory pool) reported apart"}


def bind_to_gpu_cores(local_rank):
    """Run this rank on the host cores NVML lists as nearest to its GPU, so
    that the pinned staging buffers it allocates and first touches land in
    that socket's memory.  Returns what was done, for the bench line."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = pynvml.nvmlDeviceGetCpuAffinity(
            handle, (os.cpu_count() + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words)
                for b in range(64) if (word >> b) & 1}
        allowed = os.sched_getaffinity(0)
        chosen = sorted(near & allowed)
        if chosen and len(chosen) < len(allowed):
            os.sched_setaffinity(0, chosen)
            return f"bound to {len(chosen)} of {len(allowed)} cores"
        return f"GPU reports all {len(allowed)} cores as near: not bound"
    except Exception as error:  # no NVML: leave the affinity alone
        return f"not bound ({type(error).__name__})"


def measure_e2e(problem, steps, barrier):
    """The drop-in call with host buffers: H2D of the inputs from pinned
    memory, the call, D2H of the result, every step."""
    import torch

    if problem.operation == "vadd":
        sources = [problem.x.cpu().pin_memory(), problem.y.cpu().pin_memory()]
        targets = [problem.x, problem.y]
    else:
        sources = [problem.values.cpu().pin_memory(),
                   torch.from_numpy(problem.local_offsets).pin_memory()]
        targets = [problem.values, problem.device_offsets]
    results = [problem.out]
    if problem.kind == "sum+max":
        results.append(problem.out2)
    host_results = [torch.empty(r.numel(), dtype=torch.float32).pin_memory()
                    for r in results]
    h2d = sum(4 * s.numel() for s in sources)
    d2h = sum(4 * r.numel() for r in results)

    def step():
        for target, source in zip(targets, sources):
            target.copy_(source, non_blocking=True)
        problem.drop_in_call()
        for host, result in zip(host_results, results):
            host.copy_(result, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    step()
    barrier()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    wall = time.perf_counter()
    for _ in range(steps):
        step()
    stop.record()
    barrier()
    ms = max(start.elapsed_time(stop), 1e3 * (time.perf_counter() - wall))
    return ms, h2d, d2h, sources


def measure_h2d_alone(problem, sources, world, rank, barrier):
    """This rank's host-to-device rate with the host to itself: the ranks
    take turns copying their pinned inputs (three rounds each) while the
    others wait at a barrier.  Beside the rates seen when all ranks copy at
    once (the end-to-end steps) it says whether the links are independent or
    the ranks share a host-side limit."""
    import torch

    if problem.operation == "vadd":
        targets = [problem.x, problem.y]
    else:
        targets = [problem.values, problem.device_offsets]
    rate = 0.0
    for turn in range(world):
        barrier()
        if turn == rank:
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(3):
                for target, source in zip(targets, sources):
                    target.copy_(source, non_blocking=True)
            stop.record()
            torch.cuda.current_stream().synchronize()
            copied = 3 * sum(4 * source.numel() for source in sources)
            rate = copied / (start.elapsed_time(stop) * 1e-3) / 1e9
    barrier()
    return rate


def run_ours(args):
    import torch
    import torch.distributed as dist

    from swage_b200 import multi_gpu

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

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value):
        if world == 1:
            return float(value)
        cell = torch.tensor([value], device=device, dtype=torch.float64)
        dist.all_reduce(cell, op=dist.ReduceOp.MAX)
        return float(cell.item())

    peak, peak_source = measured_peak()
    problem = Problem(args.workload, args, world, rank, device, args.shrink)
    problem.build_plans()
    gather = (args.allgather and world > 1 and problem.operation == "reduce"
              and problem.kind != "sum+max")
    if gather:
        plain_step = problem.step

        def step_with_gather():
            plain_step()
            multi_gpu.gather_results(problem.out, problem.cuts)
        problem.step = step_with_gather
    exchange = None
    if (args.peer_results and world > 1 and problem.operation == "reduce"
            and problem.kind != "sum+max"):
        exchange = multi_gpu.PeerResults(problem.cuts)
        kernel_step = problem.step

        def step_with_scatter():
            kernel_step()
            exchange.publish(problem.out)

        def step_fused():
            exchange.reduce(problem.values, problem.device_offsets,
                            problem.kind, problem.plan,
                            schedule=args.schedule)
        problem.step = (step_fused if args.peer_results == "fused"
                        else step_with_scatter)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    numbers = measure(problem, args.steps, args.warmup, barrier, peak)
    elapsed_ms = max_over_ranks(numbers["elapsed_ms"])
    if problem.plan is not None:
        problem.plan.check()
    cold = measure_cold(problem, barrier)
    mapped = None
    if world == 1 and args.shrink == 1:
        mapped = measure_mapped(problem, check=not args.no_parity)
    e2e_steps = args.e2e_steps or max(1, min(args.steps, 5))
    binding = bind_to_gpu_cores(local_rank) if world > 1 else "single rank"
    e2e_ms, h2d, d2h, host_sources = measure_e2e(problem, e2e_steps, barrier)
    h2d_rank_gbs = h2d * e2e_steps / (e2e_ms * 1e-3) / 1e9
    if world > 1:
        rates = torch.zeros(world, device=device, dtype=torch.float64)
        rates[rank] = h2d_rank_gbs
        dist.all_reduce(rates)
        h2d_rank_gbs = [round(float(r), 2) for r in rates.tolist()]
        rates.zero_()
        rates[rank] = measure_h2d_alone(problem, host_sources, world, rank,
                                        barrier)
        dist.all_reduce(rates)
        h2d_alone_gbs = [round(float(r), 2) for r in rates.tolist()]
        together, alone = sum(h2d_rank_gbs), sum(h2d_alone_gbs)
        host_limit = (
            f"all ranks copying at once move {together:.0f} GB/s in total "
            f"against {alone:.0f} GB/s if every link ran at the rate it "
            "reaches alone: "
            + ("the ranks share a host-side limit (memory bandwidth of the "
               "socket that holds the pinned buffers, or shared PCIe root "
               "ports), not their own links"
               if together < 0.8 * alone else
               "the links run independently; a rank is bound by its own link")
        )
    else:
        h2d_alone_gbs = None
        host_limit = ("one rank: bound by its own PCIe link "
                      f"({h2d_rank_gbs:.1f} GB/s over the whole step, copies "
                      "and kernel in sequence)")
    e2e_ms = max_over_ranks(e2e_ms)
    clocks = sampler.stop() if sampler is not None else None
    parity = None
    if world == 1 and not args.no_parity and args.shrink == 1:
        parity = problem.parity()

    # ---- CPU baseline on this host (rank 0, single GPU runs only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle

        oracle.build()
        threads = oracle.host_threads()
        if problem.operation == "vadd":
            sample_offsets = None
            sample_values = (host_sources[0].numpy(), host_sources[1].numpy())
            sample_count = problem.count
        else:
            # bounded sample: a prefix of whole segments, at most 2**29 values
            sample_offsets = cpu_sample(problem.local_offsets, 1 << 29)
            sample_count = int(sample_offsets[-1])
            sample_values = host_sources[0].numpy()[:sample_count]
        single = cpu_pass(problem.operation, problem.kind, sample_values,
                          sample_offsets, 1, args.block)
        cpu_pass(problem.operation, problem.kind, sample_values,
                 sample_offsets, threads, args.block)
        parallel = min(
            cpu_pass(problem.operation, problem.kind, sample_values,
                     sample_offsets, threads, args.block) for _ in range(3))
        cpu = {
            "value": sample_count / parallel / 1e9, "unit": "Gelem/s",
            "cores": threads, "kind": "port",
            "sample": f"{sample_count} of {problem.count} elements, "
                      "best of 3",
            "single_thread_value": sample_count / single / 1e9,
        }
    del host_sources
    launches = problem.launches_per_step() + (
        1 if exchange is not None and args.peer_results == "scatter" else 0)
    summary = {
        "operation": problem.operation, "kind": problem.kind,
        "count": problem.count, "segments": problem.segments,
        "bytes_per_step": problem.bytes_per_step,
        "total_elements": problem.total_elements, "text": problem.text,
        "plan_info": problem.plan_info,
        "config": workload_config(args, problem.text, problem.operation,
                                  problem.kind, problem.full_offsets),
    }
    if exchange is not None:
        exchange.close()
    peer_stores = exchange is not None
    exchange = None
    problem.close()
    del problem
    torch.cuda.empty_cache()

    # ---- the other configurations, same process, 1 GPU only ----
    others = None
    if world == 1 and not args.no_others and args.shrink == 1:
        others = {}
        for name in ALL_WORKLOADS:
            if name == args.workload:
                continue
            other = Problem(name, args, 1, 0, device)
            other.build_plans()
            got = measure(other, min(args.steps, 50), 3, barrier, peak)
            entry = {
                "what": other.text,
                "kernel_us": 1e3 * got["kernel_ms"],
                "kernel_gbs": got["achieved_gbs"],
                "frac_of_measured_copy": got["frac"],
                "pct_of_8tbs": 100.0 * got["achieved_gbs"] / NOMINAL_HBM_GBS,
                "step_us": 1e3 * got["ms_per_step"],
                "step_gbs": other.bytes_per_step
                / (got["ms_per_step"] * 1e-3) / 1e9,
                "step_gelems": other.total_elements
                / (got["ms_per_step"] * 1e-3) / 1e9,
                "l2": got["l2"],
                "schedule": (other.plan.describe()["schedule"]
                             if other.plan is not None else None),
            }
            if "kernel_warm_ms" in got:
                entry["kernel_warm_us"] = 1e3 * got["kernel_warm_ms"]
            if "launch_interval_ms" in got:
                entry["launch_interval_us"] = 1e3 * got["launch_interval_ms"]
            if not args.no_parity:
                entry["parity"] = other.parity()
            others[name] = entry
            other.close()
            del other
            torch.cuda.empty_cache()
            if name == "c2":
                entry["misaligned_views"] = measure_vadd_misaligned(
                    device, args.block)
                torch.cuda.empty_cache()

    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        total = summary["total_elements"]
        bytes_per_step = summary["bytes_per_step"]
        gelems = total / (ms_per_step * 1e-3) / 1e9
        achieved = numbers["achieved_gbs"]
        step_gbs = bytes_per_step / (ms_per_step * 1e-3) / 1e9
        name = args.workload
        line = {
            "metric": metric_name(summary["operation"]), "value": gelems,
            "unit": "Gelem/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": summary["config"],
            "run": {
                "device": "B200", "sample": "whole workload",
                "elements_rank0": summary["count"],
                "segments_rank0": summary["segments"],
                "schedule": args.schedule,
                "sharding": f"{world} element-balanced contiguous segment "
                            "ranges, no collective"
                            + (" + NCCL all-gather of results"
                               if gather else "")
                            + (" + results stored into every rank's copy "
                               "through peer-mapped memory ("
                               + ("by the reducing warps themselves"
                                  if args.peer_results == "fused"
                                  else "one kernel behind the reduction")
                               + ")" if peer_stores else ""),
                "l2": numbers["l2"]},
            "hbm_gbs_per_gpu": step_gbs,
            "pct_of_8tbs_per_gpu": 100.0 * step_gbs / NOMINAL_HBM_GBS,
            "clocks": clocks,
            "e2e": {"value": total / (e2e_ms / e2e_steps * 1e-3) / 1e9,
                    "unit": "Gelem/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps,
                    "h2d_gbs_per_rank": h2d_rank_gbs,
                    "h2d_gbs_per_rank_alone": h2d_alone_gbs,
                    "host_limit": host_limit,
                    "host_cores_rank0": binding},
            "gpu_launches": args.steps * launches,
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak,
                "traffic": (TRAFFIC_RATIO[name] * bytes_per_step
                            if name in TRAFFIC_RATIO and args.shrink == 1
                            else None),
                "traffic_source": "ncu capture of a shrunk case, scaled by "
                                  "algorithmic bytes"
                if name in TRAFFIC_RATIO else None,
                "peak_source": peak_source,
                "kernel_ms": numbers["kernel_ms"],
                "kernel_launches_timed": numbers["kernel_launches_timed"],
                "timed_in": "a separate loop after the value region",
                "algorithmic_bytes_per_launch": bytes_per_step,
                "pct_of_8tbs": 100.0 * achieved / NOMINAL_HBM_GBS,
            },
            "cold": cold,
            "mapped": mapped,
            "parity": parity,
            "cpu_baseline": cpu,
            "plan": summary["plan_info"] or None,
            "workloads": others,
        }
        if cold is not None:
            cold["warm_ms"] = ms_per_step
            cold["cold_over_warm"] = cold["ms"] / ms_per_step
        print(json.dumps(line))
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
