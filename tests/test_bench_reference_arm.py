"""The reference arm of ``bench.py`` (the CPU restatement of the reference's
sequential lowering, timed on the host cores) keeps the bench's line contract.
Runs without a GPU on a 64x shrunk workload."""

import json
import os
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parent.parent
COMMAND = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference",
           "--shrink", "64", "--steps", "2", "--warmup", "1"]


def run(extra_environment=None):
    environment = dict(os.environ)
    for name in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        environment.pop(name, None)
    environment.update(extra_environment or {})
    return subprocess.run(COMMAND, cwd=ROOT, env=environment, text=True,
                          capture_output=True, timeout=600)


def test_reference_arm_prints_one_line_with_the_contract_keys():
    done = run({"OMP_NUM_THREADS": "1"})  # what torchrun exports
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "segmented_reduce_throughput"
    assert line["unit"] == "Gelem/s" and line["higher_is_better"] is True
    assert line["steps"] == 2 and line["warmup"] == 1 and line["n_gpus"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["dtype"] == "f32" and line["data"] == "synthetic"
    assert line["config"]["workload"].startswith("c5")
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["value"] == line["value"]
    # every core the process may use, whatever OMP_NUM_THREADS a launcher set
    assert baseline["cores"] == len(os.sched_getaffinity(0))
    assert line["e2e"] == {"value": line["value"], "unit": "Gelem/s",
                           "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_other_ranks_of_a_multi_rank_launch_print_nothing():
    done = run({"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.strip() == ""
