"""Builds ``libswage_b200.so`` (CUDA kernels + C ABI) in-tree with nvcc.

Only sm_100a code is generated.  Run as ``python -m swage_b200._build`` or call
``build_library()``; the shared object lands next to this file so it is the
one ``swage_b200._native`` loads.
"""

import pathlib
import shutil
import subprocess
import sys

PACKAGE = pathlib.Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libswage_b200.so"

SOURCES = (
    "swg_api.cu",
    "swg_vadd.cu",
    "swg_segreduce.cu",
    "swg_softmax.cu",
    "swg_device_plan.cu",
    "swg_exchange.cu",
    "swg_planner.cpp",
)

NVCC_FLAGS = (
    "-O3",
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
)


def _nvcc():
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(found).exists():
        raise RuntimeError("nvcc not found; cannot build libswage_b200.so")
    return found


def _stale():
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = list(CSRC.iterdir()) + [ROOT / "include" / "swage_b200.h"]
    return any(path.stat().st_mtime > built for path in inputs)


def build_library(force=False, verbose=False):
    """Compile every source for sm_100a and link the shared library."""
    if not force and not _stale():
        return LIBRARY
    # linked under a temporary name and renamed, so that a reader never sees
    # a half-written library
    fresh = LIBRARY.with_suffix(".so.new")
    command = [_nvcc(), *NVCC_FLAGS, "-shared",
               "-I", str(ROOT / "include"), "-I", str(CSRC),
               "-o", str(fresh)]
    if verbose:
        command += ["-Xptxas", "-v"]
    command += [str(CSRC / name) for name in SOURCES]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        fresh.unlink(missing_ok=True)
        raise RuntimeError(
            "nvcc failed:\n" + result.stdout + "\n" + result.stderr
        )
    fresh.replace(LIBRARY)
    if verbose:
        sys.stderr.write(result.stderr)
    return LIBRARY


if __name__ == "__main__":
    print(build_library(force=True, verbose="-v" in sys.argv))
