"""Environment diagnostics (counterpart of the reference's ``python -m
swage.env``, ``python/swage/env.py:60-78``).

    python -m swage_b200.env

prints one ``key: value`` line per field.  The report never fails: what is
unavailable is reported as such.  The ``backends`` field is truthful: the
sm_100a library is "available" only when the shared object is built, loads,
and a CUDA device of compute capability 10.x is visible; there is no other
backend and no CPU fallback.
"""

import ctypes
import importlib.util
import platform
import sys


def driver_version():
    """CUDA driver version as ``"major.minor"``; None without a driver."""
    try:
        cuda = ctypes.CDLL("libcuda.so.1")
        version = ctypes.c_int(0)
        if cuda.cuDriverGetVersion(ctypes.byref(version)) != 0:
            return None
        return f"{version.value // 1000}.{(version.value % 1000) // 10}"
    except OSError:
        return None


def _torch_info():
    info = {"torch": None, "torch_cuda_build": None, "cuda_driver": None,
            "cuda": False, "gpu": None}
    if importlib.util.find_spec("torch") is None:
        return info
    import torch

    info["torch"] = torch.__version__
    info["torch_cuda_build"] = torch.version.cuda
    info["cuda"] = bool(torch.cuda.is_available())
    if info["cuda"]:
        info["cuda_driver"] = driver_version()
        major, minor = torch.cuda.get_device_capability()
        info["gpu"] = {
            "name": torch.cuda.get_device_name(),
            "compute_capability": f"{major}.{minor}",
        }
    return info


def _library_info():
    """State of the native library without raising."""
    from . import _native

    if not _native.LIBRARY_PATH.exists():
        return None, "not built (python -m swage_b200._build)"
    try:
        version = _native.library().swg_abi_version()
    except (OSError, RuntimeError, AttributeError) as error:
        return None, f"does not load ({error})"
    return version, f"{_native.LIBRARY_PATH.name}, ABI {version}"


def report():
    """The environment report as a dictionary."""
    from . import __version__

    info = _torch_info()
    abi, library = _library_info()
    if abi is None:
        backend = f"unavailable (library {library})"
    elif not info["cuda"]:
        backend = "unavailable (no CUDA device visible to PyTorch)"
    elif not info["gpu"]["compute_capability"].startswith("10."):
        backend = ("unavailable (the library holds sm_100a code only; device "
                   f"is {info['gpu']['compute_capability']})")
    else:
        backend = f"available ({library})"
    return {
        "swage_b200": __version__,
        "python": sys.version.split()[0],
        "platform": platform.platform(),
        "torch": info["torch"],
        "torch_cuda_build": info["torch_cuda_build"],
        "cuda_driver": info["cuda_driver"],
        "cuda": info["cuda"],
        "gpu": info["gpu"],
        "library": library,
        "backends": {
            "cuda_sm100a": backend,
            "cpu": "none (there is no CPU fallback; the CPU oracle is test "
                   "infrastructure outside this package)",
        },
    }


def main():
    for key, value in report().items():
        print(f"{key}: {value}")


if __name__ == "__main__":
    main()
