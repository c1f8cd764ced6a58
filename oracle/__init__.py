"""CPU oracle for the segmented-reduction / vector-add path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
module; it is the checker used by the parity tests, by the smoke check and by
the CPU-baseline leg of the benchmark.  Parity status: pinned against the
reference's known answers (see ``swg_oracle.c`` for the list and citations).

Two layers:

* ``swg_oracle.c`` -- the plain-C restatement of the reference's sequential
  lowering (``lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:131-183``),
  compiled by ``oracle/Makefile`` and bound here with ctypes;
* pure-Python loops (``py_segreduce``) for tiny cases, written independently
  of the C file so the two can be checked against each other.

``cpu_oracle(values, offsets, kind)`` has the calling convention of the
reference's ``swage._segmented_qualification.cpu_oracle``
(``python/swage/_segmented_qualification.py:288-329``): CPU float32 values,
CPU int32 offsets, returns a CPU float32 tensor with one result per segment.
"""

import ctypes
import math
import pathlib
import struct
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libswg_oracle.so"
_lib = None

SUM = 0
MAX = 1
MIN = 2  # the dialect's kind<min>; the reference has no lowering for it
_KINDS = {"sum": SUM, "max": MAX, "min": MIN}


def build(force=False):
    """Compile ``swg_oracle.c`` with the committed Makefile."""
    source = _HERE / "swg_oracle.c"
    if (
        not force
        and _LIB_PATH.exists()
        and _LIB_PATH.stat().st_mtime >= source.stat().st_mtime
    ):
        return _LIB_PATH
    subprocess.run(
        ["make", "-C", str(_HERE), "-B", "libswg_oracle.so"],
        check=True,
        capture_output=True,
    )
    return _LIB_PATH


def _load():
    global _lib
    if _lib is not None:
        return _lib
    build()
    lib = ctypes.CDLL(str(_LIB_PATH))
    f32p = ctypes.POINTER(ctypes.c_float)
    f64p = ctypes.POINTER(ctypes.c_double)
    i32p = ctypes.POINTER(ctypes.c_int32)
    i64 = ctypes.c_int64
    lib.swg_oracle_segreduce_f32.argtypes = [
        ctypes.c_int, f32p, i32p, f32p, i64, ctypes.c_int]
    lib.swg_oracle_segreduce_i32.argtypes = [ctypes.c_int, i32p, i32p, i32p,
                                             i64]
    lib.swg_oracle_map_f32.argtypes = [ctypes.c_int, ctypes.c_float,
                                       ctypes.c_float, f32p, f32p, i64]
    lib.swg_oracle_segsum_f64.argtypes = [f32p, i32p, f64p, i64, ctypes.c_int]
    lib.swg_oracle_segabsmax_f64.argtypes = [
        f32p, i32p, f64p, i64, ctypes.c_int]
    lib.swg_oracle_segsoftmax_f64.argtypes = [
        f32p, i32p, f64p, i64, ctypes.c_int]
    lib.swg_oracle_segsoftmax_f32.argtypes = [
        f32p, i32p, f32p, i64, ctypes.c_int]
    lib.swg_oracle_vadd_f32.argtypes = [f32p, f32p, f32p, i64, i64,
                                        ctypes.c_int]
    for name in (
        "swg_oracle_segreduce_f32", "swg_oracle_segreduce_i32",
        "swg_oracle_segsum_f64", "swg_oracle_map_f32",
        "swg_oracle_segabsmax_f64", "swg_oracle_segsoftmax_f64",
        "swg_oracle_segsoftmax_f32", "swg_oracle_vadd_f32",
        "swg_oracle_max_threads",
    ):
        getattr(lib, name).restype = ctypes.c_int
    _lib = lib
    return lib


def max_threads():
    """Host threads OpenMP would use by default on this machine."""
    return int(_load().swg_oracle_max_threads())


def host_threads():
    """Host cores this process may run on.

    Unlike ``max_threads`` this ignores ``OMP_NUM_THREADS``, which launchers
    such as ``torch.distributed.run`` set to 1 for every rank: the timed CPU
    baseline asks for the cores the machine really offers.
    """
    import os

    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return max(1, os.cpu_count() or 1)


def _f32(array):
    array = np.ascontiguousarray(array, dtype=np.float32)
    return array, array.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _i32(array):
    array = np.ascontiguousarray(array, dtype=np.int32)
    return array, array.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))


def _check_offsets(offsets, value_count):
    if offsets.ndim != 1 or offsets.size < 1:
        raise ValueError("offsets must contain at least the initial zero")
    if offsets[0] != 0 or np.any(np.diff(offsets.astype(np.int64)) < 0):
        raise ValueError("offsets must start at zero and be nondecreasing")
    if int(offsets[-1]) > value_count:
        raise ValueError("final offset exceeds value count")


def segreduce_f32(values, offsets, kind, threads=1):
    """Sequential fp32 segmented sum/max (the reference's CPU arithmetic)."""
    values, vp = _f32(values)
    offsets, op = _i32(offsets)
    _check_offsets(offsets, values.size)
    out = np.empty(offsets.size - 1, dtype=np.float32)
    used = _load().swg_oracle_segreduce_f32(
        _KINDS[kind], vp, op,
        out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
        out.size, int(threads))
    if used < 0:
        raise ValueError("reduction kind must be 'sum' or 'max'")
    return out


def segreduce_i32(values, offsets, kind):
    """Sequential int32 segmented sum (wrap-around) / max / min."""
    values, vp = _i32(values)
    offsets, op = _i32(offsets)
    _check_offsets(offsets, values.size)
    out = np.empty(offsets.size - 1, dtype=np.int32)
    used = _load().swg_oracle_segreduce_i32(
        _KINDS[kind], vp, op,
        out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), out.size)
    if used < 0:
        raise ValueError("reduction kind must be 'sum', 'max' or 'min'")
    return out


_MAPS = {"identity": 0, "abs": 1, "square": 2, "exp": 3}


def map_f32(values, fn="identity", scale=1.0, shift=0.0):
    """``fn(scale * x + shift)`` element by element in fp32 (product and sum
    rounded separately; ``exp`` evaluated in double, rounded once): what an
    element map in front of a reduction feeds it."""
    values, vp = _f32(values)
    out = np.empty(values.size, dtype=np.float32)
    used = _load().swg_oracle_map_f32(
        _MAPS[fn], float(scale), float(shift), vp,
        out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), values.size)
    if used < 0:
        raise ValueError("unknown map function")
    return out


def segsum_f64(values, offsets, threads=0):
    """fp64 accumulation per segment: the anchor of the sum tolerance."""
    values, vp = _f32(values)
    offsets, op = _i32(offsets)
    _check_offsets(offsets, values.size)
    out = np.empty(offsets.size - 1, dtype=np.float64)
    _load().swg_oracle_segsum_f64(
        vp, op, out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)),
        out.size, int(threads) or max_threads())
    return out


def segabsmax_f64(values, offsets, threads=0):
    """max|x| per segment (0 when empty)."""
    values, vp = _f32(values)
    offsets, op = _i32(offsets)
    _check_offsets(offsets, values.size)
    out = np.empty(offsets.size - 1, dtype=np.float64)
    _load().swg_oracle_segabsmax_f64(
        vp, op, out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)),
        out.size, int(threads) or max_threads())
    return out


def segsoftmax_f64(values, offsets, threads=0):
    """fp64 softmax per segment; positions outside every segment stay NaN."""
    values, vp = _f32(values)
    offsets, op = _i32(offsets)
    _check_offsets(offsets, values.size)
    out = np.full(values.size, np.nan, dtype=np.float64)
    _load().swg_oracle_segsoftmax_f64(
        vp, op, out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)),
        offsets.size - 1, int(threads) or max_threads())
    return out


def segsoftmax_f32(values, offsets, threads=1):
    """Sequential fp32 softmax (max, sum of exp, divide) per segment."""
    values, vp = _f32(values)
    offsets, op = _i32(offsets)
    _check_offsets(offsets, values.size)
    out = np.full(values.size, np.nan, dtype=np.float32)
    _load().swg_oracle_segsoftmax_f32(
        vp, op, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
        offsets.size - 1, int(threads))
    return out


def vadd_f32(x, y, n=None, block=128, threads=1):
    """out[i] = x[i] + y[i] for i < n, walked block by block."""
    x, xp = _f32(x)
    y, yp = _f32(y)
    n = min(x.size, y.size) if n is None else int(n)
    out = np.zeros(n, dtype=np.float32)
    status = _load().swg_oracle_vadd_f32(
        xp, yp, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
        n, int(block), int(threads))
    if status < 0:
        raise ValueError("block must be positive")
    return out


def sum_tolerance(values, offsets):
    """Per-segment bound 1e-5 * sqrt(len) * max|x| on |fp32 sum - fp64 sum|."""
    offsets = np.asarray(offsets, dtype=np.int64)
    lengths = np.diff(offsets).astype(np.float64)
    return 1e-5 * np.sqrt(lengths) * segabsmax_f64(values, offsets)


# --- pure-Python restatement, for tiny cases only -------------------------

def _round_f32(value):
    return struct.unpack("<f", struct.pack("<f", value))[0]


def _py_maximumf(a, b):
    if math.isnan(a) or math.isnan(b):
        return math.nan
    if a > b:
        return a
    if b > a:
        return b
    return b if math.copysign(1.0, a) < 0 else a


def py_segreduce(values, offsets, kind):
    """Loop-for-loop Python form of buildSequentialReduction (small inputs).

    Each fp32 add is emulated by rounding the double sum of two float32
    numbers back to float32, which is exact for a single addition.
    """
    values = [float(v) for v in np.asarray(values, dtype=np.float32)]
    offsets = [int(o) for o in offsets]
    out = []
    for sid in range(len(offsets) - 1):
        if kind == "sum":
            acc = 0.0
            for i in range(offsets[sid], offsets[sid + 1]):
                acc = _round_f32(acc + values[i])
        elif kind == "max":
            acc = -math.inf
            for i in range(offsets[sid], offsets[sid + 1]):
                acc = _py_maximumf(acc, values[i])
        elif kind == "min":
            acc = math.inf
            for i in range(offsets[sid], offsets[sid + 1]):
                acc = -_py_maximumf(-acc, -values[i])
        else:
            raise ValueError("reduction kind must be 'sum' or 'max'")
        out.append(acc)
    return np.asarray(out, dtype=np.float32)


def cpu_oracle(values, offsets, kind):
    """Reference-shaped entry: torch CPU tensors in, torch CPU tensor out."""
    import torch

    if kind not in ("sum", "max"):
        raise ValueError("reduction kind must be 'sum' or 'max'")
    result = segreduce_f32(
        values.detach().cpu().numpy(), offsets.detach().cpu().numpy(), kind)
    return torch.from_numpy(result)


__all__ = [
    "build", "cpu_oracle", "host_threads", "max_threads", "py_segreduce", "segabsmax_f64",
    "segreduce_f32", "segreduce_i32", "segsoftmax_f32", "segsoftmax_f64", "segsum_f64",
    "sum_tolerance", "vadd_f32",
]
