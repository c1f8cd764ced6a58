"""ctypes binding of ``libswage_b200.so`` (the C ABI in ``include/swage_b200.h``).

This takes the place of the reference's ``_CudaDriver`` ctypes wrapper
(``python/swage/_runtime.py:399-531``) and of its nanobind codegen module
(``python/SwageExtensionNanobind.cpp:27-99``): instead of compiling PTX and
calling ``cuLaunchKernel``, the Python layer calls prebuilt sm_100a kernels
through plain C functions.

There is no CPU fallback.  If the shared library is missing the loader raises
``RuntimeError`` -- it does not try to build it, and nothing else in the
package computes results on the host.
"""

import ctypes
import pathlib
import threading

LIBRARY_PATH = pathlib.Path(__file__).resolve().parent / "libswage_b200.so"

# mirrors of the header's constants
KIND_SUM, KIND_MAX, KIND_MIN = 0, 1, 2
DTYPE_F32, DTYPE_F16, DTYPE_BF16, DTYPE_I32 = range(4)
MAP_IDENTITY, MAP_ABS, MAP_SQUARE, MAP_EXP = range(4)
MAPS = {"identity": MAP_IDENTITY, "abs": MAP_ABS, "square": MAP_SQUARE,
        "exp": MAP_EXP}


class Map(ctypes.Structure):
    """``swg_map``: ``fn(scale * x + shift)`` applied before the reduction."""

    _fields_ = [("fn", ctypes.c_int32), ("scale", ctypes.c_float),
                ("shift", ctypes.c_float)]

OP_REDUCE, OP_SOFTMAX = 0, 1
(SCHED_AUTO, SCHED_WARP, SCHED_CTA, SCHED_SPLIT, SCHED_PERSISTENT,
 SCHED_RESIDENT) = range(6)
SCHEDULES = {
    "auto": SCHED_AUTO,
    "warp": SCHED_WARP,
    "cta": SCHED_CTA,
    "split": SCHED_SPLIT,
    "persistent": SCHED_PERSISTENT,
    "resident": SCHED_RESIDENT,
}
OFFSETS_REASONS = (
    "ok", "empty", "count_range", "output_small", "nonzero_start",
    "negative", "decreasing", "exceeds_values",
)

EXPORTS = (
    "swg_last_error", "swg_status_name", "swg_abi_version", "swg_vadd_f32",
    "swg_validate_offsets_i32", "swg_plan_create", "swg_plan_destroy",
    "swg_plan_describe", "swg_plan_status", "swg_plan_host_tasks",
    "swg_segreduce_f32",
    "swg_segsoftmax_f32", "swg_shard_offsets", "swg_profile_start",
    "swg_profile_stop", "swg_segreduce_f32_noalloc",
    "swg_validate_offsets_device", "swg_plan_create_device",
    "swg_segreduce_sum_max_f32", "swg_plan_create_validated",
    "swg_plan_peek_status", "swg_segreduce", "swg_plan_selftest_timeout",
    "swg_segreduce_map", "swg_scatter_results_f32", "swg_peer_buffer_create",
    "swg_peer_buffer_open", "swg_peer_buffer_close", "swg_peer_buffer_destroy",
    "swg_segreduce_peers_f32",
)

_lock = threading.Lock()
_library = None


def _declare(lib):
    c_int, c_i32, c_i64 = ctypes.c_int, ctypes.c_int32, ctypes.c_int64
    ptr = ctypes.c_void_p
    lib.swg_last_error.restype = ctypes.c_char_p
    lib.swg_last_error.argtypes = []
    lib.swg_status_name.restype = ctypes.c_char_p
    lib.swg_status_name.argtypes = [c_int]
    lib.swg_abi_version.restype = c_int
    lib.swg_abi_version.argtypes = []
    lib.swg_vadd_f32.restype = c_int
    lib.swg_vadd_f32.argtypes = [ptr, ptr, ptr, c_i32, c_i32, ptr]
    lib.swg_validate_offsets_i32.restype = c_int
    lib.swg_validate_offsets_i32.argtypes = [
        ptr, c_i64, c_i64, c_i64,
        ctypes.POINTER(c_i32), ctypes.POINTER(c_i64)]
    lib.swg_plan_create.restype = c_int
    lib.swg_plan_create.argtypes = [
        ptr, c_i32, c_i32, c_int, ctypes.POINTER(ptr)]
    lib.swg_plan_destroy.restype = c_int
    lib.swg_plan_destroy.argtypes = [ptr]
    lib.swg_plan_describe.restype = c_int
    lib.swg_plan_describe.argtypes = [ptr, ctypes.c_char_p, ctypes.c_size_t]
    lib.swg_plan_status.restype = c_int
    lib.swg_plan_status.argtypes = [ptr]
    lib.swg_plan_host_tasks.restype = c_int
    lib.swg_plan_host_tasks.argtypes = [
        ptr, c_i32, c_int, ptr, c_i64, ctypes.POINTER(c_i64),
        ctypes.c_char_p, ctypes.c_size_t]
    lib.swg_segreduce_f32.restype = c_int
    lib.swg_segreduce_f32.argtypes = [
        c_int, ptr, ptr, ptr, c_i32, c_i32, ptr, c_int, c_i32, ptr]
    lib.swg_segreduce.restype = c_int
    lib.swg_segreduce.argtypes = [
        c_int, c_int, ptr, ptr, ptr, c_i32, c_i32, ptr, c_int, c_i32, ptr]
    lib.swg_segreduce_map.restype = c_int
    lib.swg_segreduce_map.argtypes = [
        c_int, c_int, ctypes.POINTER(Map), ptr, ptr, ptr, c_i32, c_i32, ptr,
        c_int, c_i32, ptr]
    lib.swg_peer_buffer_create.restype = c_int
    lib.swg_peer_buffer_create.argtypes = [
        c_i64, ctypes.POINTER(ptr), ctypes.c_char_p]
    lib.swg_peer_buffer_open.restype = c_int
    lib.swg_peer_buffer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ptr)]
    lib.swg_peer_buffer_close.restype = c_int
    lib.swg_peer_buffer_close.argtypes = [ptr]
    lib.swg_peer_buffer_destroy.restype = c_int
    lib.swg_peer_buffer_destroy.argtypes = [ptr]
    lib.swg_segreduce_peers_f32.restype = c_int
    lib.swg_segreduce_peers_f32.argtypes = [
        c_int, ptr, ptr, ctypes.POINTER(ptr), c_i32, c_i64, c_i32, c_i32, ptr,
        c_int, ptr]
    lib.swg_scatter_results_f32.restype = c_int
    lib.swg_scatter_results_f32.argtypes = [
        ptr, c_i64, ctypes.POINTER(ptr), c_i32, c_i64, ptr]
    lib.swg_segsoftmax_f32.restype = c_int
    lib.swg_segsoftmax_f32.argtypes = [
        ptr, ptr, ptr, c_i32, c_i32, ptr, c_int, ptr]
    lib.swg_shard_offsets.restype = c_int
    lib.swg_shard_offsets.argtypes = [ptr, c_i32, c_i32, ptr]
    lib.swg_segreduce_sum_max_f32.restype = c_int
    lib.swg_segreduce_sum_max_f32.argtypes = [
        ptr, ptr, ptr, ptr, c_i32, c_i32, ptr]
    lib.swg_segreduce_f32_noalloc.restype = c_int
    lib.swg_segreduce_f32_noalloc.argtypes = [
        c_int, ptr, ptr, ptr, c_i32, c_i32, ptr]
    lib.swg_validate_offsets_device.restype = c_int
    lib.swg_validate_offsets_device.argtypes = [
        ptr, c_i32, c_i32, c_i64, ptr,
        ctypes.POINTER(c_i32), ctypes.POINTER(c_i64),
        ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(c_i32)]
    lib.swg_plan_create_device.restype = c_int
    lib.swg_plan_create_device.argtypes = [
        ptr, c_i32, c_i32, c_i64, c_int, ptr, ctypes.POINTER(ptr),
        ctypes.POINTER(c_i32), ctypes.POINTER(c_i64)]
    lib.swg_plan_create_validated.restype = c_int
    lib.swg_plan_create_validated.argtypes = [
        ptr, c_i32, c_i32, c_int, ptr, ctypes.c_uint64, ctypes.POINTER(ptr)]
    lib.swg_plan_selftest_timeout.restype = c_int
    lib.swg_plan_selftest_timeout.argtypes = [ptr, c_i32, ptr]
    lib.swg_plan_peek_status.restype = c_int
    lib.swg_plan_peek_status.argtypes = [ptr]
    lib.swg_profile_start.restype = c_int
    lib.swg_profile_start.argtypes = [c_i32, c_i32]
    lib.swg_profile_stop.restype = c_int
    lib.swg_profile_stop.argtypes = [ptr, c_i32, ctypes.POINTER(c_i32)]


def library():
    """Load the shared library once; fail loudly when it is absent."""
    global _library
    with _lock:
        if _library is None:
            if not LIBRARY_PATH.exists():
                raise RuntimeError(
                    f"{LIBRARY_PATH} is missing: build it with "
                    "'python -m swage_b200._build'. There is no CPU fallback."
                )
            lib = ctypes.CDLL(str(LIBRARY_PATH))
            _declare(lib)
            _library = lib
        return _library


def check(status, function_name):
    """Raise in the reference's driver-error style (``_runtime.py:452-469``)."""
    if status == 0:
        return
    lib = library()
    name = lib.swg_status_name(status).decode()
    text = (lib.swg_last_error() or b"").decode() or "unknown"
    raise RuntimeError(f"{function_name} failed: {name} ({status}): {text}")


def vadd(x_ptr, y_ptr, out_ptr, n, block, stream):
    check(library().swg_vadd_f32(x_ptr, y_ptr, out_ptr, n, block, stream),
          "swg_vadd_f32")


def segreduce(kind, values_ptr, offsets_ptr, out_ptr, value_count,
              segment_count, plan_handle, schedule, block, stream):
    check(
        library().swg_segreduce_f32(
            kind, values_ptr, offsets_ptr, out_ptr, value_count,
            segment_count, plan_handle, schedule, block, stream),
        "swg_segreduce_f32",
    )


def segreduce_typed(kind, dtype, values_ptr, offsets_ptr, out_ptr, value_count,
                    segment_count, plan_handle, schedule, block, stream):
    """``segreduce`` for f16 / bf16 / i32 values (``dtype``: ``DTYPE_*``)."""
    check(
        library().swg_segreduce(
            kind, dtype, values_ptr, offsets_ptr, out_ptr, value_count,
            segment_count, plan_handle, schedule, block, stream),
        "swg_segreduce",
    )


def segreduce_map(kind, dtype, fn, scale, shift, values_ptr, offsets_ptr,
                  out_ptr, value_count, segment_count, plan_handle, schedule,
                  block, stream):
    """Reduce ``fn(scale * x + shift)`` over every segment (``fn``: ``MAP_*``,
    ``dtype`` a floating ``DTYPE_*``; fp32 results)."""
    element_map = Map(fn, scale, shift)
    check(
        library().swg_segreduce_map(
            kind, dtype, ctypes.byref(element_map), values_ptr, offsets_ptr,
            out_ptr, value_count, segment_count, plan_handle, schedule, block,
            stream),
        "swg_segreduce_map",
    )


PEER_HANDLE_BYTES = 64


def peer_buffer_create(byte_count):
    """A device buffer other processes can map: ``(pointer, handle bytes)``."""
    pointer = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(PEER_HANDLE_BYTES)
    check(library().swg_peer_buffer_create(byte_count, ctypes.byref(pointer),
                                           handle),
          "swg_peer_buffer_create")
    return pointer.value, handle.raw


def peer_buffer_open(handle):
    """Map a peer's buffer into the current device's address space."""
    if len(handle) != PEER_HANDLE_BYTES:
        raise ValueError("a peer buffer handle has 64 bytes")
    pointer = ctypes.c_void_p()
    check(library().swg_peer_buffer_open(handle, ctypes.byref(pointer)),
          "swg_peer_buffer_open")
    return pointer.value


def peer_buffer_close(pointer):
    check(library().swg_peer_buffer_close(pointer), "swg_peer_buffer_close")


def peer_buffer_destroy(pointer):
    check(library().swg_peer_buffer_destroy(pointer),
          "swg_peer_buffer_destroy")


def segreduce_peers(kind, values_ptr, offsets_ptr, destination_ptrs, offset,
                    value_count, segment_count, plan_handle, schedule, stream):
    """``segreduce`` with a plan whose results go to ``destination[p][offset +
    s]`` for every destination pointer instead of a local output."""
    bases = (ctypes.c_void_p * len(destination_ptrs))(*destination_ptrs)
    check(
        library().swg_segreduce_peers_f32(
            kind, values_ptr, offsets_ptr, bases, len(destination_ptrs),
            offset, value_count, segment_count, plan_handle, schedule,
            stream),
        "swg_segreduce_peers_f32",
    )


def scatter_results(src_ptr, count, destination_ptrs, offset, stream):
    """``destination[p][offset + i] = src[i]`` for every destination pointer
    (device memory of this GPU or peer-mapped memory of another)."""
    bases = (ctypes.c_void_p * len(destination_ptrs))(*destination_ptrs)
    check(
        library().swg_scatter_results_f32(
            src_ptr, count, bases, len(destination_ptrs), offset, stream),
        "swg_scatter_results_f32",
    )


def segreduce_sum_max(values_ptr, offsets_ptr, sum_ptr, max_ptr, value_count,
                      segment_count, stream):
    """Sum and max of every segment in one pass (one launch, no plan)."""
    check(
        library().swg_segreduce_sum_max_f32(
            values_ptr, offsets_ptr, sum_ptr, max_ptr, value_count,
            segment_count, stream),
        "swg_segreduce_sum_max_f32",
    )


def segreduce_noalloc(kind, values_ptr, host_offsets_ptr, out_ptr, value_count,
                      segment_count, stream):
    """Split-schedule reduce that allocates no device memory.

    For callers that cannot call cudaMalloc (their framework's pool owns the
    memory, or an allocation's implicit synchronisation is not acceptable).
    The offsets pointer is a HOST pointer; the plan is built per call and its
    data lives in a fixed array inside the library.  Calls must not overlap on
    the GPU; inputs beyond the array's limits raise ``RuntimeError``.
    """
    check(
        library().swg_segreduce_f32_noalloc(
            kind, values_ptr, host_offsets_ptr, out_ptr, value_count,
            segment_count, stream),
        "swg_segreduce_f32_noalloc",
    )


def segsoftmax(values_ptr, offsets_ptr, out_ptr, value_count, segment_count,
               plan_handle, schedule, stream):
    check(
        library().swg_segsoftmax_f32(
            values_ptr, offsets_ptr, out_ptr, value_count, segment_count,
            plan_handle, schedule, stream),
        "swg_segsoftmax_f32",
    )


def validate_offsets(host_ptr, count, value_count, output_count):
    """Return ``(reason_name, index)``; ``("ok", -1)`` when the array is fine."""
    reason = ctypes.c_int32(0)
    index = ctypes.c_int64(-1)
    library().swg_validate_offsets_i32(
        host_ptr, count, value_count, output_count,
        ctypes.byref(reason), ctypes.byref(index))
    return OFFSETS_REASONS[reason.value], index.value


_INVALID_OFFSETS = 2  # SWG_ERR_INVALID_OFFSETS


def validate_offsets_device(device_ptr, segment_count, value_count,
                            output_count, stream):
    """Validate offsets that live on the GPU.

    Returns ``(reason_name, index, content_hash, last_offset)``; synchronises
    ``stream`` to read the verdict.
    """
    reason = ctypes.c_int32(0)
    index = ctypes.c_int64(-1)
    digest = ctypes.c_uint64(0)
    last = ctypes.c_int32(0)
    status = library().swg_validate_offsets_device(
        device_ptr, segment_count, value_count, output_count, stream,
        ctypes.byref(reason), ctypes.byref(index), ctypes.byref(digest),
        ctypes.byref(last))
    if status not in (0, _INVALID_OFFSETS):
        check(status, "swg_validate_offsets_device")
    return OFFSETS_REASONS[reason.value], index.value, digest.value, last.value


def plan_create_device(device_ptr, segment_count, value_count, output_count,
                       op, stream):
    """Validate and plan on the GPU; ``(handle, "ok", -1)`` or
    ``(None, reason_name, index)`` for offsets that break a rule."""
    handle = ctypes.c_void_p()
    reason = ctypes.c_int32(0)
    index = ctypes.c_int64(-1)
    status = library().swg_plan_create_device(
        device_ptr, segment_count, value_count, output_count, op, stream,
        ctypes.byref(handle), ctypes.byref(reason), ctypes.byref(index))
    if status == _INVALID_OFFSETS:
        return None, OFFSETS_REASONS[reason.value], index.value
    check(status, "swg_plan_create_device")
    return handle, "ok", -1


def plan_create_validated(device_ptr, segment_count, value_count, op, stream,
                          digest):
    """Plan on the GPU from offsets ``validate_offsets_device`` has just
    accepted (it returned ``digest``): no second pass, no synchronisation."""
    handle = ctypes.c_void_p()
    check(
        library().swg_plan_create_validated(
            device_ptr, segment_count, value_count, op, stream, digest,
            ctypes.byref(handle)),
        "swg_plan_create_validated",
    )
    return handle


def plan_create(host_ptr, segment_count, value_count, op):
    handle = ctypes.c_void_p()
    check(
        library().swg_plan_create(
            host_ptr, segment_count, value_count, op, ctypes.byref(handle)),
        "swg_plan_create",
    )
    return handle


def plan_destroy(handle):
    library().swg_plan_destroy(handle)


def plan_describe(handle):
    buffer = ctypes.create_string_buffer(8192)
    check(library().swg_plan_describe(handle, buffer, len(buffer)),
          "swg_plan_describe")
    return buffer.value.decode()


def plan_host_tasks(host_ptr, segment_count, op=OP_REDUCE):
    """Run the planner on the host only; return ``(tasks, description)``.

    ``tasks`` is a list of ``(segment, count_or_slot, value_begin,
    value_count, kind, head_slot, tail_slot, link_first, link_pieces)``
    tuples (the last two: where the partial slots of the cut segment a piece
    belongs to begin, and how many pieces it has).
    """
    import json

    lib = library()
    total = ctypes.c_int64(0)
    text = ctypes.create_string_buffer(8192)
    check(lib.swg_plan_host_tasks(host_ptr, segment_count, op, None, 0,
                                  ctypes.byref(total), text, len(text)),
          "swg_plan_host_tasks")
    words = (ctypes.c_int32 * (8 * max(total.value, 1)))()
    check(lib.swg_plan_host_tasks(host_ptr, segment_count, op, words,
                                  total.value, ctypes.byref(total), None, 0),
          "swg_plan_host_tasks")
    tasks = []
    for t in range(total.value):
        (seg, count, vbegin, packed, head, tail, link_first,
         link_pieces) = words[8 * t:8 * t + 8]
        packed &= 0xFFFFFFFF
        tasks.append((seg, count, vbegin, packed & ((1 << 28) - 1),
                      packed >> 28, head, tail, link_first, link_pieces))
    return tasks, json.loads(text.value.decode())


def plan_status(handle):
    check(library().swg_plan_status(handle), "swg_plan_status")


def plan_selftest_timeout(handle, limit_us, stream):
    """Queue a kernel whose bounded wait runs out after ``limit_us`` and
    reports it through the plan's error words."""
    check(library().swg_plan_selftest_timeout(handle, limit_us, stream),
          "swg_plan_selftest_timeout")


def plan_peek_status(handle):
    """Raise for an error a FINISHED launch of the plan left behind; no CUDA
    call, no synchronisation."""
    status = library().swg_plan_peek_status(handle)
    if status:
        check(status, "swg_plan_peek_status")


def shard_offsets(host_ptr, segment_count, shards):
    cuts = (ctypes.c_int32 * (shards + 1))()
    check(library().swg_shard_offsets(host_ptr, segment_count, shards, cuts),
          "swg_shard_offsets")
    return list(cuts)


def profile_start(capacity, stride=1):
    check(library().swg_profile_start(capacity, stride), "swg_profile_start")


def profile_stop(capacity):
    """Durations (ms) of the dominant kernel of each call since the start."""
    buffer = (ctypes.c_float * max(capacity, 1))()
    count = ctypes.c_int32(0)
    check(library().swg_profile_stop(buffer, capacity, ctypes.byref(count)),
          "swg_profile_stop")
    return [buffer[i] for i in range(min(count.value, capacity))]
