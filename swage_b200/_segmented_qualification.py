"""Segmented sum / max / softmax runner (drop-in for the reference's internal
``python/swage/_segmented_qualification.py``).

Same names, argument meaning and error behaviour for the launch half of that
module: ``_validate_counts`` (:20-27), ``_validate_offsets`` (:30-55),
``_validate_tensors`` (:58-93) and ``launch_gpu`` (:120-172).  The reference's
``cpu_oracle`` (:288-329) is a test checker there and is one here too: it
lives with the test infrastructure, not in this package, and nothing here
computes a result on the host.

Differences that do not change results:

* offsets are validated by one native pass instead of a Python loop over a
  list (the reference's ``:43-50``): on the GPU, without a host copy, when
  the launch is large enough to be planned (the same rules in the same order,
  so the same exception for the same input), else over a host copy;
* no per-call compilation or module load (the reference's ``:144-155``);
* ``block_size`` is still validated the same way but is only a hint: the
  physical schedule (warp / CTA / split / persistent tile tasks) is chosen by
  a plan built from the segment-length histogram;
* plans are cached per offsets content (a 64-bit digest computed by the
  validation pass on the device, or exact comparison of the host copy) and
  per stream, so repeated launches over the same CSR structure skip the
  planner and launches on different streams never share scratch.
"""

import collections
import json
import os
import sys
import threading
from typing import NamedTuple

from . import _runtime

_I32_LIMIT = 1 << 31
_KINDS = {"sum": 0, "max": 1}
# kinds the reference's dialect names but its runner rejects; accepted only
# when the caller asks for extensions
_EXTENDED_KINDS = {"min": 2}
# Below this many values + segments a launch is latency-bound whatever the
# mapping, and the plan-free schedules are used.
_PLAN_THRESHOLD = 1 << 16
_PLAN_CACHE_ENTRIES = 4


def _validate_counts(value_count, segment_count):
    """Both counts travel as signed i32 through the kernel ABI."""
    for label, count in (("value count", value_count),
                         ("segment count", segment_count)):
        if type(count) is not int or count < 0 or count >= _I32_LIMIT:
            raise ValueError(f"{label} must be a nonnegative i32")


def _validate_offsets(offsets, value_count, output_count):
    """Validate a host list of offsets; return the segment count.

    List form of the check, kept for callers that hold Python ints (the
    reference's tests call it this way).  Tensors go through
    ``_validate_host_offsets`` which applies the same rules natively.
    """
    if not offsets:
        raise ValueError("offsets must contain at least the initial zero")
    segment_count = len(offsets) - 1
    _validate_counts(value_count, segment_count)
    if type(output_count) is not int or output_count < segment_count:
        raise ValueError(
            f"output has {output_count} elements for {segment_count} segments"
        )
    if offsets[0] != 0:
        raise ValueError("offsets must start at zero")
    floor = 0
    for offset in offsets:
        if type(offset) is not int or offset < -_I32_LIMIT or (
            offset >= _I32_LIMIT
        ):
            raise ValueError("offsets must contain signed i32 values")
        if offset < 0:
            raise ValueError("offsets must not be negative")
        if offset < floor:
            raise ValueError("offsets must be nondecreasing")
        floor = offset
    if offsets[-1] > value_count:
        raise ValueError(
            f"final offset {offsets[-1]} exceeds value count {value_count}"
        )
    return segment_count


def _validate_host_offsets(host_offsets, value_count, output_count):
    """Native one-pass form of ``_validate_offsets`` for a CPU int32 tensor."""
    from . import _native

    count = host_offsets.numel()
    if count == 0:
        raise ValueError("offsets must contain at least the initial zero")
    segment_count = count - 1
    _validate_counts(value_count, segment_count)
    reason, _ = _native.validate_offsets(
        host_offsets.data_ptr(), count, value_count, output_count
    )
    if reason == "ok":
        return segment_count
    _raise_offsets_error(reason, segment_count, value_count, output_count,
                         lambda: int(host_offsets[-1]))


def _raise_offsets_error(reason, segment_count, value_count, output_count,
                         final_offset):
    """The reference's exception for the first rule the offsets break."""
    if reason == "output_small":
        raise ValueError(
            f"output has {output_count} elements for {segment_count} segments"
        )
    if reason == "nonzero_start":
        raise ValueError("offsets must start at zero")
    if reason == "negative":
        raise ValueError("offsets must not be negative")
    if reason == "decreasing":
        raise ValueError("offsets must be nondecreasing")
    if reason == "exceeds_values":
        raise ValueError(
            f"final offset {final_offset()} exceeds value count "
            f"{value_count}"
        )
    if reason == "empty":
        raise ValueError("offsets must contain at least the initial zero")
    raise ValueError("value count must be a nonnegative i32")


def _validate_tensors(values, offsets, output, *, require_cuda=True,
                      elementwise_output=False, _host_offsets=None,
                      extended_dtypes=False):
    """Check dtype / rank / layout / offsets / device; return both counts.

    Same order and messages as the reference (:58-93).  With
    ``elementwise_output`` the output holds one element per value (softmax)
    instead of one per segment.
    """
    torch = _runtime._import_torch()
    named = (("values", values), ("offsets", offsets), ("output", output))
    for name, tensor in named:
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
    wide = extended_dtypes and isinstance(values, torch.Tensor) and (
        values.dtype in (torch.float16, torch.bfloat16, torch.int32))
    for name, tensor in (named[0], named[2]):
        if wide and name == "values":
            continue
        if wide and values.dtype == torch.int32:
            if tensor.dtype != torch.int32:
                raise TypeError(
                    f"{name} must have dtype torch.int32 for int32 values")
            continue
        if tensor.dtype != torch.float32:
            raise TypeError(f"{name} must have dtype torch.float32")
    if offsets.dtype != torch.int32:
        raise TypeError("offsets must have dtype torch.int32")
    for name, tensor in named:
        if tensor.dim() != 1:
            raise TypeError(f"{name} must have rank one")
        if not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous")

    value_count = values.numel()
    output_count = output.numel()
    _last_host_offsets.value = None
    _last_digest.value = None
    if _host_offsets is None and _on_current_device(offsets, torch) and (
        value_count + offsets.numel() - 1 >= _PLAN_THRESHOLD
    ):
        # large launch: the offsets stay on the device
        segment_count = _validate_device_offsets(
            offsets, value_count,
            max(offsets.numel() - 1, 0) if elementwise_output
            else output_count,
            torch,
        )
        if elementwise_output and output_count < value_count:
            raise ValueError(
                f"output has {output_count} elements for {value_count} values"
            )
        if require_cuda:
            device = torch.cuda.current_device()
            for name, tensor in named:
                if tensor.device.type != "cuda":
                    raise TypeError(f"{name} must be a CUDA tensor")
                if tensor.device.index != device:
                    raise ValueError(
                        f"{name} must be on the current CUDA device")
        return value_count, segment_count
    host = _host_offsets
    if host is None:
        host = offsets.detach().cpu()
    if elementwise_output:
        segment_count = _validate_host_offsets(
            host, value_count, max(host.numel() - 1, 0)
        )
        if output_count < value_count:
            raise ValueError(
                f"output has {output_count} elements for {value_count} values"
            )
    else:
        segment_count = _validate_host_offsets(host, value_count, output_count)
    if require_cuda:
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is unavailable in PyTorch")
        device = torch.cuda.current_device()
        for name, tensor in named:
            if tensor.device.type != "cuda":
                raise TypeError(f"{name} must be a CUDA tensor")
            if tensor.device.index != device:
                raise ValueError(f"{name} must be on the current CUDA device")
    _last_host_offsets.value = host
    return value_count, segment_count


# the host copy made by the most recent validation on this thread, so that
# launch_gpu can hand it to the planner without a second device-to-host copy
_last_host_offsets = threading.local()
# or, when that validation ran on the device, the digest of the offsets'
# content it computed: (data pointer, segment count, hash)
_last_digest = threading.local()


def _on_current_device(tensor, torch):
    return (
        tensor.device.type == "cuda"
        and torch.cuda.is_available()
        and tensor.device.index == torch.cuda.current_device()
    )


def _validate_device_offsets(offsets, value_count, output_count, torch):
    """``_validate_offsets`` for a CUDA int32 tensor, without a host copy."""
    from . import _native

    count = offsets.numel()
    if count == 0:
        raise ValueError("offsets must contain at least the initial zero")
    segment_count = count - 1
    _validate_counts(value_count, segment_count)
    stream = _runtime._current_stream(torch)
    reason, _, digest, last = _native.validate_offsets_device(
        offsets.data_ptr(), segment_count, value_count, output_count,
        stream.cuda_stream,
    )
    if reason != "ok":
        _raise_offsets_error(reason, segment_count, value_count, output_count,
                             lambda: last)
    _last_digest.value = (offsets.data_ptr(), segment_count, digest)
    return segment_count


class SegmentPlan:
    """A schedule for one CSR offsets array on one device.

    Built by the native planner from the segment-length histogram: segments
    are bucketed by length, short ones are packed into tile tasks, long ones
    are cut into chunks whose partials a second pass merges, and a schedule is
    chosen.  From a CPU offsets tensor the planner runs on the host; from a
    CUDA tensor it runs on the GPU and the offsets never leave the device.
    The plan owns device copies of its task list, of the offsets and of the
    partial scratch.  It stays valid for as long as the offsets hold the same
    numbers; launches that share a plan must not overlap on the GPU (they
    share the merge scratch and the ticket counters): keep a plan to one
    stream, or order the streams yourself.  The plans ``launch_gpu`` and
    ``launch_softmax_gpu`` find by themselves are cached per stream.
    """

    def __init__(self, host_offsets, value_count, op="reduce", *,
                 _digest=None):
        from . import _native

        torch = _runtime._import_torch()
        if isinstance(host_offsets, torch.Tensor) and (
            host_offsets.device.type == "cuda"
        ):
            self._from_device(host_offsets, value_count, op, _native, torch,
                              _digest)
            return
        if (
            not isinstance(host_offsets, torch.Tensor)
            or host_offsets.device.type != "cpu"
            or host_offsets.dtype != torch.int32
            or host_offsets.dim() != 1
            or not host_offsets.is_contiguous()
            or host_offsets.numel() < 1
        ):
            raise TypeError(
                "plan needs a contiguous rank-one CPU int32 offsets tensor"
            )
        self._native = _native
        self.segment_count = host_offsets.numel() - 1
        self.value_count = int(value_count)
        self.op = op
        self.device = torch.cuda.current_device()
        code = _native.OP_SOFTMAX if op == "softmax" else _native.OP_REDUCE
        self._handle = _native.plan_create(
            host_offsets.data_ptr(), self.segment_count, self.value_count, code
        )
        self._dump()

    def _from_device(self, offsets, value_count, op, _native, torch,
                     digest=None):
        if (
            offsets.dtype != torch.int32
            or offsets.dim() != 1
            or not offsets.is_contiguous()
            or offsets.numel() < 1
            or not _on_current_device(offsets, torch)
        ):
            raise TypeError(
                "plan needs a contiguous rank-one int32 offsets tensor on the "
                "current CUDA device"
            )
        self._native = _native
        self.segment_count = offsets.numel() - 1
        self.value_count = int(value_count)
        self.op = op
        self.device = torch.cuda.current_device()
        code = _native.OP_SOFTMAX if op == "softmax" else _native.OP_REDUCE
        self._handle = None
        _validate_counts(self.value_count, self.segment_count)
        stream = _runtime._current_stream(torch)
        if digest is not None:
            # validated a moment ago on this stream: its summary is reused
            self._handle = _native.plan_create_validated(
                offsets.data_ptr(), self.segment_count, self.value_count,
                code, stream.cuda_stream, digest,
            )
            self._dump()
            return
        handle, reason, _ = _native.plan_create_device(
            offsets.data_ptr(), self.segment_count, self.value_count,
            self.segment_count, code, stream.cuda_stream,
        )
        if handle is None:
            _raise_offsets_error(
                reason, self.segment_count, self.value_count,
                self.segment_count, lambda: int(offsets[-1]),
            )
        self._handle = handle
        self._dump()

    def _dump(self):
        """With SWAGE_DUMP_PLAN set, every new plan is described on stderr."""
        if os.environ.get("SWAGE_DUMP_PLAN"):
            sys.stderr.write(
                "swage plan: " + self._native.plan_describe(self._handle) + "\n"
            )

    @property
    def handle(self):
        if self._handle is None:
            raise RuntimeError("plan has been closed")
        return self._handle

    def describe(self):
        """Histogram, bucket shares, task counts and the chosen schedule."""
        return json.loads(self._native.plan_describe(self.handle))

    def check(self):
        """Synchronise and raise if a bounded device-side wait gave up."""
        self._native.plan_status(self.handle)

    def peek(self):
        """Raise if a launch of this plan that has FINISHED flagged an error
        (a wait that gave up, a task or segment that does not fit the
        launch's arrays).  Costs no CUDA call; the launch functions call it
        before every launch, so a launch that went wrong is reported by the
        next one instead of passing silently."""
        self._native.plan_peek_status(self.handle)

    def close(self):
        if self._handle is not None:
            self._native.plan_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def plan_segments(offsets, value_count=None, op="reduce"):
    """Validate ``offsets`` (CPU or CUDA int32) and build a ``SegmentPlan``.

    A CUDA tensor on the current device is validated and planned on the GPU
    (``value_count`` must then be given: reading it off the tensor would
    copy); a CPU tensor by the host planner.
    """
    torch = _runtime._import_torch()
    if not isinstance(offsets, torch.Tensor):
        raise TypeError("offsets must be a torch.Tensor")
    if offsets.dtype != torch.int32:
        raise TypeError("offsets must have dtype torch.int32")
    if offsets.dim() != 1:
        raise TypeError("offsets must have rank one")
    if value_count is not None and _on_current_device(offsets, torch):
        return SegmentPlan(offsets.detach().contiguous(), value_count, op)
    host = offsets.detach().cpu().contiguous()
    if value_count is None:
        value_count = int(host[-1]) if host.numel() else 0
    _validate_host_offsets(host, int(value_count), max(host.numel() - 1, 0))
    return SegmentPlan(host, value_count, op)


_plan_cache = collections.OrderedDict()
_plan_cache_lock = threading.Lock()

# A plan owns scratch that its launches write (partials, arrival counters,
# ticket counters): two launches of one plan must not overlap on the GPU.
# Launches on one stream never do, so the caches hand out one plan per
# (offsets, stream): two streams reducing over the same CSR structure get a
# plan each.  An evicted plan is only dropped from the cache; it is closed
# when the last launch that still holds it lets go.


def _cached_plan(host_offsets, value_count, op, device, stream):
    """Plan for exactly these offsets; equality is checked on the full array."""
    torch = _runtime._import_torch()
    key = (device, stream, op, host_offsets.numel(), value_count)
    with _plan_cache_lock:
        bucket = _plan_cache.get(key)
        if bucket is not None:
            for kept, plan in bucket:
                if torch.equal(kept, host_offsets):
                    _plan_cache.move_to_end(key)
                    return plan
        plan = SegmentPlan(host_offsets, value_count, op)
        _plan_cache.setdefault(key, []).append((host_offsets.clone(), plan))
        _plan_cache.move_to_end(key)
        while sum(len(b) for b in _plan_cache.values()) > _PLAN_CACHE_ENTRIES:
            oldest = next(iter(_plan_cache))
            entries = _plan_cache[oldest]
            entries.pop(0)
            if not entries:
                del _plan_cache[oldest]
        return plan


_device_plan_cache = collections.OrderedDict()


def _cached_device_plan(offsets, value_count, op, device, stream, digest):
    """Plan built on the GPU for offsets with this content digest."""
    key = (device, stream, op, offsets.numel(), value_count, digest)
    with _plan_cache_lock:
        plan = _device_plan_cache.get(key)
        if plan is not None:
            _device_plan_cache.move_to_end(key)
            return plan
        plan = SegmentPlan(offsets, value_count, op, _digest=digest)
        _device_plan_cache[key] = plan
        while len(_device_plan_cache) > _PLAN_CACHE_ENTRIES:
            _device_plan_cache.popitem(last=False)
        return plan


def _plan_for_launch(offsets, value_count, segment_count, op, torch):
    """The cached plan for a launch that was just validated on this thread."""
    device = torch.cuda.current_device()
    stream = _runtime._current_stream(torch).cuda_stream
    digest = getattr(_last_digest, "value", None)
    _last_digest.value = None
    if digest is not None and digest[:2] == (offsets.data_ptr(),
                                             segment_count):
        return _cached_device_plan(offsets, value_count, op, device, stream,
                                   digest[2])
    host = getattr(_last_host_offsets, "value", None)
    if host is None or host.numel() != segment_count + 1:
        host = offsets.detach().cpu()
    return _cached_plan(host, value_count, op, device, stream)


def _drop_cached(plan):
    """Forget a plan whose launch went wrong; the next launch plans afresh."""
    with _plan_cache_lock:
        for key, kept in list(_device_plan_cache.items()):
            if kept is plan:
                del _device_plan_cache[key]
        for key, entries in list(_plan_cache.items()):
            entries[:] = [pair for pair in entries if pair[1] is not plan]
            if not entries:
                del _plan_cache[key]


def _peek(plan):
    try:
        plan.peek()
    except RuntimeError:
        _drop_cached(plan)
        raise


def clear_plan_cache():
    """Drop every cached plan (frees their device memory)."""
    with _plan_cache_lock:
        for entries in _plan_cache.values():
            for _, plan in entries:
                plan.close()
        _plan_cache.clear()
        for plan in _device_plan_cache.values():
            plan.close()
        _device_plan_cache.clear()


def _schedule_code(schedule):
    from . import _native

    if schedule not in _native.SCHEDULES:
        raise ValueError(
            "schedule must be one of " + ", ".join(sorted(_native.SCHEDULES))
        )
    return _native.SCHEDULES[schedule]


_thread_limits = {}


def _check_block(block_size, torch):
    if type(block_size) is not int or block_size <= 0:
        raise ValueError("block size must be a positive integer")
    device = torch.cuda.current_device()
    limit = _thread_limits.get(device)
    if limit is None:
        limit = torch.cuda.get_device_properties(device).max_threads_per_block
        _thread_limits[device] = limit
    if block_size > limit:
        raise ValueError(
            f"block size {block_size} exceeds device limit {limit}"
        )


class ElementMap(NamedTuple):
    """``fn(scale * x + shift)`` applied to every value before it is reduced:
    the dialect's ``swage.map`` region in front of a ``swage.reduce``
    (``test/Dialect/Swage/roundtrip.mlir:43-52``).  ``fn`` is ``"identity"``,
    ``"abs"``, ``"square"`` or ``"exp"``; ``scale`` and ``shift`` are values
    captured at launch.  The product and the sum are rounded separately; the
    default shift is ``-0.0``, the one addend that leaves every value, signed
    zeros included, as it is."""

    fn: str = "identity"
    scale: float = 1.0
    shift: float = -0.0


def launch_gpu(values, offsets, output, kind, block_size=128, *, plan=None,
               schedule="auto", extensions=False, map=None, _validated=None):
    """Queue one segmented ``sum`` or ``max`` on the current PyTorch stream.

    ``output[s] = reduce(values[offsets[s]:offsets[s + 1]])`` for every
    segment; an empty segment gives the identity (``+0.0`` / ``-inf``); only
    the first ``segment_count`` outputs are written.  Reference: ``launch_gpu``
    (``_segmented_qualification.py:120-172``).

    ``plan`` (a ``SegmentPlan`` for these offsets) skips validation's planner
    step; ``schedule`` forces ``warp``, ``cta``, ``split``, ``persistent`` or
    ``resident``.
    With ``extensions=True`` ``kind`` may also be ``"min"`` (NaN-propagating
    minimum from ``+inf``: the dialect's ``kind<min>``, which the reference's
    lowering rejects, ``SegmentedReduction.cpp:106-108``), and ``values`` may
    hold ``float16`` / ``bfloat16`` (widened exactly, reduced in fp32,
    ``output`` fp32) or ``int32`` (wrap-around sum, signed max / min,
    ``output`` int32): element types the dialect admits
    (``SwageOps.td:101-105``) and the lowering rejects
    (``SegmentedReduction.cpp:110-119``).  ``map`` (an ``ElementMap``,
    extensions only, floating values only) is applied to every value before it
    is reduced, in the same pass: a non-identity map region in front of the
    reduce, which the reference's lowering rejects
    (``SegmentedReduction.cpp:106-119``).  Without ``extensions`` the
    reference's errors are kept.
    """
    torch = _runtime._import_torch()
    if _validated is None:
        value_count, segment_count = _validate_tensors(
            values, offsets, output, extended_dtypes=bool(extensions))
    else:
        value_count, segment_count = _validated
    _check_block(block_size, torch)
    if kind in _KINDS:
        kind_code = _KINDS[kind]
    elif extensions and kind in _EXTENDED_KINDS:
        kind_code = _EXTENDED_KINDS[kind]
    else:
        raise ValueError("reduction kind must be 'sum' or 'max'")
    code = _schedule_code(schedule)
    if map is not None:
        if not extensions:
            raise ValueError("an element map needs extensions=True")
        if not isinstance(map, ElementMap):
            raise TypeError("map must be an ElementMap")
        if map.fn not in ("identity", "abs", "square", "exp"):
            raise ValueError(
                "map function must be 'identity', 'abs', 'square' or 'exp'")
        if values.dtype == torch.int32:
            raise TypeError("integer segments are not mapped")
    if segment_count == 0:
        return None

    from . import _native

    if plan is None and (
        code in (_native.SCHED_SPLIT, _native.SCHED_PERSISTENT,
                 _native.SCHED_RESIDENT)
        or (code == _native.SCHED_AUTO
            and value_count + segment_count >= _PLAN_THRESHOLD)
    ):
        plan = _plan_for_launch(offsets, value_count, segment_count, "reduce",
                                torch)
    _last_host_offsets.value = None
    _last_digest.value = None
    if plan is not None:
        _peek(plan)
    stream = _runtime._current_stream(torch)
    if map is not None:
        dtype = {torch.float32: _native.DTYPE_F32,
                 torch.float16: _native.DTYPE_F16,
                 torch.bfloat16: _native.DTYPE_BF16}[values.dtype]
        _native.segreduce_map(
            kind_code, dtype, _native.MAPS[map.fn], float(map.scale),
            float(map.shift), values.data_ptr(), offsets.data_ptr(),
            output.data_ptr(), value_count, segment_count,
            plan.handle if plan is not None else None,
            code, block_size, stream.cuda_stream,
        )
    elif values.dtype == torch.float32:
        _native.segreduce(
            kind_code, values.data_ptr(), offsets.data_ptr(),
            output.data_ptr(), value_count, segment_count,
            plan.handle if plan is not None else None,
            code, block_size, stream.cuda_stream,
        )
    else:
        dtype = {torch.float16: _native.DTYPE_F16,
                 torch.bfloat16: _native.DTYPE_BF16,
                 torch.int32: _native.DTYPE_I32}[values.dtype]
        _native.segreduce_typed(
            kind_code, dtype, values.data_ptr(), offsets.data_ptr(),
            output.data_ptr(), value_count, segment_count,
            plan.handle if plan is not None else None,
            code, block_size, stream.cuda_stream,
        )
    for tensor in (values, offsets, output):
        tensor.record_stream(stream)
    return None


def launch_sum_max_gpu(values, offsets, sum_output, max_output, *,
                       _validated=None):
    """Queue the segmented sum AND max of one input as a single kernel.

    ``sum_output[s]`` and ``max_output[s]`` are what two ``launch_gpu`` calls
    with ``"sum"`` and ``"max"`` give (max bit for bit, sum to the documented
    tolerance), but every value is read once.  Plan-free: meant for inputs of
    moderate size such as the canonical 4096-segment configuration.  The
    reference runs the two kinds as two launches
    (``_segmented_qualification.py:120-172``); the validation is its own,
    applied to both outputs.
    """
    torch = _runtime._import_torch()
    if _validated is None:
        value_count, segment_count = _validate_tensors(values, offsets,
                                                       sum_output)
        _last_host_offsets.value = None
        _last_digest.value = None
        if (not isinstance(max_output, torch.Tensor)
                or max_output.dtype != torch.float32):
            raise TypeError("output must have dtype torch.float32")
        if max_output.dim() != 1:
            raise TypeError("output must have rank one")
        if not max_output.is_contiguous():
            raise ValueError("output must be contiguous")
        if max_output.numel() < segment_count:
            raise ValueError(
                f"output has {max_output.numel()} elements for "
                f"{segment_count} segments")
        if max_output.device != sum_output.device:
            raise ValueError("output must be on the current CUDA device")
    else:
        value_count, segment_count = _validated
    if segment_count == 0:
        return None
    if sum_output.data_ptr() == max_output.data_ptr():
        raise ValueError("the two outputs must not alias")

    from . import _native

    stream = _runtime._current_stream(torch)
    _native.segreduce_sum_max(
        values.data_ptr(), offsets.data_ptr(), sum_output.data_ptr(),
        max_output.data_ptr(), value_count, segment_count, stream.cuda_stream)
    for tensor in (values, offsets, sum_output, max_output):
        tensor.record_stream(stream)
    return None


def launch_softmax_gpu(values, offsets, output, *, plan=None, schedule="auto",
                       _validated=None):
    """Queue one segmented softmax on the current PyTorch stream.

    ``output[i] = exp(values[i] - m) / d`` over each segment (``m`` its
    maximum, ``d`` the sum of ``exp(values - m)``); empty segments write
    nothing.  ``output`` has one element per value and must not alias
    ``values``.  The reference only defines the semantic form
    (``test/Dialect/Swage/softmax.mlir:13-31``).
    """
    torch = _runtime._import_torch()
    if _validated is None:
        value_count, segment_count = _validate_tensors(
            values, offsets, output, elementwise_output=True
        )
    else:
        value_count, segment_count = _validated
    code = _schedule_code(schedule)
    if values.data_ptr() == output.data_ptr() and value_count > 0:
        raise ValueError("output must not alias values")
    if segment_count == 0 or value_count == 0:
        return None

    from . import _native

    if plan is None and (
        code in (_native.SCHED_SPLIT, _native.SCHED_PERSISTENT,
                 _native.SCHED_RESIDENT)
        or (code == _native.SCHED_AUTO
            and value_count + segment_count >= _PLAN_THRESHOLD)
    ):
        plan = _plan_for_launch(offsets, value_count, segment_count,
                                "softmax", torch)
    _last_host_offsets.value = None
    _last_digest.value = None
    if plan is not None:
        _peek(plan)
    stream = _runtime._current_stream(torch)
    _native.segsoftmax(
        values.data_ptr(), offsets.data_ptr(), output.data_ptr(), value_count,
        segment_count, plan.handle if plan is not None else None, code,
        stream.cuda_stream,
    )
    for tensor in (values, offsets, output):
        tensor.record_stream(stream)
    return None


__all__ = [
    "SegmentPlan", "clear_plan_cache", "launch_gpu", "launch_softmax_gpu",
    "launch_sum_max_gpu", "plan_segments",
]
