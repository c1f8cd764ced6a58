"""Launch path of ``kernel.launch(arguments=..., constexprs=..., grid=...)``.

Drop-in for the reference's ``python/swage/_runtime.py``: ``launch`` (:47-86)
and ``_validate_launch`` (:100-180).  What is kept, because callers and tests
depend on it:

* every check runs before any ``data_ptr()`` is read, in the reference's
  order, with the reference's exception types and messages;
* ``n == 0`` is a validated no-op that never touches the device (:51-52);
* the launch is asynchronous on ``torch.cuda.current_stream()``, returns
  ``None``, never synchronises / copies / casts / switches device, and calls
  ``record_stream`` on each tensor afterwards (:84-86);
* nothing keeps a tensor or pointer after the call returns.

What is replaced: MLIR emission, the specialization key, the PTX process/disk
cache, ``cuModuleLoadData`` and ``cuLaunchKernel`` (:54-83, :183-531).  The
body is recognised from its AST (``_frontend._Kernel.recognize``) and the
prebuilt sm_100a kernel is called through the C ABI; ``grid`` and ``BLOCK``
stay the *logical* launch shape the caller must get right, while the physical
grid is the library's choice.

Segment kernels (the reference's README sketch, :74-86 there) launch through
the same entry: ``arguments`` holds the values, offsets and output tensors,
``constexprs`` is empty and ``grid`` is ``(segment_count,)``.
"""

from collections.abc import Mapping
from typing import NamedTuple

from . import language

_M3_PARAMETERS = ("x_ptr", "y_ptr", "output_ptr", "n", "BLOCK")


class _LaunchSpec(NamedTuple):
    """Validated facts needed after the Python trust boundary."""

    tensors: tuple
    n: int
    block: int
    grid: tuple
    target: str
    stream: object
    descriptors: tuple


def _import_torch():
    try:
        import torch
    except Exception as error:
        raise RuntimeError(
            "Swage launch requires PyTorch; install 'swage-compiler[pytorch]'"
        ) from error
    return torch


_stream_objects = {}


def _current_stream(torch):
    """``torch.cuda.current_stream()`` from a cache keyed by (device, raw
    stream handle).  Building the ``Stream`` object costs about 3 us per call
    -- as much as launching the kernel of a small input -- while asking for
    the raw handle costs 0.1 us; the object for a given handle on a given
    device is always the same stream."""
    try:
        device = torch.cuda.current_device()
        raw = torch._C._cuda_getCurrentRawStream(device)
    except AttributeError:
        return torch.cuda.current_stream()
    stream = _stream_objects.get((device, raw))
    if stream is None:
        stream = torch.cuda.current_stream()
        if len(_stream_objects) >= 64:
            _stream_objects.clear()
        _stream_objects[(device, raw)] = stream
    return stream


def launch(kernel, *, arguments, constexprs, grid):
    """Validate and asynchronously launch one recognised kernel."""
    torch = _import_torch()
    if _looks_segmented(kernel):
        return _launch_segmented(kernel, arguments, constexprs, grid, torch)
    spec = _validate_launch(kernel, arguments, constexprs, grid, torch)
    if spec.n == 0:
        return None
    program = kernel.recognize()
    if program.kind != "vector_add":
        raise ValueError("M3 launch requires the fixed vector-add kernel")

    from . import _native

    x, y, out = spec.tensors
    _native.vadd(
        x.data_ptr(), y.data_ptr(), out.data_ptr(), spec.n, spec.block,
        spec.stream.cuda_stream,
    )
    for tensor in spec.tensors:
        tensor.record_stream(spec.stream)
    return None


def _validate_launch(kernel, arguments, constexprs, grid, torch):
    if not isinstance(arguments, Mapping):
        raise TypeError("arguments must be a mapping")
    if not isinstance(constexprs, Mapping):
        raise TypeError("constexprs must be a mapping")
    block = constexprs.get("BLOCK")
    if type(block) is not int or block <= 0:
        raise ValueError("constexpr BLOCK must be a positive integer")
    grid_ok = (
        isinstance(grid, tuple) and len(grid) == 1 and type(grid[0]) is int
    )
    if not grid_ok:
        raise TypeError("grid must be a one-element tuple of integers")
    declared = tuple(a.arg for a in kernel.function.args.args)
    if declared != _M3_PARAMETERS:
        raise ValueError(
            "M3 launch requires x_ptr, y_ptr, output_ptr, n, and BLOCK "
            "parameters"
        )
    runtime_names = declared[:4]
    if set(arguments) != set(runtime_names):
        raise ValueError("arguments must contain exactly the M3 parameters")
    if set(constexprs) != {"BLOCK"}:
        raise ValueError("constexprs must contain exactly BLOCK")

    pointer_names = runtime_names[:3]
    tensors = tuple(arguments[name] for name in pointer_names)
    for name, tensor in zip(pointer_names, tensors):
        on_cuda = (
            isinstance(tensor, torch.Tensor) and tensor.device.type == "cuda"
        )
        if not on_cuda:
            raise TypeError(f"argument '{name}' must be a CUDA tensor")
        if tensor.dtype != torch.float32:
            raise TypeError(f"argument '{name}' must have dtype torch.float32")
        if tensor.dim() != 1:
            raise TypeError(f"argument '{name}' must have rank one")
        if not tensor.is_contiguous():
            raise ValueError(f"argument '{name}' must be contiguous")

    n = arguments["n"]
    if type(n) is not int or n < 0 or n >= (1 << 31):
        raise ValueError("n must be a nonnegative i32")
    for name, tensor in zip(pointer_names, tensors):
        if tensor.numel() < n:
            raise ValueError(f"n exceeds tensor length for argument '{name}'")
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is unavailable in PyTorch")
    device = torch.cuda.current_device()
    for name, tensor in zip(pointer_names, tensors):
        if tensor.device.index != device:
            raise ValueError(
                f"argument '{name}' must be on the current CUDA device"
            )

    runtime_types, _ = kernel._validate_inputs(None, arguments, constexprs)
    descriptors = tuple(
        "i32" if runtime_types[name] is language.int32
        else _pointer_descriptor(runtime_types[name])
        for name in runtime_names
    )
    if descriptors != ("ptr<f32>", "ptr<f32>", "ptr<f32>", "i32"):
        raise TypeError("M3 launch requires three f32 pointers and one i32")

    limit = torch.cuda.get_device_properties(device).max_threads_per_block
    if block > limit:
        raise ValueError(f"BLOCK {block} exceeds device limit {limit}")
    expected = (-(-n // block),)
    if grid != expected:
        raise ValueError(f"grid must equal {expected} for n and BLOCK")
    major, minor = torch.cuda.get_device_capability(device)
    return _LaunchSpec(
        tensors, n, block, grid, f"sm_{major}{minor}",
        _current_stream(torch), descriptors,
    )


def _pointer_descriptor(declared):
    element = getattr(declared, "element_type", None)
    if element is language.float32:
        return "ptr<f32>"
    if element is language.int32:
        return "ptr<i32>"
    return "unknown"


# ---------------------------------------------------------------------------
# Segment kernels through the public launch surface
# ---------------------------------------------------------------------------

def _looks_segmented(kernel):
    """Three unannotated runtime parameters, then constexpr parameters only
    (the constants a mapped reduction captures): the segment-kernel shape."""
    arguments = kernel.function.args.args
    if len(arguments) < 3:
        return False
    if any(argument.annotation is not None for argument in arguments[:3]):
        return False
    from ._frontend import _is_constexpr_annotation

    return all(_is_constexpr_annotation(argument.annotation)
               for argument in arguments[3:])


def _launch_segmented(kernel, arguments, constexprs, grid, torch):
    if not isinstance(arguments, Mapping):
        raise TypeError("arguments must be a mapping")
    if not isinstance(constexprs, Mapping):
        raise TypeError("constexprs must be a mapping")
    static_names = {a.arg for a in kernel.function.args.args[3:]}
    if not static_names and len(constexprs) != 0:
        raise ValueError("segment kernels take no constexprs")
    if set(constexprs) != static_names:
        raise ValueError(
            "constexprs must contain exactly the kernel's constexpr parameters"
        )
    for name, value in constexprs.items():
        if type(value) not in (int, float):
            raise TypeError(f"constexpr '{name}' must be an int or a float")
    grid_ok = (
        isinstance(grid, tuple) and len(grid) == 1 and type(grid[0]) is int
    )
    if not grid_ok:
        raise TypeError("grid must be a one-element tuple of integers")
    program = kernel.recognize()
    if not program.kind.startswith("segmented_"):
        raise ValueError("kernel is not a segment kernel")
    names = [program.roles[role] for role in ("values", "offsets", "out")]
    if set(arguments) != set(names):
        raise ValueError(
            "arguments must contain exactly the kernel's three pointers"
        )
    values, offsets, output = (arguments[name] for name in names)

    from . import _segmented_qualification as runner

    softmax = program.kind == "segmented_softmax"
    value_count, segment_count = runner._validate_tensors(
        values, offsets, output, elementwise_output=softmax
    )
    if grid != (segment_count,):
        raise ValueError(
            f"grid must equal {(segment_count,)} for the offsets given"
        )
    if softmax:
        return runner.launch_softmax_gpu(
            values, offsets, output, _validated=(value_count, segment_count)
        )
    element_map = None
    if program.map is not None:
        from ._frontend import constant_value

        function, scale, shift = program.map
        element_map = runner.ElementMap(
            function, constant_value(scale, constexprs),
            constant_value(shift, constexprs))
    return runner.launch_gpu(
        values, offsets, output, program.kind[len("segmented_"):],
        extensions=True, map=element_map,
        _validated=(value_count, segment_count),
    )
