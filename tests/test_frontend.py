"""Kernel capture, input validation and program recognition (no GPU)."""

import subprocess
import sys

import pytest

import swage_b200 as sw
import swage_b200.language as sl


@sw.jit
def add_kernel(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):  # noqa: D103
    pid = sl.program_id(0)
    offsets = pid * BLOCK + sl.arange(0, BLOCK)
    mask = offsets < n
    x = sl.load(x_ptr + offsets, mask=mask, other=0.0)
    y = sl.load(y_ptr + offsets, mask=mask, other=0.0)
    sl.store(output_ptr + offsets, x + y, mask=mask)


@sw.jit
def segmented_sum(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    segment = sl.segment(values_ptr, offsets_ptr, sid)
    x = sl.load_segment(segment)
    sl.store(output_ptr + sid, sl.sum(x))


@sw.jit
def segmented_max(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    sl.store(output_ptr + sid, sl.max(x))


@sw.jit
def segmented_softmax(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    segment = sl.segment(values_ptr, offsets_ptr, sid)

    x = sl.load_segment(segment)
    maximum = sl.max(x)
    numerator = sl.exp(x - maximum)
    denominator = sl.sum(numerator)

    sl.store_segment(output_ptr, segment, numerator / denominator)


def test_import_pulls_in_neither_torch_nor_the_native_library():
    code = (
        "import sys, swage_b200, swage_b200.language\n"
        "assert 'torch' not in sys.modules\n"
        "assert 'swage_b200._native' not in sys.modules\n"
        "assert 'ctypes' not in sys.modules or True\n"
    )
    result = subprocess.run([sys.executable, "-c", code],
                            capture_output=True, text=True,
                            cwd=str(__import__("pathlib").Path(__file__)
                                    .resolve().parent.parent))
    assert result.returncode == 0, result.stderr


@pytest.mark.parametrize("call", [
    lambda: sl.program_id(0), lambda: sl.arange(0, 1), lambda: sl.load(None),
    lambda: sl.store(None, None), lambda: sl.segment_id(0),
    lambda: sl.load_segment(None), lambda: sl.max(None), lambda: sl.sum(None),
    lambda: sl.exp(None), lambda: sl.segment(None, None, None),
    lambda: sl.store_segment(None, None, None),
])
def test_symbolic_calls_fail_outside_a_kernel(call):
    with pytest.raises(RuntimeError, match="only available inside @swage.jit"):
        call()


def test_decorating_does_not_run_the_body():
    calls = []

    @sw.jit
    def kernel():
        calls.append("ran")

    assert calls == [] and kernel.__name__ == "kernel"
    with pytest.raises(RuntimeError, match=r"use kernel\.launch\(\)"):
        kernel()


def test_stacked_decorators_are_rejected():
    def passthrough(function):
        return function

    with pytest.raises(sw.CompilationError,
                       match="only @swage.jit may decorate a kernel"):
        @sw.jit
        @passthrough
        def kernel():
            return


def test_recognises_the_four_programs():
    assert add_kernel.recognize().kind == "vector_add"
    assert add_kernel.recognize().roles == {
        "x": "x_ptr", "y": "y_ptr", "out": "output_ptr", "n": "n"}
    assert segmented_sum.recognize().kind == "segmented_sum"
    assert segmented_max.recognize().kind == "segmented_max"
    program = segmented_softmax.recognize()
    assert program.kind == "segmented_softmax"
    assert program.roles == {"values": "values_ptr", "offsets": "offsets_ptr",
                             "out": "output_ptr"}


@sw.jit
def sum_of_squares(values_ptr, offsets_ptr, output_ptr,  # noqa: D103
                   SCALE: sl.constexpr):
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    y = x * SCALE - 1.5
    sl.store(output_ptr + sid, sl.sum(y * y))


@sw.jit
def max_magnitude(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    sl.store(output_ptr + sid, sl.max(sl.abs(-x)))


@sw.jit
def sum_of_exponentials(values_ptr, offsets_ptr, output_ptr,  # noqa: D103
                        SHIFT: sl.constexpr):
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    sl.store(output_ptr + sid, sl.min(sl.exp(SHIFT + 2 * x)))


@sw.jit
def reassociated(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    sl.store(output_ptr + sid, sl.sum((x - 1.0) * 2.0))


@sw.jit
def map_after_the_function(values_ptr, offsets_ptr, output_ptr):  # noqa: D103
    sid = sl.segment_id(0)
    x = sl.load_segment(sl.segment(values_ptr, offsets_ptr, sid))
    sl.store(output_ptr + sid, sl.sum(sl.exp(x) * 2.0))


def test_recognises_maps_in_front_of_a_reduction():
    """``fn(scale * x + shift)`` with fn in identity / abs / square / exp and
    the constants literals or constexpr parameters; only forms that ARE one
    multiply and one add in fp32 are taken (nothing is reassociated)."""
    from swage_b200._frontend import constant_value

    program = sum_of_squares.recognize()
    assert program.kind == "segmented_sum"
    function, scale, shift = program.map
    assert function == "square"
    assert constant_value(scale, {"SCALE": 3}) == 3.0
    assert constant_value(shift, {"SCALE": 3}) == -1.5

    program = max_magnitude.recognize()
    assert program.kind == "segmented_max"
    function, scale, shift = program.map
    assert function == "abs"
    assert constant_value(scale, {}) == -1.0
    value = constant_value(shift, {})
    assert value == 0.0 and str(value) == "-0.0"  # the neutral addend

    program = sum_of_exponentials.recognize()
    assert program.kind == "segmented_min"
    function, scale, shift = program.map
    assert (function, constant_value(scale, {}),
            constant_value(shift, {"SHIFT": 0.25})) == ("exp", 2.0, 0.25)

    assert segmented_sum.recognize().map is None
    for kernel in (reassociated, map_after_the_function):
        with pytest.raises(sw.CompilationError,
                           match="not one of the supported"):
            kernel.recognize()


def test_non_canonical_bodies_are_compilation_errors():
    @sw.jit
    def swapped(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):
        pid = sl.program_id(0)
        offsets = pid * BLOCK + sl.arange(0, BLOCK)
        mask = offsets < n
        x = sl.load(x_ptr + offsets, mask=mask, other=0.0)
        y = sl.load(y_ptr + offsets, mask=mask, other=0.0)
        sl.store(output_ptr + offsets, y + x, mask=mask)  # y + x, not x + y

    with pytest.raises(sw.CompilationError, match="not one of the supported"):
        swapped.recognize()

    @sw.jit
    def unmasked(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):
        pid = sl.program_id(0)
        offsets = pid * BLOCK + sl.arange(0, BLOCK)
        x = sl.load(x_ptr + offsets, mask=offsets < n, other=0.0)
        sl.store(output_ptr + offsets, x + x, mask=offsets < n)

    with pytest.raises(sw.CompilationError, match="not one of the supported"):
        unmasked.recognize()

    @sw.jit
    def loops(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):
        for _ in range(3):
            pass

    with pytest.raises(sw.CompilationError,
                       match="unsupported statement 'For'") as caught:
        loops.recognize()
    assert str(caught.value).startswith(f"{__file__}:")
    assert ": loops: " in str(caught.value)

    @sw.jit
    def axis_one(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):
        pid = sl.program_id(1)
        sl.store(output_ptr + pid, x_ptr, mask=None)

    with pytest.raises(sw.CompilationError, match="axis 0"):
        axis_one.recognize()


@pytest.mark.parametrize(("value", "reason"), [
    (True, "constexpr 'VALUE' must be an integer"),
    (1.5, "constexpr 'VALUE' must be an integer"),
    (1 << 63, "constexpr 'VALUE' must fit signed 64-bit"),
    (-(1 << 63) - 1, "constexpr 'VALUE' must fit signed 64-bit"),
])
def test_constexpr_values_are_validated(value, reason):
    @sw.jit
    def kernel(VALUE: sl.constexpr):
        return

    with pytest.raises(sw.CompilationError, match=reason):
        kernel.emit_mlir(signature={}, constexprs={"VALUE": value})


def test_input_mode_and_key_diagnostics():
    @sw.jit
    def kernel(value):
        return

    with pytest.raises(sw.CompilationError,
                       match="exactly one of signature or arguments"):
        kernel.emit_mlir(constexprs={})
    with pytest.raises(sw.CompilationError,
                       match="exactly one of signature or arguments"):
        kernel.emit_mlir(signature={}, arguments={}, constexprs={})
    with pytest.raises(
        sw.CompilationError,
        match="arguments keys must match runtime parameters; missing: value",
    ):
        kernel.emit_mlir(arguments={}, constexprs={})
    with pytest.raises(sw.CompilationError,
                       match="runtime parameter 'value' must be passed in"):
        kernel.emit_mlir(signature={}, constexprs={"value": 1})
    with pytest.raises(sw.CompilationError,
                       match="unsupported type for parameter 'value'"):
        kernel.emit_mlir(signature={"value": sl.float32}, constexprs={})
    # valid inputs: the reference would now emit MLIR; this library says why not
    with pytest.raises(RuntimeError, match="compile-only MLIR emission"):
        kernel.emit_mlir(signature={"value": sl.int32}, constexprs={})


@pytest.mark.parametrize("value", [True, -(1 << 31) - 1, 1 << 31, 1.5, object()])
def test_inferred_scalars_reject_unsupported_values(value):
    @sw.jit
    def kernel(runtime_value):
        return

    with pytest.raises(
        sw.CompilationError,
        match="unsupported argument for parameter 'runtime_value'",
    ):
        kernel.emit_mlir(arguments={"runtime_value": value}, constexprs={})


def test_install_as_makes_reference_style_imports_work():
    code = (
        "import swage_b200; swage_b200.install_as('swage')\n"
        "import swage as sw, swage.language as sl\n"
        "from swage._segmented_qualification import launch_gpu, "
        "_validate_offsets\n"
        "assert sw.jit is swage_b200.jit and sl.constexpr is not None\n"
    )
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    result = subprocess.run([sys.executable, "-c", code], capture_output=True,
                            text=True, cwd=str(root))
    assert result.returncode == 0, result.stderr
