"""Launch validation and ABI marshalling with a stand-in PyTorch (no GPU).

The expected exception types and messages come from
``tests/golden/launch_validation.json`` which records what the reference's own
``kernel.launch`` does for the same inputs.
"""

import gc
import json
import pathlib
import sys
import weakref

import pytest

import fakes
import swage_b200 as sw
import swage_b200.language as sl

GOLDEN = json.loads(
    (pathlib.Path(__file__).parent / "golden" / "launch_validation.json")
    .read_text())


@sw.jit
def add_kernel(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):  # noqa: D103
    pid = sl.program_id(0)
    offsets = pid * BLOCK + sl.arange(0, BLOCK)
    mask = offsets < n
    x = sl.load(x_ptr + offsets, mask=mask, other=0.0)
    y = sl.load(y_ptr + offsets, mask=mask, other=0.0)
    sl.store(output_ptr + offsets, x + y, mask=mask)


class RecordingNative:
    """Stands in for ``swage_b200._native`` and records the C-ABI calls."""

    def __init__(self):
        self.calls = []

    def vadd(self, *arguments):
        self.calls.append(("vadd",) + arguments)


@pytest.fixture
def recording_native(monkeypatch):
    import swage_b200

    native = RecordingNative()
    monkeypatch.setitem(sys.modules, "swage_b200._native", native)
    monkeypatch.setattr(swage_b200, "_native", native, raising=False)
    return native


def test_launch_marshals_raw_pointers_on_the_current_stream(
        monkeypatch, recording_native):
    torch, stream = fakes.fake_torch()
    monkeypatch.setitem(sys.modules, "torch", torch)
    arguments = fakes.vector_add_arguments(torch)

    result = add_kernel.launch(arguments=arguments,
                               constexprs={"BLOCK": 128}, grid=(2,))

    assert result is None
    assert recording_native.calls == [
        ("vadd", 0x1000, 0x2000, 0x3000, 129, 128, 0xABCD)]
    for name in ("x_ptr", "y_ptr", "output_ptr"):
        assert arguments[name].streams == [stream]
        assert arguments[name].pointer_reads == 1


def test_repeated_launches_do_not_retain_tensors(monkeypatch, recording_native):
    torch, _ = fakes.fake_torch()
    monkeypatch.setitem(sys.modules, "torch", torch)
    first = fakes.vector_add_arguments(torch)
    reference = weakref.ref(first["x_ptr"])
    for arguments in (first, fakes.vector_add_arguments(torch)):
        add_kernel.launch(arguments=arguments, constexprs={"BLOCK": 128},
                          grid=(2,))
    del arguments, first
    gc.collect()
    assert len(recording_native.calls) == 2
    assert reference() is None


@pytest.mark.parametrize("case", fakes.LAUNCH_CASES, ids=lambda c: c[0])
def test_launch_validation_matches_the_reference(
        case, monkeypatch, recording_native):
    expected = GOLDEN[case[0]]
    torch, _, arguments, constexprs, grid = fakes.build_launch_case(case)
    monkeypatch.setitem(sys.modules, "torch", torch)

    def run():
        return add_kernel.launch(arguments=arguments, constexprs=constexprs,
                                 grid=grid)

    if "raises" in expected:
        with pytest.raises(Exception) as caught:
            run()
        assert type(caught.value).__name__ == expected["raises"]
        assert expected["message"] in str(caught.value)
    else:
        assert run() == expected["returns"]
    # rejected and empty launches never reach the device or a data pointer
    assert recording_native.calls == []
    if isinstance(arguments, dict):
        for value in arguments.values():
            if isinstance(value, fakes.FakeTensor):
                assert value.pointer_reads == 0


def test_missing_pytorch_is_reported(monkeypatch):
    from swage_b200 import _runtime

    real_import = __import__

    def without_torch(name, *args, **kwargs):
        if name == "torch":
            raise ImportError("missing")
        return real_import(name, *args, **kwargs)

    monkeypatch.setattr("builtins.__import__", without_torch)
    with pytest.raises(RuntimeError, match="requires PyTorch"):
        _runtime._import_torch()


def test_missing_native_library_fails_loudly(monkeypatch, tmp_path):
    from swage_b200 import _native

    monkeypatch.setattr(_native, "_library", None)
    monkeypatch.setattr(_native, "LIBRARY_PATH", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _native.library()


def test_native_errors_use_the_driver_error_format(native_library):
    from swage_b200 import _native

    with pytest.raises(
        RuntimeError,
        match=r"swg_vadd_f32 failed: SWG_ERR_INVALID_ARGUMENT \(1\): ",
    ):
        _native.vadd(0, 0, 0, -5, 128, 0)
