"""The C-ABI library loads and exports what the header declares (no GPU)."""

import ctypes
import pathlib
import re

from swage_b200 import _native

HEADER = pathlib.Path(__file__).resolve().parent.parent / "include" / \
    "swage_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(swg_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_function_is_exported(native_library):
    names = declared_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(native_library, name), f"{name} is not exported"


def test_python_binding_lists_the_same_functions():
    assert sorted(_native.EXPORTS) == declared_functions()


def test_version_and_status_names(native_library):
    assert native_library.swg_abi_version() == 1
    assert native_library.swg_status_name(0) == b"SWG_OK"
    assert native_library.swg_status_name(6) == b"SWG_ERR_DEVICE_TIMEOUT"
    assert native_library.swg_last_error() is not None


def test_header_is_plain_c(tmp_path):
    import subprocess

    source = tmp_path / "probe.c"
    source.write_text('#include "swage_b200.h"\nint main(void){return 0;}\n')
    result = subprocess.run(
        ["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(HEADER.parent),
         "-c", str(source), "-o", str(tmp_path / "probe.o")],
        capture_output=True, text=True)
    assert result.returncode == 0, result.stderr


def test_signatures_take_no_framework_types():
    code = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    assert "torch" not in code.lower() and "at::" not in code
    assert "#include <cuda" not in code
    assert isinstance(ctypes.sizeof(ctypes.c_void_p), int)
