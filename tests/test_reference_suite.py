"""The reference's own runtime test files, unmodified, against this library.

``python/tests/mlir/test_runtime.py`` and
``python/tests/mlir/test_segmented_runtime.py`` of the reference import only
``swage``, ``swage.language``, ``swage._segmented_qualification`` and
``torch``.  With this library aliased under that name (``install_as``) they
run as they are: the validation and oracle cases everywhere, the launch cases
wherever a CUDA device is present as well.  The files are read from a
reference checkout (``SWAGE_REFERENCE``; default: a directory ``reference``
beside this repository) and are never copied; without a checkout the test is
skipped.
"""

import os
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
REFERENCE = pathlib.Path(
    os.environ.get("SWAGE_REFERENCE", ROOT.parent / "reference"))
FILES = ("python/tests/mlir/test_runtime.py",
         "python/tests/mlir/test_segmented_runtime.py")


@pytest.mark.parametrize("relative", FILES)
def test_reference_test_file_passes_unmodified(relative, tmp_path):
    path = REFERENCE / relative
    if not path.exists():
        pytest.skip(f"no reference checkout at {REFERENCE}")
    environment = dict(os.environ)
    environment["PYTHONPATH"] = os.pathsep.join(
        [str(ROOT), str(ROOT / "tests")]
        + ([environment["PYTHONPATH"]] if "PYTHONPATH" in environment else []))
    result = subprocess.run(
        [sys.executable, "-m", "pytest", "-q", "-p", "reference_shim",
         "-p", "no:cacheprovider", "--rootdir", str(tmp_path), str(path)],
        cwd=tmp_path, env=environment, capture_output=True, text=True,
        timeout=600)
    tail = (result.stdout + result.stderr)[-2000:]
    assert result.returncode == 0, tail
    assert " passed" in result.stdout or " skipped" in result.stdout, tail
    assert " failed" not in result.stdout, tail
