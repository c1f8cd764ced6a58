"""swage_b200: B200-native segmented sum / max / softmax and vector add.

Same public surface as the reference's ``swage`` package
(``python/swage/__init__.py:4-8``): ``jit`` and ``CompilationError``, with the
kernel language in ``swage_b200.language``.  Importing the package imports
neither PyTorch nor the native library.

``install_as("swage")`` registers this package under another module name so
code written as ``import swage as sw; import swage.language as sl`` runs
unchanged.
"""

import sys

from ._frontend import CompilationError, jit

__version__ = "0.1.0"


def install_as(name="swage"):
    """Alias this package (and its submodules) under ``name`` in sys.modules."""
    import importlib

    package = sys.modules[__name__]
    sys.modules[name] = package
    for submodule in ("language", "_frontend", "_runtime",
                      "_segmented_qualification", "env"):
        module = importlib.import_module(f"{__name__}.{submodule}")
        sys.modules[f"{name}.{submodule}"] = module
    return package


__all__ = ["CompilationError", "install_as", "jit"]
