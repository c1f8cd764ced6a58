"""Markers of the restricted kernel language (drop-in for ``swage.language``).

Same public names and meaning as the reference's ``python/swage/language.py``
(:41-86): ``constexpr``, ``float32``, ``int32``, ``pointer()`` describe
parameters; ``program_id``, ``arange``, ``load`` and ``store`` only have a
meaning inside an ``@jit`` body, which is parsed and never executed, so
calling them from ordinary Python raises ``RuntimeError``.

The segment-local names sketched in the reference's README (:74-86) --
``segment_id``, ``segment``, ``load_segment``, ``max``, ``exp``, ``sum``,
``store_segment`` -- are provided as well so segmented sum, max and softmax
kernels can be written against the same surface; the reference itself does
not define them yet.
"""


class _ScalarType:
    """A scalar element type; instances are compared by identity."""

    __slots__ = ("value",)

    def __init__(self, value):
        self.value = value

    def __repr__(self):
        return f"swage.language.{self.value}"


class _Marker:
    """A parameter marker that is not a runtime type."""

    __slots__ = ("value",)

    def __init__(self, value):
        self.value = value

    def __repr__(self):
        return f"swage.language.{self.value}"


class _PointerType:
    """Pointer-to-scalar descriptor used in explicit kernel signatures."""

    __slots__ = ("element_type",)

    def __init__(self, element_type):
        self.element_type = element_type

    def __eq__(self, other):
        if not isinstance(other, _PointerType):
            return False
        return other.element_type is self.element_type

    def __hash__(self):
        return hash(("pointer", id(self.element_type)))

    def __repr__(self):
        return f"pointer({self.element_type.value})"


constexpr = _Marker("constexpr")
float32 = _ScalarType("float32")
int32 = _ScalarType("int32")


def pointer(element_type):
    """Describe a pointer to ``element_type``."""
    return _PointerType(element_type)


def _outside_kernel(name):
    raise RuntimeError(
        f"swage.language.{name} is only available inside @swage.jit kernels"
    )


def program_id(axis):
    """Logical program coordinate (symbolic)."""
    _outside_kernel("program_id")


def arange(start, end):
    """Compile-time sized index vector (symbolic)."""
    _outside_kernel("arange")


def load(pointer_value, *, mask=None, other=None):
    """Masked vector load (symbolic)."""
    _outside_kernel("load")


def store(pointer_value, value, *, mask=None):
    """Masked vector store (symbolic)."""
    _outside_kernel("store")


def segment_id(axis):
    """Logical segment coordinate (symbolic)."""
    _outside_kernel("segment_id")


def segment(values_pointer, offsets_pointer, index):
    """The dense range values[offsets[index]:offsets[index + 1]] (symbolic)."""
    _outside_kernel("segment")


def load_segment(segment_value):
    """All elements of a segment (symbolic)."""
    _outside_kernel("load_segment")


def store_segment(pointer_value, segment_value, value):
    """Write one value per element into the segment's own range (symbolic)."""
    _outside_kernel("store_segment")


def max(value):  # noqa: A001 - name fixed by the kernel language
    """NaN-propagating maximum over a segment (symbolic)."""
    _outside_kernel("max")


def min(value):  # noqa: A001 - name fixed by the kernel language
    """NaN-propagating minimum over a segment (symbolic).  An extension: the
    reference's dialect has ``kind<min>``, its frontend and lowering do not."""
    _outside_kernel("min")


def sum(value):  # noqa: A001 - name fixed by the kernel language
    """Sum over a segment (symbolic)."""
    _outside_kernel("sum")


def exp(value):
    """Elementwise exponential (symbolic)."""
    _outside_kernel("exp")


def abs(value):  # noqa: A001 - name fixed by the kernel language
    """Elementwise absolute value (symbolic).  An extension: usable in front
    of a segment reduction (a ``swage.map`` region feeding ``swage.reduce``),
    which the reference's lowering does not accept."""
    _outside_kernel("abs")


__all__ = [
    "abs",
    "arange",
    "constexpr",
    "exp",
    "float32",
    "int32",
    "load",
    "load_segment",
    "max",
    "min",
    "pointer",
    "program_id",
    "segment",
    "segment_id",
    "store",
    "store_segment",
    "sum",
]
