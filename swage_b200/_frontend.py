"""``@jit`` capture, input validation and kernel recognition.

Drop-in for the launch-facing half of the reference's
``python/swage/_frontend.py``: ``jit`` (:744-746), ``_Kernel`` (:32-324) with
``launch`` (:84-93), ``__call__`` (:78-82), ``_validate_inputs`` (:115-227) and
the ``file:line:col: kernel: reason`` diagnostics of ``_raise`` (:319-324).

The reference turns the captured AST into MLIR (``_Emitter``, :327-732) and
lets the compiler decide whether the module is the canonical fixed-block
vector add (``lib/Conversion/FixedBlockToGPU/FixedBlockToGPU.cpp:62-175``).
Here there is no compiler: the body is reduced to a small symbolic term and
matched against the canonical programs this library has hand-written CUDA
kernels for.  Anything else is a ``CompilationError``; nothing is ever
executed or approximated.

Importing this module imports neither PyTorch nor the native library.
"""

import ast
import functools
import inspect
import textwrap
from collections.abc import Mapping
from typing import NamedTuple

from . import language


class CompilationError(Exception):
    """A source-located error in a kernel definition."""


class _Program(NamedTuple):
    """What a kernel body was recognised as.

    ``kind`` is one of ``vector_add``, ``segmented_sum``, ``segmented_max``,
    ``segmented_min`` or ``segmented_softmax``; ``roles`` maps the role of each
    runtime parameter (``x``, ``y``, ``out``, ``n`` or ``values``, ``offsets``,
    ``out``) to its name in the kernel signature.  ``map`` is set for a
    segmented reduction of mapped elements: ``(fn, scale, shift)`` with ``fn``
    one of ``identity``, ``abs``, ``square``, ``exp`` and the two constants as
    terms over literals and constexpr parameters (see ``constant_value``).
    """

    kind: str
    roles: dict
    map: tuple = None


def constant_value(term, constexprs):
    """Evaluate a constant term of a recognised map with the launch's
    constexpr values."""
    tag = term[0]
    if tag in ("int", "num"):
        return float(term[1])
    if tag == "static":
        return float(constexprs[term[1]])
    if tag == "neg":
        return -constant_value(term[1], constexprs)
    raise ValueError(f"not a constant term: {term!r}")


def _is_constexpr_annotation(node):
    if not isinstance(node, ast.Attribute) or node.attr != "constexpr":
        return False
    return isinstance(node.value, ast.Name) and node.value.id == "sl"


class _Kernel:
    """Captured kernel source; the Python body is never run."""

    def __init__(self, function):
        self.python_function = function
        self.filename = inspect.getsourcefile(function) or "<unknown>"
        name = function.__name__
        try:
            lines, self.source_line = inspect.getsourcelines(function)
        except (OSError, TypeError) as error:
            raise CompilationError(
                f"{self.filename}:1:1: {name}: source is unavailable"
            ) from error
        first = lines[0]
        self.source_indent = len(first) - len(first.lstrip())
        try:
            tree = ast.parse(textwrap.dedent("".join(lines)))
        except SyntaxError as error:
            line = self.source_line + (error.lineno or 1) - 1
            column = (error.offset or 1) + self.source_indent
            raise CompilationError(
                f"{self.filename}:{line}:{column}: {name}: {error.msg}"
            ) from error
        body = tree.body
        if len(body) != 1 or not isinstance(body[0], ast.FunctionDef):
            raise CompilationError(
                f"{self.filename}:{self.source_line}:"
                f"{self.source_indent + 1}: {name}: "
                "expected one function definition"
            )
        self.function = body[0]
        functools.update_wrapper(self, function)
        self._program = None
        for decorator in self.function.decorator_list:
            named_jit = isinstance(decorator, ast.Name) and decorator.id == "jit"
            dotted_jit = (
                isinstance(decorator, ast.Attribute) and decorator.attr == "jit"
            )
            if not (named_jit or dotted_jit):
                self._raise(decorator, "only @swage.jit may decorate a kernel")

    # -- public surface ----------------------------------------------------

    def __call__(self, *args, **kwargs):
        raise RuntimeError(
            f"Swage kernel '{self.__name__}' is not directly callable; "
            "use kernel.launch()"
        )

    def launch(self, *, arguments, constexprs, grid):
        """Validate, then queue the kernel on the current PyTorch stream.

        Keyword-only, asynchronous, returns ``None``; same contract as the
        reference's ``_Kernel.launch`` (``_frontend.py:84-93``).
        """
        from ._runtime import launch

        return launch(
            self, arguments=arguments, constexprs=constexprs, grid=grid
        )

    def emit_mlir(self, *, signature=None, arguments=None, constexprs):
        """Validate the inputs the way the reference does, then refuse.

        The reference returns a live ``mlir_swage`` module here
        (``_frontend.py:95-113``).  This library has no MLIR in it -- kernels
        are prebuilt sm_100a code -- so after the same input validation the
        call reports that compile-only emission is unavailable.
        """
        self._validate_inputs(signature, arguments, constexprs)
        raise RuntimeError(
            "emit_mlir is compile-only MLIR emission and needs the "
            "reference's mlir_swage bindings; this library launches "
            "prebuilt CUDA kernels instead (use kernel.launch())"
        )

    def recognize(self):
        """Match the body against the supported canonical programs."""
        if self._program is None:
            self._program = _Recognizer(self).run()
        return self._program

    # -- validation (reference: _frontend.py:115-298) -----------------------

    def _validate_inputs(self, signature, arguments, constexprs):
        if (signature is None) == (arguments is None):
            self._raise(
                self.function,
                "exactly one of signature or arguments is required",
            )
        explicit = signature is not None
        label = "signature" if explicit else "arguments"
        supplied = signature if explicit else arguments
        if not isinstance(supplied, Mapping):
            self._raise(self.function, f"{label} must be a mapping")
        if not isinstance(constexprs, Mapping):
            self._raise(self.function, "constexprs must be a mapping")
        if not all(isinstance(key, str) for key in supplied):
            self._raise(self.function, f"{label} keys must be strings")
        if not all(isinstance(key, str) for key in constexprs):
            self._raise(self.function, "constexprs keys must be strings")

        syntax = self.function.args
        rejected_forms = (
            (syntax.posonlyargs[:1], "positional-only parameters"),
            (syntax.kwonlyargs[:1], "keyword-only parameters"),
            ([syntax.vararg] if syntax.vararg else [],
             "variadic positional parameters"),
            ([syntax.kwarg] if syntax.kwarg else [],
             "variadic keyword parameters"),
        )
        for nodes, what in rejected_forms:
            if nodes:
                self._raise(nodes[0], f"{what} are unsupported")

        ordered = [argument.arg for argument in syntax.args]
        static_names = {
            argument.arg
            for argument in syntax.args
            if _is_constexpr_annotation(argument.annotation)
        }
        runtime_ordered = [name for name in ordered if name not in static_names]
        runtime_names = set(runtime_ordered)

        wrong_side = set(supplied) & static_names
        if wrong_side:
            self._raise(
                self.function,
                f"constexpr parameter '{min(wrong_side)}' must be passed "
                "in constexprs",
            )
        wrong_side = set(constexprs) & runtime_names
        if wrong_side:
            self._raise(
                self.function,
                f"runtime parameter '{min(wrong_side)}' must be passed in "
                f"{label}",
            )
        self._match_keys(label, "runtime parameters", set(supplied),
                         runtime_names)
        self._match_keys("constexprs", "constexpr parameters",
                         set(constexprs), static_names)

        if explicit:
            runtime_types = self._check_signature(signature, runtime_ordered)
        else:
            runtime_types = self._infer_signature(arguments, runtime_ordered)

        for name in ordered:
            if name not in static_names:
                continue
            value = constexprs[name]
            is_int = type(value) is int
            if name == "BLOCK" and (not is_int or value <= 0):
                self._raise(
                    self.function,
                    "constexpr 'BLOCK' must be a positive integer",
                )
            if not is_int:
                self._raise(
                    self.function, f"constexpr '{name}' must be an integer"
                )
            if value < -(1 << 63) or value > (1 << 63) - 1:
                if name == "BLOCK":
                    self._raise(
                        self.function,
                        "constexpr 'BLOCK' must fit a signed 64-bit MLIR "
                        "dimension",
                    )
                self._raise(
                    self.function,
                    f"constexpr '{name}' must fit signed 64-bit",
                )
        return runtime_types, dict(constexprs)

    def _match_keys(self, label, what, actual, expected):
        if actual == expected:
            return
        parts = []
        missing = sorted(expected - actual)
        extra = sorted(actual - expected)
        if missing:
            parts.append("missing: " + ", ".join(missing))
        if extra:
            parts.append("extra: " + ", ".join(extra))
        self._raise(
            self.function,
            f"{label} keys must match {what}; {'; '.join(parts)}",
        )

    def _check_signature(self, signature, runtime_ordered):
        for name in runtime_ordered:
            declared = signature[name]
            if declared is language.int32:
                continue
            if isinstance(declared, language._PointerType) and (
                declared.element_type is language.float32
                or declared.element_type is language.int32
            ):
                continue
            self._raise(
                self.function, f"unsupported type for parameter '{name}'"
            )
        return dict(signature)

    def _infer_signature(self, arguments, runtime_ordered):
        """Read dtype/rank/layout metadata only -- never a data pointer.

        Reference: ``_frontend.py:245-298``.  int32 rank-one tensors are
        accepted in addition (they are the CSR offsets of segment kernels).
        """
        try:
            import torch

            float32, int32 = torch.float32, getattr(torch, "int32", None)
            strided, tensor_type = torch.strided, torch.Tensor
        except Exception:
            self._raise(
                self.function,
                "PyTorch metadata inference requires "
                "'swage-compiler[pytorch]'",
            )
        inferred = {}
        for name in runtime_ordered:
            value = arguments[name]
            if type(value) is int and -(1 << 31) <= value < (1 << 31):
                inferred[name] = language.int32
                continue
            if not isinstance(value, tensor_type):
                self._raise(
                    self.function,
                    f"unsupported argument for parameter '{name}'",
                )
            try:
                facts = (
                    value.layout,
                    value.dtype,
                    value.dim(),
                    value.device.type,
                    value.is_contiguous(),
                )
            except Exception:
                self._raise(
                    self.function,
                    f"could not read PyTorch metadata for parameter "
                    f"'{name}'; install 'swage-compiler[pytorch]'",
                )
            layout, dtype, rank, device_type, contiguous = facts
            element = None
            if dtype == float32:
                element = language.float32
            elif int32 is not None and dtype == int32:
                element = language.int32
            problem = None
            if layout != strided:
                problem = f"layout {layout}"
            elif element is None:
                problem = f"dtype {dtype}"
            elif rank != 1:
                problem = f"rank {rank}"
            elif device_type not in ("cpu", "cuda"):
                problem = f"device type '{device_type}'"
            elif not contiguous:
                problem = "non-contiguous"
            if problem is not None:
                self._raise(
                    self.function,
                    f"unsupported argument for parameter '{name}': {problem}",
                )
            inferred[name] = language.pointer(element)
        return inferred

    def _raise(self, node, reason):
        line = self.source_line + node.lineno - 1
        column = node.col_offset + self.source_indent + 1
        raise CompilationError(
            f"{self.filename}:{line}:{column}: {self.__name__}: {reason}"
        )


# ---------------------------------------------------------------------------
# Recognition of the canonical programs
# ---------------------------------------------------------------------------
#
# The body is evaluated symbolically into nested tuples ("terms"):
#   ("param", name) | ("static", name) | ("int", v) | ("pid",) | ("lanes",)
#   ("add", a, b) | ("mul", a, b) | ("sub", a, b) | ("div", a, b) | ("lt", a, b)
#   ("load", address, mask) | ("sid",) | ("segment", values, offsets, index)
#   ("elements", segment) | ("max", x) | ("min", x) | ("sum", x) | ("exp", x)
#   ("abs", x) | ("neg", x) | ("num", v)
# and a list of effects ("store", address, value, mask) or
# ("store_segment", pointer, segment, value).  Matching is then plain tuple
# comparison against the canonical forms below.

_SEGMENT_CALLS = {
    "segment_id", "segment", "load_segment", "store_segment", "max", "min",
    "sum", "exp", "abs",
}


class _Recognizer:
    def __init__(self, kernel):
        self.kernel = kernel
        arguments = kernel.function.args.args
        self.static = {
            argument.arg
            for argument in arguments
            if _is_constexpr_annotation(argument.annotation)
        }
        self.runtime = [a.arg for a in arguments if a.arg not in self.static]
        self.names = {name: ("param", name) for name in self.runtime}
        self.effects = []

    def fail(self, node, reason):
        self.kernel._raise(node, reason)

    def run(self):
        body = self.kernel.function.body
        for statement in body[:-1]:
            if isinstance(statement, ast.Return):
                self.fail(statement, "empty return must be the final statement")
        for statement in body:
            self.statement(statement)
        return self.classify()

    # -- statements -----------------------------------------------------

    def statement(self, node):
        if isinstance(node, ast.Assign):
            single = len(node.targets) == 1 and isinstance(
                node.targets[0], ast.Name
            )
            if not single:
                self.fail(node, "only single-name assignments are supported")
            target = node.targets[0]
            if target.id in self.static:
                self.fail(
                    target,
                    f"cannot assign to constexpr parameter '{target.id}'",
                )
            self.names[target.id] = self.term(node.value)
        elif isinstance(node, ast.Expr):
            call = node.value
            name = _call_name(call) if isinstance(call, ast.Call) else None
            if name == "store":
                self.store(call)
            elif name == "store_segment":
                self.store_segment(call)
            elif isinstance(call, ast.Constant) and isinstance(call.value, str):
                return  # docstring
            else:
                self.fail(node, "only sl.store may be used as a statement")
        elif isinstance(node, ast.Return):
            if node.value is not None:
                self.fail(node, "return values are unsupported")
        else:
            self.fail(node, f"unsupported statement '{type(node).__name__}'")

    # -- expressions ----------------------------------------------------

    def term(self, node):
        if isinstance(node, ast.Name):
            if node.id in self.names:
                return self.names[node.id]
            if node.id in self.static:
                return ("static", node.id)
            self.fail(node, f"unknown name '{node.id}'")
        if isinstance(node, ast.Constant) and type(node.value) is int:
            return ("int", node.value)
        if isinstance(node, ast.Constant) and type(node.value) is float:
            return ("num", node.value)
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
            return ("neg", self.term(node.operand))
        if isinstance(node, ast.BinOp):
            operators = {ast.Add: "add", ast.Mult: "mul", ast.Sub: "sub",
                         ast.Div: "div"}
            tag = operators.get(type(node.op))
            if tag is None:
                self.fail(
                    node,
                    f"unsupported binary operator '{type(node.op).__name__}'",
                )
            return (tag, self.term(node.left), self.term(node.right))
        if isinstance(node, ast.Compare):
            if len(node.ops) != 1 or not isinstance(node.ops[0], ast.Lt):
                self.fail(node, "only a single '<' comparison is supported")
            return ("lt", self.term(node.left), self.term(node.comparators[0]))
        if isinstance(node, ast.Call):
            return self.call(node)
        self.fail(node, f"unsupported expression '{type(node).__name__}'")

    def keywords(self, node):
        if any(keyword.arg is None for keyword in node.keywords):
            self.fail(node, "keyword expansion is unsupported")
        seen = {}
        for keyword in node.keywords:
            if keyword.arg in seen:
                self.fail(node, "duplicate keyword argument")
            seen[keyword.arg] = keyword.value
        return seen

    def call(self, node):
        name = _call_name(node)
        if name == "store":
            self.fail(
                node, "sl.store is only supported as an expression statement"
            )
        if name == "program_id" or name == "segment_id":
            if node.keywords or len(node.args) != 1:
                self.fail(node, f"sl.{name} expects one axis literal")
            axis = node.args[0]
            if (
                not isinstance(axis, ast.Constant)
                or type(axis.value) is not int
                or axis.value < 0
            ):
                self.fail(
                    axis, f"{name} axis must be a nonnegative integer"
                )
            if axis.value != 0:
                self.fail(axis, f"only sl.{name} axis 0 is supported")
            return ("pid",) if name == "program_id" else ("sid",)
        if name == "arange":
            if node.keywords or len(node.args) != 2:
                self.fail(node, "sl.arange expects start and end")
            start, end = node.args
            canonical = (
                isinstance(start, ast.Constant)
                and type(start.value) is int
                and start.value == 0
                and isinstance(end, ast.Name)
                and end.id == "BLOCK"
            )
            if not canonical:
                self.fail(node, "only sl.arange(0, BLOCK) is supported")
            if "BLOCK" not in self.static:
                self.fail(node, "BLOCK is required for vector operations")
            return ("lanes",)
        if name == "load":
            options = self.keywords(node)
            if len(node.args) != 1 or set(options) != {"mask", "other"}:
                self.fail(
                    node, "sl.load expects address, mask=..., and other=..."
                )
            other = options["other"]
            if not isinstance(other, ast.Constant) or type(other.value) not in (
                int, float,
            ):
                self.fail(other, "sl.load other must be a numeric literal")
            address = self.term(node.args[0])
            if not _is_address(address):
                self.fail(node.args[0], "sl.load requires pointer + offsets")
            return ("load", address, self.term(options["mask"]))
        if name in _SEGMENT_CALLS:
            if node.keywords:
                self.fail(node, f"sl.{name} takes positional arguments only")
            arity = {"segment": 3}.get(name, 1)
            if len(node.args) != arity:
                self.fail(node, f"sl.{name} expects {arity} argument(s)")
            operands = tuple(self.term(argument) for argument in node.args)
            tag = "elements" if name == "load_segment" else name
            return (tag,) + operands
        self.fail(node, "unsupported call")

    def store(self, node):
        options = self.keywords(node)
        if len(node.args) != 2 or set(options) - {"mask"}:
            self.fail(node, "sl.store expects address, value, and mask=...")
        address = self.term(node.args[0])
        if not _is_address(address):
            self.fail(node.args[0], "sl.store requires pointer + offsets")
        mask = self.term(options["mask"]) if "mask" in options else None
        self.effects.append(("store", address, self.term(node.args[1]), mask))

    def store_segment(self, node):
        if node.keywords or len(node.args) != 3:
            self.fail(
                node, "sl.store_segment expects pointer, segment, and value"
            )
        pointer, segment, value = (self.term(a) for a in node.args)
        self.effects.append(("store_segment", pointer, segment, value))

    # -- matching -------------------------------------------------------

    def classify(self):
        function = self.kernel.function
        if len(self.effects) != 1:
            self.fail(function, "expected exactly one store in the kernel")
        effect = self.effects[0]
        program = self._vector_add(effect) or self._segmented(effect)
        if program is None:
            self.fail(
                function,
                "kernel is not one of the supported programs: fixed-block "
                "vector add, segmented sum, segmented max, segmented softmax",
            )
        return program

    def _vector_add(self, effect):
        if effect[0] != "store" or len(self.runtime) != 4:
            return None
        x, y, out, n = (("param", name) for name in self.runtime)
        # offsets = program_id(0) * BLOCK + arange(0, BLOCK); mask = offsets < n
        # (FixedBlockToGPU.cpp:62-84: program id on the left of the multiply,
        # the lane step on the right of the add, signed '<' against n)
        offsets = ("add", ("mul", ("pid",), ("static", "BLOCK")), ("lanes",))
        mask = ("lt", offsets, n)
        wanted = (
            "store",
            ("add", out, offsets),
            ("add", ("load", ("add", x, offsets), mask),
             ("load", ("add", y, offsets), mask)),
            mask,
        )
        if effect != wanted:
            return None
        return _Program(
            "vector_add",
            dict(zip(("x", "y", "out", "n"), self.runtime)),
        )

    def _segmented(self, effect):
        if len(self.runtime) != 3:
            return None
        values, offsets, out = (("param", name) for name in self.runtime)
        segment = ("segment", values, offsets, ("sid",))
        x = ("elements", segment)
        roles = dict(zip(("values", "offsets", "out"), self.runtime))
        for kind in ("sum", "max", "min"):
            if effect[:2] != ("store", ("add", out, ("sid",))):
                break
            reduced = effect[2]
            if effect[3] is not None or reduced[0] != kind or (
                    len(reduced) != 2):
                continue
            if reduced[1] == x and not self.static:
                return _Program(f"segmented_{kind}", roles)
            element_map = _match_map(reduced[1], x)
            if element_map is not None and element_map[0] is not None:
                return _Program(f"segmented_{kind}", roles, element_map)
        if self.static:
            return None
        # softmax in the reference's semantic form
        # (test/Dialect/Swage/softmax.mlir:13-31): max, sum of exp(x - max),
        # exp(x - max) / sum, stored over the segment's own range.
        numerator = ("exp", ("sub", x, ("max", x)))
        wanted = (
            "store_segment", out, segment,
            ("div", numerator, ("sum", numerator)),
        )
        if effect == wanted:
            return _Program("segmented_softmax", roles)
        return None


def _is_constant(term):
    """A literal, a constexpr parameter, or the negation of one."""
    if not isinstance(term, tuple):
        return False
    if term[0] in ("int", "num", "static"):
        return True
    return term[0] == "neg" and _is_constant(term[1])


def _match_affine(term, x):
    """``(scale, shift)`` as constant terms when ``term`` is one of the exact
    affine forms of ``x`` -- ``x``, ``-x``, ``x * c``, ``c * x``, each
    optionally ``+ d``, ``d +`` or ``- d`` -- else ``None``.  Only forms whose
    fp32 evaluation IS one multiply and one add are taken: nothing is
    reassociated (``(x - c) * d`` is not ``x * d - c * d`` in fp32), so the
    kernel's arithmetic is the expression's.  A missing shift is ``-0.0``,
    which leaves every value, signed zeros included, as it is."""
    one, no_shift = ("num", 1.0), ("num", -0.0)

    def scaled(t):
        if t == x:
            return one
        if t == ("neg", x):
            return ("num", -1.0)
        if t[0] == "mul" and t[1] == x and _is_constant(t[2]):
            return t[2]
        if t[0] == "mul" and t[2] == x and _is_constant(t[1]):
            return t[1]
        return None

    if not isinstance(term, tuple):
        return None
    scale = scaled(term)
    if scale is not None:
        return scale, no_shift
    if term[0] == "add":
        for product, constant in ((term[1], term[2]), (term[2], term[1])):
            scale = scaled(product) if isinstance(product, tuple) else None
            if scale is not None and _is_constant(constant):
                return scale, constant
    if term[0] == "sub" and isinstance(term[1], tuple):
        scale = scaled(term[1])
        if scale is not None and _is_constant(term[2]):
            return scale, ("neg", term[2])
    return None


def _match_map(term, x):
    """``(fn, scale, shift)`` when ``term`` is ``A``, ``sl.abs(A)``,
    ``sl.exp(A)`` or ``A * A`` with ``A`` an affine form of the segment's
    elements ``x`` (see ``_match_affine``); ``None`` otherwise."""
    if not isinstance(term, tuple):
        return None
    function, inner = "identity", term
    if term[0] in ("abs", "exp") and len(term) == 2:
        function, inner = term[0], term[1]
    elif term[0] == "mul" and term[1] == term[2] and not _is_constant(term[1]):
        function, inner = "square", term[1]
    affine = _match_affine(inner, x)
    if affine is None:
        return None
    return (function,) + affine


def _call_name(node):
    target = node.func
    if (
        isinstance(target, ast.Attribute)
        and isinstance(target.value, ast.Name)
        and target.value.id == "sl"
    ):
        return target.attr
    return None


def _is_address(term):
    return (
        isinstance(term, tuple)
        and term[0] == "add"
        and isinstance(term[1], tuple)
        and term[1][0] == "param"
    )


def jit(function):
    """Capture ``function`` as a non-executing kernel."""
    return _Kernel(function)


__all__ = ["CompilationError", "jit"]
