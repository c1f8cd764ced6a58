"""Regenerates the golden fixtures in this directory.

Run where a checkout of the reference is at hand:

    python tests/golden/make_golden.py PATH_TO_REFERENCE_CHECKOUT

Three fixtures are written:

* ``offset_validation.json`` -- what the REFERENCE's own ``_validate_offsets``
  and ``_validate_counts`` (``python/swage/_segmented_qualification.py:20-55``)
  return or raise for every case in ``tests/fakes.py::OFFSET_CASES``.  The
  reference's pure-Python package is imported and executed for this.
* ``launch_validation.json`` -- what the REFERENCE's own ``kernel.launch``
  (``python/swage/_runtime.py:47-180``) raises for every case in
  ``tests/fakes.py::LAUNCH_CASES`` when PyTorch is replaced by the metadata-only
  stand-in of ``tests/fakes.py`` (the same technique as the reference's
  ``tests/python/test_runtime.py:29-132``).  Only rejected launches and the
  empty launch are recorded: an accepted launch needs the reference's LLVM
  toolchain, which is not part of its source tree.
* ``segmented_known_answers.json`` -- the known answers the reference's tests
  hold for segmented sum/max, with expected outputs as exact float32 bit
  patterns:
    - ``test/Conversion/SwageToCPU/segmented-sum-runner.mlir:37-53,67-68``
    - ``python/tests/mlir/test_segmented_runtime.py:15-36`` (eight length
      cases, values ``((i % 17) - 8) / 4``): sums are computed in exact
      rational arithmetic -- every value is a multiple of 1/4 and every
      partial sum is far below 2**24 / 4, so ANY summation order, in fp32,
      gives exactly this number;
    - ``python/tests/mlir/test_segmented_runtime.py:151-181`` (NaN / -inf).
  The script cross-checks them against ``torch`` the way the reference's
  ``_pytorch_reference`` (:39-50) does.

The committed JSON files are what the tests read; this script is only needed
to regenerate them.
"""

import fractions
import json
import math
import pathlib
import struct
import sys

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import fakes  # noqa: E402


def bits(value):
    return struct.unpack("<I", struct.pack("<f", value))[0]


def outcome(call):
    try:
        result = call()
    except Exception as error:  # noqa: BLE001 - recording the behaviour
        return {"raises": type(error).__name__, "message": str(error)}
    return {"returns": result}


def offset_validation(reference):
    from swage import _segmented_qualification as runner

    cases = {}
    for name, offsets, value_count, output_count in fakes.OFFSET_CASES:
        cases[name] = {
            "offsets": offsets,
            "value_count": value_count,
            "output_count": True if output_count is True else output_count,
            "outcome": outcome(
                lambda: runner._validate_offsets(
                    list(offsets), value_count, output_count
                )
            ),
        }
    counts = {}
    for value_count, segment_count in [
        (0, 0), (-1, 0), (0, -1), (1 << 31, 0), (0, 1 << 31),
        ((1 << 31) - 1, (1 << 31) - 1), (True, 0), (1.0, 0),
    ]:
        counts[f"{value_count!r},{segment_count!r}"] = outcome(
            lambda: runner._validate_counts(value_count, segment_count)
        )
    return {"offsets": cases, "counts": counts}


def launch_validation(reference):
    import swage as sw
    import swage.language as sl

    @sw.jit
    def add_kernel(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):
        pid = sl.program_id(0)
        offsets = pid * BLOCK + sl.arange(0, BLOCK)
        mask = offsets < n
        x = sl.load(x_ptr + offsets, mask=mask, other=0.0)
        y = sl.load(y_ptr + offsets, mask=mask, other=0.0)
        sl.store(output_ptr + offsets, x + y, mask=mask)

    recorded = {}
    for case in fakes.LAUNCH_CASES:
        torch, _, arguments, constexprs, grid = fakes.build_launch_case(case)
        previous = sys.modules.get("torch")
        sys.modules["torch"] = torch
        try:
            result = outcome(
                lambda: add_kernel.launch(
                    arguments=arguments, constexprs=constexprs, grid=grid
                )
            )
        finally:
            if previous is None:
                del sys.modules["torch"]
            else:
                sys.modules["torch"] = previous
        if "message" in result:
            # strip the file:line:col prefix of source-located diagnostics
            marker = ": add_kernel: "
            if marker in result["message"]:
                result["message"] = result["message"].split(marker, 1)[1]
        recorded[case[0]] = result
    return recorded


LENGTH_CASES = {
    "empty": [0],
    "singleton": [1],
    "block-boundary": [128],
    "non-multiple": [129],
    "large": [4097],
    "uniform": [33, 33, 33, 33],
    "skewed": [1, 257, 2, 3837],
    "repeated-empty": [0, 2, 0, 0, 3],
}


def known_answers():
    import torch

    cases = {}
    for name, lengths in LENGTH_CASES.items():
        offsets = [0]
        for length in lengths:
            offsets.append(offsets[-1] + length)
        exact = [fractions.Fraction((i % 17) - 8, 4) for i in range(offsets[-1])]
        values = torch.tensor([float(v) for v in exact], dtype=torch.float32)
        sums, maxes = [], []
        for s in range(len(lengths)):
            piece = exact[offsets[s]:offsets[s + 1]]
            total = sum(piece, fractions.Fraction(0))
            assert float(total) == struct.unpack(
                "<f", struct.pack("<f", float(total)))[0]
            sums.append(bits(float(total)))
            maxes.append(bits(float(max(piece)) if piece else -math.inf))
            segment = values[offsets[s]:offsets[s + 1]]
            assert float(segment.sum()) == float(total)
            if piece:
                assert float(segment.max()) == float(max(piece))
        cases[name] = {
            "lengths": lengths,
            "values": "((i % 17) - 8) / 4",
            "sum_bits": sums,
            "max_bits": maxes,
        }
    literal = {
        "lit-sum-runner": {
            "values_bits": [bits(v) for v in (2.0, 3.0, 4.0, 5.0)],
            "offsets": [0, 0, 1, 4, 4],
            "kind": "sum",
            "expected_bits": [bits(v) for v in (0.0, 2.0, 12.0, 0.0)],
        },
        "nan-and-empty-max": {
            "values_bits": [bits(v) for v in
                            (1.0, math.nan, 3.0, 4.0, 5.0)],
            "offsets": [0, 3, 3, 5],
            "kind": "max",
            # NaN is compared as "is NaN" (the reference uses equal_nan)
            "expected_bits": [bits(math.nan), bits(-math.inf), bits(5.0)],
        },
    }
    return {"length_cases": cases, "literal_cases": literal}


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py PATH_TO_REFERENCE_CHECKOUT")
    reference = pathlib.Path(sys.argv[1])
    sys.path.insert(0, str(reference / "python"))
    written = {
        "offset_validation.json": offset_validation(reference),
        "launch_validation.json": launch_validation(reference),
        "segmented_known_answers.json": known_answers(),
    }
    for name, content in written.items():
        (HERE / name).write_text(json.dumps(content, indent=1, sort_keys=True)
                                 + "\n")
        print("wrote", HERE / name)


if __name__ == "__main__":
    main()
