"""A stand-in for PyTorch that lets launch validation run without CUDA.

Used by the CPU tests of this repository and by ``tests/golden/make_golden.py``
(which drives the reference's own ``launch`` with the same stand-in to record
its error behaviour).  Only the attributes the launch path reads exist.
"""

import types


class FakeDevice:
    def __init__(self, kind, index):
        self.type = kind
        self.index = index


class FakeTensor:
    """Metadata-only tensor; ``data_ptr`` reads are counted."""

    def __init__(self, torch, *, size=129, device="cuda", index=0, dtype=None,
                 rank=1, contiguous=True, pointer=0x1000):
        self.layout = torch.strided
        self.dtype = torch.float32 if dtype is None else dtype
        self.device = FakeDevice(device, index)
        self._size = size
        self._rank = rank
        self._contiguous = contiguous
        self._pointer = pointer
        self.pointer_reads = 0
        self.streams = []

    def dim(self):
        return self._rank

    def is_contiguous(self):
        return self._contiguous

    def numel(self):
        return self._size

    def data_ptr(self):
        self.pointer_reads += 1
        return self._pointer

    def record_stream(self, stream):
        self.streams.append(stream)


def fake_torch(*, available=True, current_device=0, max_threads=1024,
               capability=(10, 0)):
    torch = types.ModuleType("torch")
    torch.float32 = "fake.float32"
    torch.int32 = "fake.int32"
    torch.strided = "fake.strided"
    stream = types.SimpleNamespace(cuda_stream=0xABCD)
    properties = types.SimpleNamespace(max_threads_per_block=max_threads)
    torch.cuda = types.SimpleNamespace(
        is_available=lambda: available,
        current_device=lambda: current_device,
        current_stream=lambda: stream,
        get_device_capability=lambda _device=None: capability,
        get_device_properties=lambda _device=None: properties,
    )
    torch.version = types.SimpleNamespace(cuda="12.9")
    torch.Tensor = FakeTensor
    return torch, stream


def vector_add_arguments(torch, *, n=129, **tensor_options):
    return {
        "x_ptr": FakeTensor(torch, pointer=0x1000, **tensor_options),
        "y_ptr": FakeTensor(torch, pointer=0x2000, **tensor_options),
        "output_ptr": FakeTensor(torch, pointer=0x3000, **tensor_options),
        "n": n,
    }


# Launch-validation cases shared by the golden generator and the tests.
# Each: (name, tensor options, n, constexprs, grid, extra)
LAUNCH_CASES = [
    ("arguments-not-mapping", {}, 129, {"BLOCK": 128}, (2,),
     {"arguments": "bad"}),
    ("constexprs-not-mapping", {}, 129, "bad", (2,), {}),
    ("block-zero", {}, 129, {"BLOCK": 0}, (2,), {}),
    ("block-bool", {}, 129, {"BLOCK": True}, (2,), {}),
    ("block-missing", {}, 129, {}, (2,), {}),
    ("grid-list", {}, 129, {"BLOCK": 128}, [2], {}),
    ("grid-two", {}, 129, {"BLOCK": 128}, (2, 1), {}),
    ("grid-float", {}, 129, {"BLOCK": 128}, (2.0,), {}),
    ("grid-wrong", {}, 129, {"BLOCK": 128}, (1,), {}),
    ("block-over-limit", {}, 129, {"BLOCK": 2048}, (1,), {}),
    ("extra-constexpr", {}, 129, {"BLOCK": 128, "OTHER": 1}, (2,), {}),
    ("missing-argument", {}, 129, {"BLOCK": 128}, (2,), {"drop": "y_ptr"}),
    ("cpu-tensor", {"device": "cpu"}, 1, {"BLOCK": 128}, (1,), {}),
    ("other-device", {"index": 1}, 1, {"BLOCK": 128}, (1,), {}),
    ("rank-two", {"rank": 2}, 1, {"BLOCK": 128}, (1,), {}),
    ("non-contiguous", {"contiguous": False}, 1, {"BLOCK": 128}, (1,), {}),
    ("wrong-dtype", {"dtype": "fake.float64"}, 1, {"BLOCK": 128}, (1,), {}),
    ("n-over-length", {"size": 3}, 4, {"BLOCK": 128}, (1,), {}),
    ("n-negative", {}, -1, {"BLOCK": 128}, (1,), {}),
    ("n-too-large", {}, 1 << 31, {"BLOCK": 128}, (1,), {}),
    ("n-bool", {}, True, {"BLOCK": 128}, (1,), {}),
    ("n-float", {}, 4.0, {"BLOCK": 128}, (1,), {}),
    ("not-a-tensor", {}, 1, {"BLOCK": 128}, (1,), {"replace": ("x_ptr", 7)}),
    ("cuda-unavailable", {}, 129, {"BLOCK": 128}, (2,), {"available": False}),
    ("empty-launch", {"size": 0}, 0, {"BLOCK": 128}, (0,), {}),
]


def build_launch_case(case):
    """Return ``(torch, stream, arguments, constexprs, grid)`` for a case."""
    _, options, n, constexprs, grid, extra = case
    torch, stream = fake_torch(available=extra.get("available", True))
    arguments = vector_add_arguments(torch, n=n, **options)
    if "drop" in extra:
        del arguments[extra["drop"]]
    if "replace" in extra:
        name, value = extra["replace"]
        arguments[name] = value
    if "arguments" in extra:
        arguments = extra["arguments"]
    return torch, stream, arguments, constexprs, grid


OFFSET_CASES = [
    ("ok-simple", [0, 0, 1, 4, 4], 4, 4),
    ("ok-trailing-values", [0, 2], 5, 1),
    ("ok-bigger-output", [0, 2, 3], 3, 10),
    ("ok-single-zero", [0], 0, 0),
    ("empty-list", [], 0, 0),
    ("nonzero-start", [1, 1], 1, 1),
    ("negative", [0, -1], 1, 1),
    ("negative-start", [-1, 0], 1, 1),
    ("decreasing", [0, 2, 1], 2, 2),
    ("negative-after-decrease", [0, 5, -1], 5, 2),
    ("exceeds", [0, 2], 1, 1),
    ("output-small", [0, 1, 1], 1, 1),
    ("value-count-negative", [0, 0], -1, 1),
    ("value-count-large", [0, 0], 1 << 31, 1),
    ("output-count-bool", [0, 1], 1, True),
]
