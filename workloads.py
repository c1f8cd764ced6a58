"""Seeded synthetic inputs with the shapes and distributions of the benchmark
configurations (the reference measures on no dataset; these stand in).

Offsets are drawn with numpy on the host (identical on every rank and
machine); values are drawn on the device with a seeded torch generator.  Used
by the parity tests, the smoke check and the benchmark -- not by the library.

Configurations (names as in the benchmark output):

``c1``  canonical: ``segments`` segments, lengths uniform in {0..2048}, values
        N(0, 1)                                   (default 4096 segments)
``c2``  vector add: n = 2**28 - 37, x, y ~ N(0, 1)
``c3``  lognormal lengths (mu 5, sigma 1.5, clipped to [1, 2**20]), 2**20
        segments, total capped at 2**30 by truncating trailing segments,
        values uniform in [-1e3, 1e3] with about 1 % of the positions of each
        segment overwritten by a copy of that segment's maximum
``c4``  softmax: 262144 segments, 50 % lengths in {1..32}, 40 % in
        {33..4096}, 10 % in {4097..65536}, values N(0, variance 4)
``c5``  extreme skew: 2**22 segments, 64 of length 2**23, 355 more long ones
        sharing what is left of 2**30 elements, every other length uniform in
        {0..8}, long segments placed by a seeded permutation, values N(0, 1)
"""

import numpy as np

SEEDS = {"c1": 1, "c2": 2, "c3": 3, "c4": 4, "c5": 5}


def _offsets(lengths):
    offsets = np.zeros(len(lengths) + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    assert offsets[-1] < (1 << 31), "total exceeds int32 offsets"
    return offsets.astype(np.int32)


def c1_offsets(segments=4096, seed=SEEDS["c1"]):
    rng = np.random.default_rng(seed)
    return _offsets(rng.integers(0, 2049, size=segments))


def c3_offsets(segments=1 << 20, cap=1 << 30, seed=SEEDS["c3"]):
    rng = np.random.default_rng(seed)
    lengths = np.rint(rng.lognormal(5.0, 1.5, size=segments))
    lengths = np.clip(lengths, 1, 1 << 20).astype(np.int64)
    total = np.cumsum(lengths)
    keep = int(np.searchsorted(total, cap, side="right"))
    return _offsets(lengths[:keep])


def c4_offsets(segments=262144, seed=SEEDS["c4"]):
    rng = np.random.default_rng(seed)
    bucket = rng.choice(3, size=segments, p=[0.5, 0.4, 0.1])
    low = np.array([1, 33, 4097])[bucket]
    high = np.array([32, 4096, 65536])[bucket]
    lengths = rng.integers(low, high + 1)
    return _offsets(lengths)


def c5_offsets(segments=1 << 22, total=1 << 30, giants=64,
               giant_length=1 << 23, seed=SEEDS["c5"]):
    """Scaled-down variants keep the proportions: pass smaller arguments."""
    rng = np.random.default_rng(seed)
    long_count = max(giants, int(round(segments * 1e-4)))
    lengths = rng.integers(0, 9, size=segments).astype(np.int64)
    where = rng.permutation(segments)[:long_count]
    lengths[where] = 0
    remainder = total - giants * giant_length - int(lengths.sum())
    larges = long_count - giants
    assert remainder >= 0, "giants do not fit in the total"
    lengths[where[:giants]] = giant_length
    if larges > 0:
        share = np.full(larges, remainder // larges, dtype=np.int64)
        share[: remainder % larges] += 1
        lengths[where[giants:]] = share
    else:
        lengths[where[0]] += remainder
    offsets = _offsets(lengths)
    assert int(offsets[-1]) == total
    return offsets


def normal_values(count, device, seed, scale=1.0):
    import torch

    generator = torch.Generator(device=device).manual_seed(seed)
    values = torch.randn(count, generator=generator, device=device,
                         dtype=torch.float32)
    if scale != 1.0:
        values *= scale
    return values


def c3_values(offsets, device, seed=SEEDS["c3"]):
    """U[-1e3, 1e3] with ~1 % per-segment duplicates of the segment maximum."""
    import torch

    count = int(offsets[-1])
    generator = torch.Generator(device=device).manual_seed(seed)
    values = torch.rand(count, generator=generator, device=device,
                        dtype=torch.float32)
    values = values * 2000.0 - 1000.0
    lengths = torch.from_numpy(np.diff(offsets).astype(np.int64)).to(device)
    peaks = torch.segment_reduce(values, "max", lengths=lengths)
    marks = torch.rand(count, generator=generator, device=device) < 0.01
    positions = torch.nonzero(marks).squeeze(1)
    bounds = torch.from_numpy(offsets.astype(np.int64)).to(device)
    owner = torch.searchsorted(bounds, positions, right=True) - 1
    values[positions] = peaks[owner]
    return values


def reduce_bytes(value_count, segment_count):
    """Algorithmic bytes of one segmented sum or max."""
    return 4 * value_count + 4 * (segment_count + 1) + 4 * segment_count


def softmax_bytes(value_count, segment_count):
    return 8 * value_count + 4 * (segment_count + 1)


def vadd_bytes(n):
    return 12 * n
