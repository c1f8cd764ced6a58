"""Offsets validation, planner and sharding: host logic only (no GPU)."""

import json
import pathlib

import numpy as np
import pytest
import torch

from swage_b200 import _native
from swage_b200._segmented_qualification import (
    _validate_counts,
    _validate_host_offsets,
    _validate_offsets,
    _validate_tensors,
)

GOLDEN = json.loads(
    (pathlib.Path(__file__).parent / "golden" / "offset_validation.json")
    .read_text())


def expect(outcome, call):
    if "raises" in outcome:
        with pytest.raises(Exception) as caught:
            call()
        assert type(caught.value).__name__ == outcome["raises"]
        assert str(caught.value) == outcome["message"]
    else:
        assert call() == outcome["returns"]


@pytest.mark.parametrize("name", sorted(GOLDEN["offsets"]))
def test_list_validation_matches_the_reference(name):
    case = GOLDEN["offsets"][name]
    expect(case["outcome"], lambda: _validate_offsets(
        list(case["offsets"]), case["value_count"], case["output_count"]))


@pytest.mark.parametrize("name", sorted(GOLDEN["offsets"]))
def test_native_validation_matches_the_reference(name, native_library):
    case = GOLDEN["offsets"][name]
    if not case["offsets"] or case["output_count"] is True:
        pytest.skip("not expressible as an int32 tensor / int count")
    host = torch.tensor(case["offsets"], dtype=torch.int32)
    expect(case["outcome"], lambda: _validate_host_offsets(
        host, case["value_count"], case["output_count"]))


@pytest.mark.parametrize("key", sorted(GOLDEN["counts"]))
def test_count_validation_matches_the_reference(key):
    value_count, segment_count = eval(key)  # noqa: S307 - fixture literals
    expect(GOLDEN["counts"][key],
           lambda: _validate_counts(value_count, segment_count))


def test_tensor_metadata_is_validated_before_any_device_access(native_library):
    values, output = torch.empty(2), torch.empty(1)
    with pytest.raises(TypeError, match="offsets must have dtype torch.int32"):
        _validate_tensors(values, torch.tensor([0, 2]), output)
    with pytest.raises(TypeError, match="offsets must have rank one"):
        _validate_tensors(values, torch.tensor([[0, 2]], dtype=torch.int32),
                          output)
    with pytest.raises(ValueError, match="output has 1 elements"):
        _validate_tensors(values, torch.tensor([0, 1, 2], dtype=torch.int32),
                          output)
    with pytest.raises(TypeError, match="values must have dtype"):
        _validate_tensors(values.double(),
                          torch.tensor([0, 2], dtype=torch.int32), output)
    with pytest.raises(ValueError, match="values must be contiguous"):
        _validate_tensors(torch.empty(4)[::2],
                          torch.tensor([0, 2], dtype=torch.int32), output)
    with pytest.raises(TypeError, match="values must be a torch.Tensor"):
        _validate_tensors([1.0], torch.tensor([0, 1], dtype=torch.int32),
                          output)
    assert _validate_tensors(
        values, torch.tensor([0, 2], dtype=torch.int32), output,
        require_cuda=False) == (2, 1)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA is unavailable"):
            _validate_tensors(values, torch.tensor([0, 2], dtype=torch.int32),
                              output)


def _plan(lengths):
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    tasks, info = _native.plan_host_tasks(offsets.ctypes.data, len(lengths))
    return offsets, tasks, info


def check_tasks_cover_everything(offsets, tasks, info):
    """Every value belongs to exactly one task; every segment is either whole
    in one packed task or cut into pieces with consecutive partial slots."""
    segments = len(offsets) - 1
    whole = np.zeros(segments, dtype=np.int64)
    covered = np.zeros(int(offsets[-1]) + 1, dtype=np.int64)
    tile, items = info["tile_values"], info["tile_items"]
    pieces = {}
    links = {}  # segment -> what its tasks say about its slots
    for (seg, count, vbegin, vcount, kind, head, tail, link_first,
         link_pieces) in tasks:
        assert 0 <= vcount <= tile
        covered[vbegin] += 1
        covered[vbegin + vcount] -= 1
        vend = vbegin + vcount
        if kind == 0:
            assert 1 <= count <= info["tile_max_segments"]
            assert vcount + count <= items
            assert not (count == 1 and head >= 0 and tail >= 0)
            last = seg + count - 1
            first_whole, last_whole = seg, last
            if head >= 0:  # began in an earlier task
                assert offsets[seg] < vbegin
                end = min(int(offsets[seg + 1]), vend)
                pieces.setdefault(seg, []).append((vbegin, end - vbegin, head))
                links.setdefault(seg, []).append(("first", link_first))
                first_whole = seg + 1
            else:
                assert offsets[seg] == vbegin
            if tail >= 0:  # continues in a later task
                assert offsets[last + 1] > vend
                start = max(int(offsets[last]), vbegin)
                pieces.setdefault(last, []).append((start, vend - start, tail))
                links.setdefault(last, []).append(("pieces", link_pieces))
                last_whole = last - 1
            else:
                assert offsets[last + 1] == vend
            whole[first_whole:last_whole + 1] += 1
        else:
            assert kind == 1 and head == -1 and tail == -1
            assert offsets[seg] <= vbegin and vend <= offsets[seg + 1]
            if count < 0:
                assert offsets[seg] == vbegin and offsets[seg + 1] == vend
                whole[seg] += 1
            else:
                pieces.setdefault(seg, []).append((vbegin, vcount, count))
                links.setdefault(seg, []).append(("first", link_first))
                links.setdefault(seg, []).append(("pieces", link_pieces))
    for seg, parts in pieces.items():
        assert whole[seg] == 0
        whole[seg] += 1
        parts.sort()
        assert len(parts) >= 2
        assert parts[0][0] == offsets[seg]
        assert parts[-1][0] + parts[-1][1] == offsets[seg + 1]
        for (b0, c0, _), (b1, _, _) in zip(parts, parts[1:]):
            assert b0 + c0 == b1
        slots = [slot for _, _, slot in parts]
        assert slots == list(range(slots[0], slots[0] + len(slots)))
        # every piece knows where the segment's slots begin and how many
        # pieces there are: what the in-kernel merge goes by
        for what, said in links[seg]:
            assert said == (slots[0] if what == "first" else len(slots))
    assert np.all(whole == 1)
    assert np.all(np.cumsum(covered)[:-1] == 1)
    assert info["tasks"] == len(tasks)
    assert info["split_segments"] == len(pieces)
    assert info["partial_slots"] == sum(len(p) for p in pieces.values())
    assert sum(info["histogram"]) == segments
    assert sum(info["elements_in_bin"]) == int(offsets[-1])


@pytest.mark.parametrize("lengths", [
    [0], [1], [128], [129], [4097], [33, 33, 33, 33], [1, 257, 2, 3837],
    [0, 2, 0, 0, 3], [0] * 5000, [8192], [8193], [2048, 2049, 1, 0, 100000],
    [1024, 1025, 2047, 2048, 2049, 2050, 4095, 4096, 4097],
    [2031, 2032, 2033, 1, 2030, 2, 129, 1900, 130, 1901, 128, 1903],
    [300] * 200, [1500, 700] * 50, [2000, 31, 2000, 33, 2000, 160],
    [3] * 10000,
], ids=str)
def test_planner_tasks_partition_the_input(lengths, native_library):
    offsets, tasks, info = _plan(lengths)
    check_tasks_cover_everything(offsets, tasks, info)


def test_planner_on_random_skewed_lengths(native_library):
    rng = np.random.default_rng(3)
    lengths = rng.integers(0, 9, size=20000)
    lengths[rng.choice(20000, 5, replace=False)] = rng.integers(
        10_000, 300_000, size=5)
    offsets, tasks, info = _plan(lengths)
    check_tasks_cover_everything(offsets, tasks, info)
    assert info["max_length"] == int(lengths.max())
    assert info["split_segments"] >= 5
    # short bins hold the many tiny segments
    assert sum(info["histogram"][:5]) == 20000 - 5


def test_planner_rejects_bad_offsets(native_library):
    bad = np.array([0, 3, 2], dtype=np.int32)
    with pytest.raises(RuntimeError, match="SWG_ERR_INVALID_OFFSETS"):
        _native.plan_host_tasks(bad.ctypes.data, 2)


@pytest.mark.parametrize("shards", [1, 2, 3, 4, 8])
def test_sharding_is_contiguous_and_element_balanced(shards, native_library):
    rng = np.random.default_rng(9)
    lengths = rng.integers(0, 9, size=50000)
    lengths[rng.choice(50000, 12, replace=False)] = 40000
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    cuts = _native.shard_offsets(offsets.ctypes.data, len(lengths), shards)
    assert cuts[0] == 0 and cuts[-1] == len(lengths)
    assert all(a <= b for a, b in zip(cuts, cuts[1:]))
    sizes = [int(offsets[b] - offsets[a]) for a, b in zip(cuts, cuts[1:])]
    assert sum(sizes) == int(offsets[-1])
    ideal = offsets[-1] / shards
    # a cut can be off by at most half of the segment it falls into
    assert max(abs(s - ideal) for s in sizes) <= 40000


def test_sharding_edge_cases(native_library):
    offsets = np.array([0, 0, 0, 0], dtype=np.int32)
    assert _native.shard_offsets(offsets.ctypes.data, 3, 2)[-1] == 3
    one = np.array([0, 10], dtype=np.int32)
    cuts = _native.shard_offsets(one.ctypes.data, 1, 4)
    assert cuts[0] == 0 and cuts[-1] == 1 and sorted(cuts) == cuts
    with pytest.raises(RuntimeError, match="SWG_ERR_INVALID_ARGUMENT"):
        _native.shard_offsets(one.ctypes.data, 1, 0)
