"""Sharding of one segmented problem over the GPUs of a node.

Segments are independent and their outputs disjoint, so the path shards with
no data-path collective: the offsets array is cut into contiguous segment
ranges balanced by element count, each rank keeps its slice of the values and
its rebased offsets resident on its own GPU and calls the single-GPU entry
points.  The reference is single-GPU (``python/swage/_runtime.py:146-151``
insists on the current device), so nothing here mirrors a reference function.

``gather_results`` is the optional exchange step: an all-gather of the
per-segment results (NCCL over NVLink on GPUs; gloo works for CPU tensors).
"""

from . import _runtime


def shard_cuts(host_offsets, shards):
    """Segment index where each shard begins (``shards + 1`` entries)."""
    from . import _native

    torch = _runtime._import_torch()
    if (
        not isinstance(host_offsets, torch.Tensor)
        or host_offsets.device.type != "cpu"
        or host_offsets.dtype != torch.int32
        or host_offsets.dim() != 1
        or not host_offsets.is_contiguous()
        or host_offsets.numel() < 1
    ):
        raise TypeError(
            "shard_cuts needs a contiguous rank-one CPU int32 offsets tensor"
        )
    if type(shards) is not int or shards < 1:
        raise ValueError("shards must be a positive integer")
    return _native.shard_offsets(
        host_offsets.data_ptr(), host_offsets.numel() - 1, shards
    )


def local_shard(host_offsets, cuts, rank):
    """Rebased offsets of shard ``rank`` and its value range ``[begin, end)``."""
    first, last = cuts[rank], cuts[rank + 1]
    begin = int(host_offsets[first])
    end = int(host_offsets[last])
    local = (host_offsets[first:last + 1] - begin).contiguous()
    return local, begin, end


def gather_results(local_output, cuts, group=None):
    """All-gather per-segment results; every rank gets all of them, in order.

    Shards hold different numbers of segments, so each rank pads to the
    longest shard, one ``all_gather_into_tensor`` moves the padded rows and
    the padding is dropped again.
    """
    torch = _runtime._import_torch()
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if len(cuts) != world + 1:
        raise ValueError("cuts must have world_size + 1 entries")
    counts = [cuts[g + 1] - cuts[g] for g in range(world)]
    if local_output.numel() < counts[rank]:
        raise ValueError("local output is shorter than this rank's shard")
    longest = max(counts) if counts else 0
    padded = local_output.new_zeros(longest)
    padded[:counts[rank]] = local_output[:counts[rank]]
    gathered = local_output.new_empty(world * longest)
    dist.all_gather_into_tensor(gathered, padded, group=group)
    rows = gathered.view(world, longest)
    return torch.cat([rows[g, :counts[g]] for g in range(world)])


__all__ = ["gather_results", "local_shard", "shard_cuts"]
