"""Sharding of one segmented problem over the GPUs of a node.

Segments are independent and their outputs disjoint, so the path shards with
no data-path collective: the offsets array is cut into contiguous segment
ranges balanced by element count, each rank keeps its slice of the values and
its rebased offsets resident on its own GPU and calls the single-GPU entry
points.  The reference is single-GPU (``python/swage/_runtime.py:146-151``
insists on the current device), so nothing here mirrors a reference function.

``gather_results`` is the optional exchange step as a collective: an
all-gather of the per-segment results (NCCL over NVLink on GPUs; gloo works
for CPU tensors).  ``PeerResults`` is the same exchange without a collective:
every rank stores its results straight into every rank's copy of the full
result array (plain stores into peer-mapped memory), one small kernel queued
behind the reduction.
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


class PeerResults:
    """Every rank's copy of the full per-segment result array, filled by the
    ranks themselves.

    Each rank owns one fp32 buffer of ``cuts[-1]`` results on its GPU and maps
    every other rank's buffer into its own address space (CUDA IPC over the
    handles exchanged with ``all_gather_object``).  ``publish(local_output)``
    queues ONE kernel on the current stream that stores this rank's
    ``cuts[rank + 1] - cuts[rank]`` results at their place in every copy --
    plain 128-bit stores over NVLink, no multicast, no load from peer memory,
    nothing waits on another GPU.  ``reduce(values, offsets, kind, plan)``
    goes one step further: the reduction's own warps store each result into
    every copy as they produce it.  ``wait()`` (synchronise the stream, then
    a host barrier) is when ``results`` is complete on every rank.

    One process per GPU, all on one node.  Collective: every rank of ``group``
    constructs, and later closes, its ``PeerResults`` together.  ``results``
    is a view of library-owned memory: it must not be used after ``close()``.
    """

    def __init__(self, cuts, group=None):
        from . import _native

        torch = _runtime._import_torch()
        import torch.distributed as dist

        self._dist = dist
        self._group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        cuts = [int(c) for c in cuts]
        if len(cuts) != self.world + 1 or cuts[0] != 0 or any(
                b < a for a, b in zip(cuts, cuts[1:])):
            raise ValueError(
                "cuts must be world_size + 1 nondecreasing segment indices "
                "starting at zero")
        self.cuts = cuts
        self.total = cuts[-1]
        self.device = torch.cuda.current_device()
        self._own, handle = _native.peer_buffer_create(4 * max(self.total, 4))
        self._mapped = {}
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self._bases = []
        for peer, peer_handle in enumerate(handles):
            if peer == self.rank:
                self._bases.append(self._own)
            else:
                self._mapped[peer] = _native.peer_buffer_open(peer_handle)
                self._bases.append(self._mapped[peer])
        self.results = _device_view(torch, self._own, self.total, self.device)
        dist.barrier(group)  # every mapping exists before anyone publishes

    def publish(self, local_output):
        """Queue the stores of this rank's results into every copy."""
        from . import _native

        torch = _runtime._import_torch()
        count = self.cuts[self.rank + 1] - self.cuts[self.rank]
        if (not isinstance(local_output, torch.Tensor)
                or local_output.dtype != torch.float32
                or not local_output.is_contiguous()
                or local_output.device.type != "cuda"
                or local_output.device.index != self.device):
            raise TypeError(
                "local output must be a contiguous fp32 tensor on this "
                "rank's GPU")
        if local_output.numel() < count:
            raise ValueError("local output is shorter than this rank's shard")
        if self._own is None:
            raise RuntimeError("the peer buffers are closed")
        stream = _runtime._current_stream(torch)
        _native.scatter_results(local_output.data_ptr(), count, self._bases,
                                self.cuts[self.rank], stream.cuda_stream)
        local_output.record_stream(stream)

    def reduce(self, values, offsets, kind, plan, schedule="auto"):
        """Reduce this rank's shard and store every result straight into every
        rank's copy, in ONE launch sequence (tile kernel + merge pass): the
        reducing warps themselves issue the stores over NVLink, so the
        exchange rides along with the reduction -- no collective and no copy
        kernel behind it.  ``values`` / ``offsets`` are this rank's shard
        (offsets rebased to zero, on its GPU), ``plan`` a ``SegmentPlan`` for
        them (``plan_segments``); the caller has validated the offsets (the
        plan was built from them).  Same bits as ``launch_gpu`` with that
        plan.  ``wait()`` as after ``publish``.
        """
        from . import _native
        from . import _segmented_qualification as runner

        torch = _runtime._import_torch()
        count = self.cuts[self.rank + 1] - self.cuts[self.rank]
        for name, tensor, dtype in (("values", values, torch.float32),
                                    ("offsets", offsets, torch.int32)):
            if (not isinstance(tensor, torch.Tensor) or tensor.dtype != dtype
                    or tensor.dim() != 1 or not tensor.is_contiguous()
                    or tensor.device.type != "cuda"
                    or tensor.device.index != self.device):
                raise TypeError(
                    f"{name} must be a contiguous rank-one {dtype} tensor on "
                    "this rank's GPU")
        if offsets.numel() != count + 1:
            raise ValueError(
                f"offsets describe {offsets.numel() - 1} segments, this "
                f"rank's shard has {count}")
        if kind in runner._KINDS:
            kind_code = runner._KINDS[kind]
        elif kind in runner._EXTENDED_KINDS:
            kind_code = runner._EXTENDED_KINDS[kind]
        else:
            raise ValueError("reduction kind must be 'sum', 'max' or 'min'")
        if not isinstance(plan, runner.SegmentPlan):
            raise TypeError("plan must be a SegmentPlan for these offsets")
        if self._own is None:
            raise RuntimeError("the peer buffers are closed")
        if count == 0:
            return
        runner._peek(plan)
        stream = _runtime._current_stream(torch)
        _native.segreduce_peers(
            kind_code, values.data_ptr(), offsets.data_ptr(), self._bases,
            self.cuts[self.rank], values.numel(), count, plan.handle,
            runner._schedule_code(schedule), stream.cuda_stream)
        for tensor in (values, offsets):
            tensor.record_stream(stream)

    def wait(self):
        """On return ``results`` holds every rank's published results."""
        torch = _runtime._import_torch()
        _runtime._current_stream(torch).synchronize()
        self._dist.barrier(self._group)

    def close(self):
        """Unmap the peers' buffers, then (after a barrier) free this rank's."""
        from . import _native

        if self._own is None:
            return
        torch = _runtime._import_torch()
        torch.cuda.synchronize()
        self.results = None
        for pointer in self._mapped.values():
            _native.peer_buffer_close(pointer)
        self._mapped = {}
        self._dist.barrier(self._group)  # nobody maps this buffer any more
        _native.peer_buffer_destroy(self._own)
        self._own = None
        self._bases = []


class _DeviceArray:
    """Describes library-owned device memory to ``torch.as_tensor``."""

    def __init__(self, pointer, count):
        self.__cuda_array_interface__ = {
            "shape": (count,), "typestr": "<f4", "data": (pointer, False),
            "version": 2, "strides": None,
        }


def _device_view(torch, pointer, count, device):
    if count == 0:
        return torch.empty(0, dtype=torch.float32, device=f"cuda:{device}")
    return torch.as_tensor(_DeviceArray(pointer, count),
                           device=f"cuda:{device}")


__all__ = ["PeerResults", "gather_results", "local_shard", "shard_cuts"]
