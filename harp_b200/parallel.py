"""Data-parallel plumbing: batch sharding and gradient / partial-result all-reduce.

The reference has no distributed code at all (no collective call site, Rc-based
single-thread graph: src/graph/node.rs:222).  The sharded paths here are new:
one process per GPU, `torch.distributed` for rendezvous and the collectives
(NCCL on GPUs, gloo in the CPU tests), the library's own stream for ordering.
Every rank runs the same kernel list on its shard; the only exchange of a
training step is the SUM all-reduce of the gradients between backward and the
parameter update (learning rate divided by the world size = gradient mean), and
for sharded reductions the all-reduce of the per-rank partial results.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import numpy as np


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [lo, hi) of `n` items owned by `rank` (sizes differ by at most 1)."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class _CudaAlias:
    """Zero-copy view of a device buffer for torch (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, nelem: int):
        self.__cuda_array_interface__ = {"shape": (nelem,), "typestr": "<f4", "data": (ptr, False), "version": 3}


def make_allreduce(buffers: Sequence, op: str = "sum", device=None, local_rank: int = 0) -> Callable[[], None]:
    """A callable that all-reduces `buffers` in place across the default process
    group.  B200 buffers are aliased as torch tensors and the collective is issued
    on the library's stream, so it is ordered after the kernels that produced the
    data and before those that consume it; numpy arrays (CPU tests) go through
    ``torch.from_numpy``."""
    import torch
    import torch.distributed as dist
    rop = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX}[op]
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return lambda: None
    if buffers and isinstance(buffers[0], np.ndarray):
        tensors = [torch.from_numpy(b) for b in buffers]

        def run_cpu():
            for t in tensors:
                dist.all_reduce(t, op=rop)
        return run_cpu
    tdev = torch.device("cuda", local_rank)
    tensors = [torch.as_tensor(_CudaAlias(b.device_ptr(), b.numel()), device=tdev) for b in buffers]
    ext = torch.cuda.ExternalStream(device.stream(), device=tdev)

    def run_gpu():
        with torch.cuda.stream(ext):
            for t in tensors:
                dist.all_reduce(t, op=rop)
    return run_gpu
