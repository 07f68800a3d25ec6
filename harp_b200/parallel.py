"""Data-parallel plumbing: sharding rules and the communicator a step runs over.

The reference has no distributed code at all (no collective call site, Rc-based
single-thread graph: src/graph/node.rs:222).  The sharded paths here are new:
one process per GPU, every rank runs the same kernel list on its shard, and the
only exchanges are

* training steps (batch shards): one SUM all-reduce of the flat gradient buffer
  per step, fused with the SGD update (``eb200_comm_allreduce_sgd``; learning
  rate divided by the world size = gradient mean);
* row-sharded reductions: the all-reduce of the per-rank partial results
  (``eb200_kernel_set_allreduce`` / ``eb200_comm_allreduce``);
* dense contractions sharded by rows of A and C (B replicated in every GPU's
  own memory) or by batch index: no exchange at all.

Collectives on GPUs go through the library's own communicator
(``harp_b200.backend.B200Comm``: a one-shot NVLink kernel for small messages,
NCCL otherwise).  ``torch.distributed`` is only the host-side rendezvous that
carries the communicator's unique id between the processes, and the transport of
``HostComm``, the CPU stand-in with the same interface used by the multi-process
tests (gloo).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np

from . import desc as D


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [lo, hi) of `n` items owned by `rank` (sizes differ by at most 1)."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def gemm_row_shard(m: int, k: int, n: int, rank: int, world: int) -> dict:
    """C = A.B with A and C partitioned by rows, B replicated in every GPU's own
    memory: rank r computes C[lo:hi, :] = A[lo:hi, :] . B.  No exchange."""
    lo, hi = shard_range(m, rank, world)
    return {"rows": (lo, hi), "m_local": hi - lo, "a_elems": (lo * k, hi * k), "c_elems": (lo * n, hi * n),
            "b_replicated_bytes": 4 * k * n}


def batch_shard(batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Batched contraction / training batch partitioned by batch index."""
    return shard_range(batch, rank, world)


def exchange_unique_id(rank: int, world: int) -> Optional[bytes]:
    """Rank 0 makes the communicator's unique id; the default ``torch.distributed``
    group carries it to the other ranks (host-side rendezvous only)."""
    if world == 1:
        return None
    import torch.distributed as dist
    from .backend import B200Comm
    box = [B200Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]


def init_comm(device, rank: int, world: int):
    """This rank's ``B200Comm`` (all ranks call it together)."""
    from .backend import B200Comm
    return B200Comm(device, rank, world, exchange_unique_id(rank, world))


class HostComm:
    """CPU stand-in for ``B200Comm`` over numpy arrays and the default
    ``torch.distributed`` group (gloo): same calls, same semantics (results summed
    in rank order are identical on every rank).  Lets the sharding logic and the
    step loop run as world_size > 1 processes on a machine without GPUs."""

    def __init__(self, rank: int, nranks: int):
        self.rank, self.nranks = rank, nranks
        self.calls = 0

    def info(self):
        return {"rank": self.rank, "nranks": self.nranks, "one_shot": False, "calls_one_shot": 0, "calls_nccl": self.calls}

    def _gather(self, a: np.ndarray):
        import torch
        import torch.distributed as dist
        self.calls += 1
        if self.nranks == 1:
            return [a.copy()]
        parts = [torch.empty(a.size, dtype=torch.float32) for _ in range(self.nranks)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(a, np.float32).reshape(-1).copy()))
        return [p.numpy() for p in parts]

    def allreduce(self, buf: np.ndarray, op: int = D.R_SUM, offset: int = 0, count: Optional[int] = None, side_stream: bool = False):
        n = buf.size - offset if count is None else count
        view = buf.reshape(-1)[offset:offset + n]
        parts = self._gather(view)
        acc = parts[0].copy()
        for p in parts[1:]:                     # rank order, like the device kernel
            if op == D.R_SUM:
                acc = acc + p
            elif op == D.R_MAX:
                acc = np.maximum(acc, p)
            elif op == D.R_MIN:
                acc = np.minimum(acc, p)
            else:
                acc = acc * p
        view[...] = acc

    def allreduce_sgd(self, params: np.ndarray, grads: np.ndarray, lr: float, offset: int = 0, count: Optional[int] = None,
                      side_stream: bool = False):
        n = params.size - offset if count is None else count
        parts = self._gather(grads.reshape(-1)[offset:offset + n])
        acc = parts[0].copy()
        for p in parts[1:]:
            acc = acc + p
        pv = params.reshape(-1)[offset:offset + n]
        pv[...] = pv - np.float32(lr) * acc

    def join(self):
        pass

    def attach(self, kernel):
        kernel.comm = self

    def destroy(self):
        pass
