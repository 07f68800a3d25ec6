"""The N>1 host logic on CPU: two gloo ranks run the data-parallel step (oracle
kernels, sharded batch, gradient all-reduce, lr/world) and must land on the same
parameters as one rank over the whole batch; the row-sharded column max must
equal the global one after a MAX all-reduce."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

from harp_b200 import parallel as P
from harp_b200 import workloads as W


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _small_mlp(lo, hi, total=32):
    from harp_b200.frontend import Tensor
    rng = np.random.default_rng(3)
    X = rng.uniform(-np.pi, np.pi, (total, 1)).astype(np.float32)
    T = np.sin(X).astype(np.float32)
    prng = np.random.default_rng(30)
    vals = [prng.standard_normal((8, 1)).astype(np.float32) * 0.5, np.zeros(8, np.float32),
            prng.standard_normal((1, 8)).astype(np.float32) * 0.5, np.zeros(1, np.float32)]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    h = Tensor.input(X[lo:hi]).linear(ps[0], ps[1]).tanh().linear(ps[2], ps[3])
    d = h - Tensor.input(T[lo:hi])
    loss = (d * d).sum() * (1.0 / (hi - lo))
    return loss, ps, loss.backward(ps)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from harp_b200.frontend import Program
    from oracle.executor import OracleExecutor
    lo, hi = P.shard_range(32, rank, world)
    loss, ps, grads = _small_mlp(lo, hi)
    prog = Program([loss], OracleExecutor(), sgd=list(zip(ps, grads)), lr=0.1 / world, persistent=True, flat=True)
    prog.run_forward()
    allreduce = P.make_allreduce(prog.grad_buffers(), "sum")
    for _ in range(3):
        prog.run(allreduce)
    params = [prog.fetch(p).copy() for p in ps]
    # sharded column max: each rank reduces its row block, MAX all-reduce combines
    x = W.cfg2_input(64, 48)
    part = x[slice(*P.shard_range(64, rank, world))].max(axis=0).copy()
    P.make_allreduce([part], "max")()
    if rank == 0:
        q.put((params, part))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_range_covers_everything_once():
    for n, w_ in ((4096, 8), (10, 3), (7, 8)):
        spans = [P.shard_range(n, r, w_) for r in range(w_)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1


def test_two_gloo_ranks_match_one_rank():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    params2, zmax = q.get()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    # single rank, whole batch, same learning rate
    from harp_b200.frontend import Program
    from oracle.executor import OracleExecutor
    loss, ps, grads = _small_mlp(0, 32)
    prog = Program([loss], OracleExecutor(), sgd=list(zip(ps, grads)), lr=0.1, persistent=True)
    for _ in range(3):
        prog.run()
    for a, p in zip(params2, ps):
        b = prog.fetch(p)
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)
    assert (zmax == W.cfg2_input(64, 48).max(axis=0)).all()
