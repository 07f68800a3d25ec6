"""The N>1 host logic on CPU: gloo ranks run the data-parallel step (oracle
kernels, sharded batch, fused gradient all-reduce + update through the CPU
stand-in of the communicator, overlapped bucket included) and must land on the
same parameters as one rank over the whole batch; the row-sharded column max
must equal the global one after a MAX all-reduce; row- and batch-sharded
contractions must tile the unsharded result exactly."""
import os
import socket
import traceback

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

from harp_b200 import desc as D
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


def _worker_body(rank, world):
    from harp_b200.frontend import Program
    from oracle import c_emit as O
    from oracle.executor import OracleExecutor
    comm = P.HostComm(rank, world)
    out = {}
    # (1) data-parallel training step, fused all-reduce + SGD, early bucket overlapped
    lo, hi = P.shard_range(32, rank, world)
    loss, ps, grads = _small_mlp(lo, hi)
    prog = Program([loss], OracleExecutor(), sgd=list(zip(ps, grads)), lr=0.1 / world, persistent=True, flat=True, comm=comm)
    out["buckets"] = list(prog.buckets)
    for _ in range(3):
        prog.run()
    out["params"] = [prog.fetch(p).copy() for p in ps]
    # (2) the same with Adam: plain all-reduce of the flat gradients, then the stateful update
    loss, ps, grads = _small_mlp(lo, hi)
    prog = Program([loss], OracleExecutor(), sgd=list(zip(ps, grads)), lr=0.01, persistent=True, flat=True,
                   optimizer="adam", comm=comm)
    for _ in range(3):
        prog.run()
    out["adam"] = [prog.fetch(p).copy() for p in ps]
    # (3) row-sharded column max: each rank reduces its row block, MAX all-reduce combines
    x = W.cfg2_input(64, 48)
    r0, r1 = P.shard_range(64, rank, world)
    part = O.run(W.cfg2_z(r1 - r0, 48), [x[r0:r1]])
    comm.allreduce(part, D.R_MAX)
    out["zmax"] = part
    # (4) dense contraction, A and C row-sharded, B replicated; batched contraction sharded by batch index
    a, b = W.uniform_pm1((24, 16), 5), W.uniform_pm1((16, 20), 6)
    sh = P.gemm_row_shard(24, 16, 20, rank, world)
    out["c_rows"] = (sh["rows"], O.run(W.matmul_desc(sh["m_local"], 16, 20), [a[sh["rows"][0]:sh["rows"][1]], b]))
    ab, bb = W.uniform_pm1((6, 8, 8), 7), W.uniform_pm1((6, 8, 8), 8)
    b0, b1 = P.batch_shard(6, rank, world)
    out["c_batch"] = ((b0, b1), O.run(W.matmul_desc(8, 8, 8, batch=b1 - b0), [ab[b0:b1], bb[b0:b1]]))
    return out


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        res = _worker_body(rank, world)
        q.put((rank, "ok", res))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def _run_ranks(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=240)
            assert status == "ok", payload
            results[rank] = payload
    finally:
        for p in procs:
            p.join(30)
            if p.is_alive():
                p.terminate()
    return results


def test_shard_range_covers_everything_once():
    for n, w_ in ((4096, 8), (10, 3), (7, 8), (64, 8), (8192, 4)):
        spans = [P.shard_range(n, r, w_) for r in range(w_)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    sh = [P.gemm_row_shard(8192, 8192, 8192, r, 8) for r in range(8)]
    assert all(s["m_local"] == 1024 and s["b_replicated_bytes"] == 4 * 8192 * 8192 for s in sh)
    assert [s["c_elems"][0] for s in sh] == [r * 1024 * 8192 for r in range(8)]


def test_two_gloo_ranks_match_one_rank():
    from harp_b200.frontend import Program
    from oracle import c_emit as O
    from oracle.executor import OracleExecutor
    res = _run_ranks(2)
    # single rank, whole batch, same learning rate
    loss, ps, grads = _small_mlp(0, 32)
    prog = Program([loss], OracleExecutor(), sgd=list(zip(ps, grads)), lr=0.1, persistent=True)
    for _ in range(3):
        prog.run()
    for r in (0, 1):
        for a, p in zip(res[r]["params"], ps):
            np.testing.assert_allclose(a, prog.fetch(p), rtol=1e-4, atol=1e-6)
    # both ranks hold bit-identical parameters (sums are taken in rank order on every rank)
    for a, b in zip(res[0]["params"], res[1]["params"]):
        assert a.tobytes() == b.tobytes()
    for a, b in zip(res[0]["adam"], res[1]["adam"]):
        assert a.tobytes() == b.tobytes()
    # the overlapped bucket was planned (two ranks) and covers part of the flat buffer only
    assert len(res[0]["buckets"]) == 1 and res[0]["buckets"] == res[1]["buckets"]
    # Adam over the summed gradient of the shards = Adam over 2x the mean gradient of the whole batch
    loss, ps, grads = _small_mlp(0, 32)
    prog = Program([loss * 2.0], OracleExecutor(), sgd=list(zip(ps, (loss * 2.0).backward(ps))), lr=0.01, persistent=True,
                   flat=True, optimizer="adam")
    for _ in range(3):
        prog.run()
    for a, p in zip(res[0]["adam"], ps):
        np.testing.assert_allclose(a, prog.fetch(p), rtol=2e-3, atol=1e-5)
    x = W.cfg2_input(64, 48)
    assert (res[0]["zmax"] == x.max(axis=0)).all() and (res[1]["zmax"] == x.max(axis=0)).all()
    # sharded contractions tile the unsharded results bit for bit (same loop nest per output element)
    a, b = W.uniform_pm1((24, 16), 5), W.uniform_pm1((16, 20), 6)
    full = O.run(W.matmul_desc(24, 16, 20), [a, b]).reshape(24, 20)
    for r in (0, 1):
        (lo, hi), c = res[r]["c_rows"]
        assert c.reshape(hi - lo, 20).tobytes() == full[lo:hi].tobytes()
    ab, bb = W.uniform_pm1((6, 8, 8), 7), W.uniform_pm1((6, 8, 8), 8)
    fullb = O.run(W.matmul_desc(8, 8, 8, batch=6), [ab, bb]).reshape(6, 8, 8)
    for r in (0, 1):
        (lo, hi), c = res[r]["c_batch"]
        assert c.reshape(hi - lo, 8, 8).tobytes() == fullb[lo:hi].tobytes()
