"""Collectives of the C ABI on real GPUs.

One rank: the communicator degenerates to local kernels and must reproduce the
unfused paths bit for bit.  Two ranks (run when the box has at least two GPUs):
one process per GPU; the one-shot NVLink all-reduce, its fused SGD and
reduce-finish forms, the side-stream form, replay from a CUDA graph and the NCCL
path for large messages, each against numpy on the gathered inputs."""
import ctypes as C
import traceback

import numpy as np
import pytest

from harp_b200 import capi
from harp_b200 import desc as D
from harp_b200 import workloads as W
from harp_b200.backend import B200BackendRegistry, B200Comm

pytestmark = pytest.mark.gpu


def _buf(reg, dev, a):
    b = reg.allocate_buffer(dev, [a.size])
    b.write_vec(a)
    return b


def test_single_rank_communicator_matches_the_plain_kernels(dev, registry):
    comm = B200Comm(dev, 0, 1)
    assert comm.info()["nranks"] == 1
    rng = np.random.default_rng(0)
    n = 225034
    p, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    # all-reduce over one rank leaves the data alone
    bg = _buf(registry, dev, g)
    comm.allreduce(bg, D.R_SUM)
    comm.allreduce(bg, D.R_MAX, side_stream=True)
    comm.join()
    assert bg.read_vec().tobytes() == g.tobytes()
    # fused all-reduce + SGD == the SGD kernel
    bp1, bp2 = _buf(registry, dev, p), _buf(registry, dev, p)
    kd = D.KernelDesc(D.K_SGD, [n], [D.contiguous([n]), D.contiguous([n])], D.contiguous([n]), scalar=0.01)
    registry.compile_ast(dev, kd).execute([bp1, bg], [bp1])
    comm.allreduce_sgd(bp2, bg, 0.01)
    assert bp1.read_vec().tobytes() == bp2.read_vec().tobytes()
    # an offset / count range only touches that range
    bp3 = _buf(registry, dev, p)
    comm.allreduce_sgd(bp3, bg, 0.01, offset=1024, count=5000, side_stream=True)
    comm.join()
    got, ref = bp3.read_vec(), bp1.read_vec()
    assert got[1024:6024].tobytes() == ref[1024:6024].tobytes()
    assert got[:1024].tobytes() == p[:1024].tobytes() and got[6024:].tobytes() == p[6024:].tobytes()
    # a split column reduce with the communicator attached folds its partials in the collective's kernel
    x = W.cfg2_input(2048, 4096)
    kz = W.cfg2_z(2048, 4096)
    bx = _buf(registry, dev, x)
    z1, z2 = registry.allocate_buffer(dev, [4096]), registry.allocate_buffer(dev, [4096])
    k1, k2 = registry.compile_ast(dev, kz), registry.compile_ast(dev, kz)
    assert k1.impl.endswith("_split")
    comm.attach(k2)
    k1.execute([bx], [z1]); k2.execute([bx], [z2])
    assert z1.read_vec().tobytes() == z2.read_vec().tobytes() == x.max(axis=0).tobytes()
    assert comm.info()["calls_one_shot"] >= 3      # the two fused updates and the fused reduce finish
    comm.destroy()


def _rank_main(rank, world, uid_q, out_q):
    try:
        reg = B200BackendRegistry()
        dev = reg.create_device(rank)
        if rank == 0:
            uid = B200Comm.unique_id()
            for _ in range(world - 1):
                uid_q.put(uid)
        else:
            uid = uid_q.get(timeout=120)
        comm = B200Comm(dev, rank, world, uid)
        info = comm.info()
        res = {"one_shot": info["one_shot"]}
        def data(n, seed):       # what rank r contributes: every rank can rebuild all of them
            return [np.random.default_rng(1000 * seed + r).standard_normal(n).astype(np.float32) for r in range(world)]
        # plain all-reduce at several sizes: one element, ragged, the benchmark's messages, one beyond the inbox (NCCL)
        for n in (1, 5, 8192, 66561, 225034, 600001):
            parts = data(n, n)
            for op, fold in ((D.R_SUM, lambda a, b: a + b), (D.R_MAX, np.maximum)):
                b = _buf(reg, dev, parts[rank])
                comm.allreduce(b, op)
                ref = parts[0].copy()
                for q in parts[1:]:
                    ref = fold(ref, q)
                got = b.read_vec()
                # max is exact; the one-shot kernel adds in rank order like `ref` (and with two ranks any
                # order gives the same sum); NCCL on more ranks may add in another order
                exact = op == D.R_MAX or world == 2 or (info["one_shot"] and n <= 524288)
                ok = got.tobytes() == ref.tobytes() if exact else np.allclose(got, ref, rtol=1e-6, atol=1e-6)
                assert ok, (n, op)
        # fused all-reduce + SGD, twice in a row, the second on the side stream
        n = 225034
        parts = data(n, 7)
        p0 = np.random.default_rng(5).standard_normal(n).astype(np.float32)
        bp, bg = _buf(reg, dev, p0), _buf(reg, dev, parts[rank])
        comm.allreduce_sgd(bp, bg, 0.01 / world)
        comm.allreduce_sgd(bp, bg, 0.01 / world, side_stream=True)
        comm.join()
        s = parts[0].copy()
        for q in parts[1:]:
            s = s + q
        lr = np.float32(0.01 / world)
        ref = p0 - lr * s
        ref = ref - lr * s
        got = bp.read_vec()
        assert got.tobytes() == ref.tobytes() if info["one_shot"] else np.allclose(got, ref, rtol=1e-6, atol=1e-6)
        assert bg.read_vec().tobytes() == parts[rank].tobytes()         # the gradients keep this rank's values
        # row-sharded column max: the reduce kernel's finish pass does the exchange
        rows, cols = 4096, 8192
        x = W.cfg2_input(rows, cols, seed=2)
        lo, hi = rank * rows // world, (rank + 1) * rows // world
        kz = reg.compile_ast(dev, W.cfg2_z(hi - lo, cols))
        comm.attach(kz)
        bx, bz = _buf(reg, dev, x[lo:hi]), reg.allocate_buffer(dev, [cols])
        for _ in range(3):
            kz.execute([bx], [bz])
        assert bz.read_vec().tobytes() == x.max(axis=0).tobytes()
        # replay from a CUDA graph: the sequence number lives on the device
        parts = data(8192, 9)
        bv = _buf(reg, dev, parts[rank])
        dev.synchronize()
        dev.graph_begin()
        comm.allreduce(bv, D.R_SUM, side_stream=True)
        comm.join()
        comm.allreduce(bv, D.R_SUM)
        graph = dev.graph_end()
        s = parts[0].copy()
        for q in parts[1:]:
            s = s + q
        for rep in range(3):
            graph.launch()
        # every all-reduce of values that are equal on all ranks multiplies by `world`: after the first
        # replay v = world * S, and each further replay multiplies by world^2
        expect = s * np.float32(world)
        for _ in range(2):
            expect = expect * np.float32(world) * np.float32(world)
        got = bv.read_vec()
        assert np.allclose(got, expect, rtol=1e-5), (got[:4], expect[:4])
        dev.synchronize()
        res["calls"] = comm.info()
        comm.destroy()
        out_q.put((rank, "ok", res))
    except Exception:
        out_q.put((rank, "error", traceback.format_exc()))


def test_two_ranks_one_process_per_gpu():
    n = C.c_int()
    capi.call("eb200_device_count", C.byref(n))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    world = 2
    uid_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, uid_q, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = out_q.get(timeout=300)
            assert status == "ok", payload
            results[rank] = payload
    finally:
        for p in procs:
            p.join(30)
            if p.is_alive():
                p.terminate()
    assert results[0]["one_shot"] == results[1]["one_shot"]
    assert results[0]["calls"]["calls_one_shot"] > 0 or not results[0]["one_shot"]
