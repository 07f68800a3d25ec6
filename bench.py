#!/usr/bin/env python
"""Benchmark of the hot path on B200: BASELINE config 2 (fused elementwise +
reduce, column max, transposing copy over x f32 [8192, 8192]).

One step = one pass of the three lowered kernels over one x:
    y = sum(exp(0.5*x + 1.0) * x, axis=1)   fused chain + row reduce   268 468 224 B
    z = max(x, axis=0)                       column reduce              268 468 224 B
    t = x.permute(1,0).contiguous()          transposing copy           536 870 912 B
Algorithmic bytes per step = 1 073 807 360 (each kernel reads x once; outputs
written once).  With N GPUs every rank holds its own [8192, 8192] row block of a
global [8192*N, 8192] tensor (weak scaling); y and t need no exchange, the
column-max partials are combined by one 32 KB MAX-allreduce per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Prints ONE JSON line (rank 0).  `value` is device-timed with inputs resident in
HBM; `e2e` goes through the same C-ABI calls with host buffers, host<->device
copies inside the timed region.  `--impl reference` times the reference's CPU
path (the oracle's emitted C with OpenMP, all host threads) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS = 8192, 8192
BYTES_Y = 4 * ROWS * COLS + 4 * ROWS + 8
BYTES_Z = 4 * ROWS * COLS + 4 * COLS
BYTES_T = 8 * ROWS * COLS
BYTES_STEP = BYTES_Y + BYTES_Z + BYTES_T
METRIC = "fused_elemwise_reduce_throughput"
UNIT = "GB/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures
# summarised under profiles/ (None until a capture exists for that kernel).
NCU_TRAFFIC = {"reduce_inner": 272_698_000, "reduce_outer": 272_148_000, "transpose_copy": 489_688_000}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML while the GPU is busy
    (read-only queries; nothing is set)."""

    def __init__(self, index: int, period_s: float = 0.005):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples = []          # (t, sm_mhz, reasons_bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()

    def summary(self, windows):
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                 0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in windows)]
        use = inside if inside else self.samples
        if not use:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mask = 0
        for s in use:
            mask |= s[2]
        return {"sm_mhz": float(np.median([s[1] for s in use])), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for b, n in names.items() if mask & b), "samples": len(use)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ---------------------------------------------------------------------------------------
def run_cpu_workload(x, openmp: bool, rows: int):
    """One pass of the three kernels on the CPU oracle over the first `rows` rows."""
    from harp_b200 import workloads as W
    from oracle import c_emit as O
    c0, c1 = W.cfg2_consts()
    xs = np.ascontiguousarray(x[:rows])
    ks = [O.OracleKernel(k, openmp=openmp) for k in (W.cfg2_y(rows, COLS), W.cfg2_z(rows, COLS), W.cfg2_t(rows, COLS))]
    outs = [np.zeros(rows, np.float32), np.zeros(COLS, np.float32), np.zeros(rows * COLS, np.float32)]

    def step():
        ks[0]([c0, xs, c1], outs[0])
        ks[1]([xs], outs[1])
        ks[2]([xs], outs[2])
    bytes_step = (4 * rows * COLS + 4 * rows + 8) + (4 * rows * COLS + 4 * COLS) + 8 * rows * COLS
    return step, bytes_step


def cpu_baseline(x, seconds_allowed: float = 20.0):
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    step, nbytes = run_cpu_workload(x, True, ROWS)
    t0 = time.perf_counter(); step(); first = time.perf_counter() - t0
    best = first
    reps = 1
    while reps < 3 and (reps + 1) * first < seconds_allowed:
        t0 = time.perf_counter(); step(); best = min(best, time.perf_counter() - t0)
        reps += 1
    out = {"value": nbytes / best / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
           "sample": f"full [8192,8192] workload, emitted C with OpenMP (gcc -O3 -ffast-math -fopenmp), best of {reps}",
           "seconds": best}
    # single-thread C backend on a quarter of the rows
    step1, nbytes1 = run_cpu_workload(x, False, ROWS // 4)
    t0 = time.perf_counter(); step1(); t1 = time.perf_counter() - t0
    out["c_backend_1thread_gbs"] = nbytes1 / t1 / 1e9
    return out


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    from harp_b200 import workloads as W
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    x = W.cfg2_input(ROWS, COLS)
    # size the per-step sample so that warmup+steps end within ~2 minutes
    step, nbytes = run_cpu_workload(x, True, ROWS)
    t0 = time.perf_counter(); step(); full = time.perf_counter() - t0
    rows = ROWS
    total_steps = args.steps + args.warmup
    while rows > 256 and full * rows / ROWS * total_steps > 120.0:
        rows //= 2
    if rows != ROWS:
        step, nbytes = run_cpu_workload(x, True, rows)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = nbytes * args.steps / dt / 1e9
    sample = f"rows [0,{rows}) of x [8192,8192] per step; emitted C with OpenMP on {cores} host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 2: y=sum(exp(.5x+1)*x,axis=1), z=max(x,axis=0), t=x.permute(1,0).contiguous(); x f32 [8192,8192] N(0,1) seed 2",
                   "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
def run_b200(args):
    rank, local_rank, world = dist_env()
    n = args.gpus
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from harp_b200 import workloads as W
    from harp_b200.backend import B200BackendRegistry, PinnedArray, launch_count

    reg = B200BackendRegistry()
    dev = reg.create_device(local_rank)
    sampler = ClockSampler(local_rank)
    c0, c1 = W.cfg2_consts()
    x_host = PinnedArray((ROWS, COLS))
    x_host.array[...] = W.cfg2_input(ROWS, COLS, seed=2 + rank)   # this rank's row block
    bx = reg.allocate_buffer(dev, [ROWS, COLS])
    b0 = reg.allocate_buffer(dev, [1]); b0.write_vec(c0)
    b1 = reg.allocate_buffer(dev, [1]); b1.write_vec(c1)
    by = reg.allocate_buffer(dev, [ROWS])
    bz = reg.allocate_buffer(dev, [COLS])
    bt = reg.allocate_buffer(dev, [COLS, ROWS])
    bx.write_async(x_host.ptr, x_host.nbytes)
    ky = reg.compile_ast(dev, W.cfg2_y())
    kz = reg.compile_ast(dev, W.cfg2_z())
    kt = reg.compile_ast(dev, W.cfg2_t())
    dev.synchronize()

    allreduce_z = None
    if world > 1:
        from harp_b200 import parallel
        allreduce_z = parallel.make_allreduce([bz], "max", dev, local_rank)   # on the library's own stream

    def step():
        ky.execute([b0, bx, b1], [by])
        kz.execute([bx], [bz])
        if allreduce_z:
            allreduce_z()
        kt.execute([bx], [bt])

    def barrier():
        if world > 1:
            import torch
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()
        dev.synchronize()

    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- device-timed region: K steps between two events; on every 8th step three more events
    #      separate the kernels (recording an event between every pair of kernels on every step
    #      cost the region ~10 us per step: 196 vs 185.5 us) ---------------------------------
    K = args.steps
    SAMPLE = 8
    evs = {s_: [dev.event() for _ in range(4)] for s_ in range(0, K, SAMPLE)}
    e_begin, e_end = dev.event(), dev.event()
    l0 = launch_count()
    w0 = time.perf_counter()
    e_begin.record()
    for s_ in range(K):
        e = evs.get(s_)
        if e is None:
            step()
            continue
        e[0].record(); ky.execute([b0, bx, b1], [by])
        e[1].record(); kz.execute([bx], [bz])
        if allreduce_z:
            allreduce_z()
        e[2].record(); kt.execute([bx], [bt])
        e[3].record()
    e_end.record()
    barrier()
    w1 = time.perf_counter()
    launches = launch_count() - l0
    total_ms = e_begin.elapsed_ms(e_end)
    ns = len(evs)
    t_y = sum(e[0].elapsed_ms(e[1]) for e in evs.values()) / ns
    t_z = sum(e[1].elapsed_ms(e[2]) for e in evs.values()) / ns
    t_t = sum(e[2].elapsed_ms(e[3]) for e in evs.values()) / ns

    # ---- end-to-end: host buffers in, host buffers out, every step --------------------
    # Double-buffered: the upload of batch i+1, the kernels of batch i and the
    # download of batch i's results run concurrently (copies on two side streams,
    # ordered against the compute stream by events).  Every step still moves its
    # own x up and its own y, z, t down inside the timed region.
    y_host, z_host, t_host = PinnedArray((ROWS,)), PinnedArray((COLS,)), PinnedArray((COLS, ROWS))
    KE = max(4, min(K, 20))
    up, down = dev.copy_stream(), dev.copy_stream()
    xs = [bx, reg.allocate_buffer(dev, [ROWS, COLS])]
    outs = [(by, bz, bt), (reg.allocate_buffer(dev, [ROWS]), reg.allocate_buffer(dev, [COLS]), reg.allocate_buffer(dev, [COLS, ROWS]))]
    ev_up = [dev.event(), dev.event()]       # upload into xs[i] finished
    ev_k = [dev.event(), dev.event()]        # kernels on slot i finished
    ev_down = [dev.event(), dev.event()]     # download of outs[i] finished

    def e2e_run(steps):
        for i in range(steps + 1):
            sl = i & 1
            if i < steps:                      # upload batch i (needs the kernels that last read this slot)
                if i >= 2:
                    dev.wait_event(ev_k[sl], up)
                xs[sl].write_on(up, x_host.ptr, x_host.nbytes)
                ev_up[sl].record(up)
                dev.wait_event(ev_up[sl])      # compute stream: kernels of batch i wait for its upload
                if i >= 2:
                    dev.wait_event(ev_down[sl])    # ... and for the previous results of this slot to have left
                if allreduce_z and i >= 1:
                    dev.wait_event(ev_down[1 - sl])   # both slots share the all-reduced z buffer
                oy, oz, ot = outs[sl]
                ky.execute([b0, xs[sl], b1], [oy])
                kz.execute([xs[sl]], [oz])
                if allreduce_z:
                    allreduce_z()
                kt.execute([xs[sl]], [ot])
                ev_k[sl].record()
                dev.wait_event(ev_k[sl], down)  # download batch i's results
                oy.read_on(down, y_host.ptr, y_host.nbytes)
                oz.read_on(down, z_host.ptr, z_host.nbytes)
                ot.read_on(down, t_host.ptr, t_host.nbytes)
                ev_down[sl].record(down)
        down.synchronize()                     # the caller holds every result
        dev.synchronize()
    if allreduce_z:                            # the collective aliases bz only: keep slot outputs on bz
        outs[1] = (outs[1][0], bz, outs[1][2])
    e2e_run(2)
    barrier()
    ea, eb = dev.event(), dev.event()
    w2 = time.perf_counter()
    ea.record()
    e2e_run(KE)
    eb.record()
    barrier()
    w3 = time.perf_counter()
    e2e_ms = ea.elapsed_ms(eb)
    sampler.stop()

    # release the config 2 buffers, then time the other configurations
    extra = None
    if not args.no_extra:
        for b_ in (bx, by, bz, bt, xs[1], outs[1][0], outs[1][2]):
            b_.release()
        for h_ in (y_host, z_host, t_host):
            h_.free()
        extra = extra_measurements(reg, dev, rank, world, local_rank, quick=args.steps < 20)
    if world > 1:
        import torch
        import torch.distributed as dist
        tm = torch.tensor([total_ms, e2e_ms, t_y, t_z, t_t], device="cuda", dtype=torch.float64)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, t_y, t_z, t_t = tm.tolist()
    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    value = BYTES_STEP * n * K / (total_ms * 1e-3) / 1e9
    e2e = BYTES_STEP * n * KE / (e2e_ms * 1e-3) / 1e9
    kernels = {}
    for name, impl, b, ms in (("y_fused_row_sum", ky.impl, BYTES_Y, t_y), ("z_col_max", kz.impl, BYTES_Z, t_z),
                              ("t_transpose", kt.impl, BYTES_T, t_t)):
        gbs = b / (ms * 1e-3) / 1e9
        kernels[name] = {"impl": impl, "ms": ms, "algo_bytes": b, "achieved_gbs": gbs, "frac_of_" + peak_kind: gbs / peak}
    top = max(kernels.items(), key=lambda kv: kv[1]["ms"])
    traffic = NCU_TRAFFIC.get("transpose_copy" if top[0] == "t_transpose" else
                              ("reduce_outer" if top[0] == "z_col_max" else "reduce_inner"))
    roofline = {"bound": "hbm", "kernel": top[1]["impl"], "achieved": top[1]["achieved_gbs"], "peak": peak,
                "peak_source": f"{peak_kind} copy bandwidth (MEASURED_PEAKS.json)" if peak_kind == "measured" else "fallback 6650 GB/s",
                "unit": "GB/s", "frac": top[1]["achieved_gbs"] / peak, "traffic": traffic,
                "time_share": top[1]["ms"] / (t_y + t_z + t_t)}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 2: y=sum(exp(.5x+1)*x,axis=1), z=max(x,axis=0), t=x.permute(1,0).contiguous(); x f32 [8192,8192] N(0,1) seed 2 per GPU",
                   "l2": "inputs larger than L2 (x is 256 MiB, L2 126 MB)",
                   "sharding": "row blocks of a global [8192*N, 8192] tensor; MAX-allreduce of the 32 KB column-max partials" if n > 1 else "single GPU",
                   "algo_bytes_per_step_per_gpu": BYTES_STEP,
                   "kernel_events": f"per-kernel durations from events on every {SAMPLE}th timed step ({ns} of {K})"},
        "roofline": roofline, "kernels": kernels,
        "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(x_host.nbytes),
                "d2h_bytes_per_step": int(y_host.nbytes + z_host.nbytes + t_host.nbytes), "steps": KE,
                "ms_per_step": e2e_ms / KE},
        "gpu_launches": int(launches),
        "clocks": sampler.summary([(w0, w1), (w2, w3)]),
    }
    if n == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(x_host.array)
    if extra is not None:
        line["extra"] = extra
    print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def time_kernel(dev, kern, ins, outs, reps=5, warm=2):
    for _ in range(warm):
        kern.execute(ins, outs)
    dev.synchronize()
    dev.timer_begin()
    for _ in range(reps):
        kern.execute(ins, outs)
    return dev.timer_end() / reps


CONV_SHAPES = [("cnn_conv1_1x28x28_to_32", (4096, 1, 28, 28, 32, 3, 3, 0)),
               ("cnn_conv2_32x13x13_to_64", (4096, 32, 13, 13, 64, 3, 3, 0)),
               ("conv_64x56x56_to_128_pad1", (256, 64, 56, 56, 128, 3, 3, 1))]


def conv_measurements(reg, dev, rng, quick=False, shapes=None, reps=None):
    """conv2d as one kernel (bias + ReLU in the epilogue, output [N, Co, Ho, Wo]): the two
    layers of config 4 at batch 4096 and one padded 64->128 layer, TF32 and 3xTF32
    (the first layer, K = 9, runs the streaming f32 kernel whatever the mode).
    Inputs are larger than L2 except where `shapes` asks for a small profiling case."""
    from harp_b200 import desc as D
    res = {}
    for name, (n, c, h, w_, co, kh, kw, pad) in (shapes or CONV_SHAPES):
        ho, wo = h + 2 * pad - kh + 1, w_ + 2 * pad - kw + 1
        bx = reg.allocate_buffer(dev, [n * c * h * w_]); bw = reg.allocate_buffer(dev, [co * c * kh * kw])
        bb = reg.allocate_buffer(dev, [co]); bo = reg.allocate_buffer(dev, [n * ho * wo * co])
        bx.write_vec(rng.uniform(-1, 1, n * c * h * w_).astype(np.float32))
        bw.write_vec(rng.uniform(-1, 1, co * c * kh * kw).astype(np.float32))
        bb.write_vec(rng.uniform(-1, 1, co).astype(np.float32))
        for mode, mname in ((D.GEMM_TF32, "tf32"), (D.GEMM_3XTF32, "3xtf32")):
            kern = reg.compile_ast(dev, D.conv2d(n, c, h, w_, co, kh, kw, pad=pad, relu=True, mode=mode, nchw=True))
            ms = time_kernel(dev, kern, [bx, bw, bb], [bo], reps=reps or (3 if quick else 10))
            res[f"{name}_{mname}"] = {"impl": kern.impl, "ms": ms, "tflops": 2.0 * n * ho * wo * co * c * kh * kw / ms / 1e9,
                                      "gbs_x_plus_out": 4.0 * (n * c * h * w_ + n * ho * wo * co) / ms / 1e6}
        for b_ in (bx, bw, bb, bo):
            b_.release()
    return res


def run_only_conv(args):
    """`--only conv2d`: a small case of the convolution kernel alone (for profiler captures);
    `--only conv2d_grad`: the gradient forms and the streaming small-K kernels of config 4's layers at batch 1024."""
    from harp_b200 import desc as D
    from harp_b200.backend import B200BackendRegistry
    reg = B200BackendRegistry()
    dev = reg.create_device(0)
    rng = np.random.default_rng(5)
    if args.only == "conv2d":
        res = conv_measurements(reg, dev, rng, shapes=[("cnn_conv2_batch2048", (2048, 32, 13, 13, 64, 3, 3, 0))], reps=2)
        print(json.dumps({"only": "conv2d", "conv2d": res}))
        return
    n = 1024
    res = {}

    def run(name, kd, sizes, out_size):
        bufs = []
        for sz in sizes:
            b = reg.allocate_buffer(dev, [sz])
            b.write_vec(rng.uniform(-1, 1, sz).astype(np.float32))
            bufs.append(b)
        bo = reg.allocate_buffer(dev, [out_size])
        kern = reg.compile_ast(dev, kd)
        res[name] = {"impl": kern.impl, "ms": time_kernel(dev, kern, bufs, [bo], reps=2, warm=1)}
    # conv2 of config 4: input gradient (flag 128) and weight gradient (flag 256) on the tensor cores
    run("conv2_dgrad", D.conv2d(n, 64, 11, 11, 32, 3, 3, pad=2, bias=False, flip=True, nchw=True), [n * 64 * 121, 64 * 32 * 9], n * 32 * 169)
    run("conv2_wgrad", D.conv2d_wgrad(n, 32, 13, 13, 64, 3, 3), [n * 32 * 169, n * 121 * 64], 64 * 288)
    # conv1 (K = 9): streaming f32 kernels
    run("conv1_forward", D.conv2d(n, 1, 28, 28, 32, 3, 3, relu=True, nchw=True), [n * 784, 288, 32], n * 32 * 676)
    run("conv1_wgrad", D.conv2d_wgrad(n, 1, 28, 28, 32, 3, 3, g_nchw=True), [n * 784, n * 32 * 676], 288)
    print(json.dumps({"only": "conv2d_grad", "kernels": res}))


def extra_measurements(reg, dev, rank, world, local_rank, quick=False):
    """The other BASELINE configurations, timed with CUDA events on the library's
    stream: dense contractions (configs 1 and 5, rank 0 only), the MLP step
    (config 3, rank 0 only) and the data-parallel CNN step (config 4, all ranks)."""
    from harp_b200 import desc as D
    from harp_b200 import workloads as W
    from harp_b200.frontend import B200Executor, Program
    out = {}
    rng = np.random.default_rng(5)
    if rank == 0:
        gemm = {}
        shapes = [("cfg1_512", 512, 512, 512, 0), ("cfg5_8192", 8192, 8192, 8192, 0), ("cfg5_batched_64x1024", 1024, 1024, 1024, 64)]
        for name, m, k_, n, batch in shapes:
            bs = max(batch, 1)
            ba = reg.allocate_buffer(dev, [bs * m * k_]); bb = reg.allocate_buffer(dev, [bs * k_ * n])
            bo = reg.allocate_buffer(dev, [bs * m * n])
            ba.write_vec(rng.uniform(-1, 1, bs * m * k_).astype(np.float32))
            bb.write_vec(rng.uniform(-1, 1, bs * k_ * n).astype(np.float32))
            for mode, mname in ((D.GEMM_TF32, "tf32"), (D.GEMM_3XTF32, "3xtf32")):
                kern = reg.compile_ast(dev, W.matmul_desc(m, k_, n, batch=batch, mode=mode))
                ms = time_kernel(dev, kern, [ba, bb], [bo], reps=3 if quick else 10)
                gemm[f"{name}_{mname}"] = {"impl": kern.impl, "ms": ms, "tflops": 2.0 * bs * m * k_ * n / ms / 1e9}
            for b_ in (ba, bb, bo):
                b_.release()
        out["matmul"] = gemm
        out["conv2d"] = conv_measurements(reg, dev, rng, quick)
        # config 3: MLP training step, whole step as one CUDA graph
        ex = B200Executor(dev, reg)
        loss, ps, grads, _ = W.mlp_graph(65536, 256)
        prog = Program([loss], ex, sgd=list(zip(ps, grads)), lr=1e-3, persistent=True, flat=True)
        prog.capture()
        steps = 20 if quick else 100
        for _ in range(3):
            prog.run()
        dev.synchronize(); dev.timer_begin()
        for _ in range(steps):
            prog.run()
        ms = dev.timer_end() / steps
        out["mlp_cfg3"] = {"ms_per_step": ms, "samples_per_s": 65536 / ms * 1e3, "kernels_per_step": len(prog.kernels) + len(prog.sgd_kernels),
                           "derived_tflops": 2.597e10 / ms / 1e9, "loss_after": float(prog.fetch(loss)), "steps": steps + 3 + 1}
        del prog
    # config 4: CNN, global batch 4096 sharded over the ranks, gradient all-reduce.
    # "cnn_cfg4": this backend's forms of the same functions (one implicit-GEMM kernel per
    # convolution / input gradient / weight gradient, pools over strided views);
    # "cnn_cfg4_reference_spelling" (one GPU only): eclat's own composition of them.
    def cnn_step(fused):
        ex = B200Executor(dev, reg)
        n_local = 4096 // world
        loss, ps, grads, _ = W.cnn_graph(n_local, seed=4 + rank, fused_conv=fused)
        prog = Program([loss], ex, sgd=list(zip(ps, grads)), lr=1e-2 / world, persistent=True, flat=True)
        between = None
        if world > 1:
            from harp_b200 import parallel
            prog.capture(include_update=False)
            between = parallel.make_allreduce(prog.grad_buffers(), "sum", dev, local_rank)
        else:
            prog.capture()
        steps = 5 if quick else 20
        for _ in range(3):
            prog.run(between)
        dev.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        dev.timer_begin()
        for _ in range(steps):
            prog.run(between)
        ms = dev.timer_end() / steps
        if world > 1:
            import torch
            import torch.distributed as dist
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return {"ms_per_step": ms, "img_per_s": 4096 / ms * 1e3, "global_batch": 4096, "per_gpu_batch": n_local,
                "kernels_per_step": len(prog.kernels) + len(prog.sgd_kernels),
                "allreduce_bytes_per_step": 225034 * 4 if world > 1 else 0, "loss_after": float(prog.fetch(loss))}
    out["cnn_cfg4"] = cnn_step(True)
    if world == 1:
        out["cnn_cfg4_reference_spelling"] = cnn_step(False)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="only config 2 (skip matmul / MLP / CNN measurements)")
    ap.add_argument("--only", default="", choices=["", "conv2d", "conv2d_grad"], help="run one small kernel case alone (profiler captures); prints no bench line")
    args = ap.parse_args()
    if args.only:
        run_only_conv(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
