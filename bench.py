#!/usr/bin/env python
"""Benchmark of the hot path on B200: config 2 (fused elementwise + reduce,
column max, transposing copy over x f32 [8192, 8192]).

One step = one pass of the three lowered kernels over one x:
    y = sum(exp(0.5*x + 1.0) * x, axis=1)   fused chain + row reduce   268 468 232 B
    z = max(x, axis=0)                       column reduce              268 468 224 B
    t = x.permute(1,0).contiguous()          transposing copy           536 870 912 B
Algorithmic bytes per step = 1 073 807 368 (each kernel reads x once; outputs
written once).  With N GPUs every rank holds its own [8192, 8192] row block of a
global [8192*N, 8192] tensor (weak scaling); y and t need no exchange, the
column-max partials are combined by one 32 KB MAX all-reduce per step through the
library's own communicator (eb200_comm_*: a one-shot NVLink kernel), issued on
its side stream so the transposing copy overlaps it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Prints ONE JSON line (rank 0).  `value` is device-timed with inputs resident in
HBM; `e2e` goes through the same C-ABI calls with host buffers, host<->device
copies inside the timed region.  `--impl reference` times the reference's CPU
path (the oracle's emitted C with OpenMP, all host threads) on a bounded sample.
`extra` carries the other configurations: dense contractions (configs 1 and 5,
row- / batch-sharded over the ranks), the MLP step (config 3, batch-sharded), the
CNN step (config 4, batch-sharded, gradient all-reduce fused with the update),
config 2 split by rows of ONE tensor (strong scaling), and single-kernel
measurements of the remaining kernel classes.
"""
from __future__ import annotations

import argparse
import ctypes
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
WORKLOAD = ("config 2: y=sum(exp(.5x+1)*x,axis=1), z=max(x,axis=0), t=x.permute(1,0).contiguous(); "
            "x f32 [8192,8192] N(0,1) seed 2")

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures
# summarised under profiles/ (None until a capture exists for that kernel).
NCU_TRAFFIC = {"reduce_inner": 272_698_000, "reduce_outer": 272_148_000, "transpose_copy": 425_400_000}


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s burst, source): the driver-written measurement of this pool's
    B200s when present, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), float(j.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


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
def use_all_host_threads() -> int:
    """Makes OpenMP use every host core and returns the thread count it reports.
    A launcher may have exported OMP_NUM_THREADS=1 (torch.distributed.run does): the
    variable is overwritten, and a runtime that is already loaded is told directly."""
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    try:
        gomp = ctypes.CDLL("libgomp.so.1")
        gomp.omp_set_num_threads(cores)
        return int(gomp.omp_get_max_threads())
    except OSError:
        return cores


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
    threads = use_all_host_threads()
    step, nbytes = run_cpu_workload(x, True, ROWS)
    t0 = time.perf_counter(); step(); first = time.perf_counter() - t0
    best = first
    reps = 1
    while reps < 3 and (reps + 1) * first < seconds_allowed:
        t0 = time.perf_counter(); step(); best = min(best, time.perf_counter() - t0)
        reps += 1
    out = {"value": nbytes / best / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": f"full [8192,8192] workload, emitted C with OpenMP (gcc -O3 -ffast-math -fopenmp) on {threads} threads, best of {reps}",
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
    threads = use_all_host_threads()
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
    sample = f"rows [0,{rows}) of x [8192,8192] per step; emitted C with OpenMP on {threads} host threads (of {os.cpu_count()} cores)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "inputs larger than L2 (x is 256 MiB, L2 126 MB)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
class Ranks:
    """The processes of a multi-GPU run: barrier and max-over-ranks of device timings
    (torch.distributed is the host-side rendezvous only; data-path collectives go
    through the library's communicator)."""

    def __init__(self, rank, local_rank, world):
        self.rank, self.local_rank, self.world = rank, local_rank, world
        if world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            self.torch, self.dist = torch, dist

    def barrier(self, dev):
        dev.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def run_b200(args):
    rank, local_rank, world = dist_env()
    n = args.gpus
    ranks = Ranks(rank, local_rank, world)
    from harp_b200 import desc as D
    from harp_b200 import parallel
    from harp_b200 import workloads as W
    from harp_b200.backend import B200BackendRegistry, PinnedArray, launch_count

    reg = B200BackendRegistry()
    dev = reg.create_device(local_rank)
    comm = parallel.init_comm(dev, rank, world) if world > 1 else None
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

    # the column-max partials of the ranks: "async" = one-shot all-reduce on the communicator's side
    # stream, overlapped with the transposing copy; "fused" = pushed to the peers by the pass that
    # folds the split reduce's partials (one kernel, on the compute stream)
    z_mode = args.z_allreduce if comm is not None else "none"
    if z_mode == "fused":
        comm.attach(kz)

    def step(x=bx, oy=by, oz=bz, ot=bt):
        ky.execute([b0, x, b1], [oy])
        if z_mode == "async":
            comm.join()            # the previous step's all-reduce: it had that step's copy and this y to hide behind
        kz.execute([x], [oz])
        if z_mode == "async":
            comm.allreduce(oz, D.R_MAX, side_stream=True)
        kt.execute([x], [ot])

    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    ranks.barrier(dev)

    # ---- device-timed region: K steps between two events; on every 8th step three more events
    #      separate the kernels (an event between every pair of kernels on every step cost the
    #      region ~10 us per step) ------------------------------------------------------------
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
        if z_mode == "async":
            comm.join()
        e[1].record(); kz.execute([bx], [bz])
        if z_mode == "async":
            comm.allreduce(bz, D.R_MAX, side_stream=True)
        e[2].record(); kt.execute([bx], [bt])
        e[3].record()
    if z_mode == "async":
        comm.join()                # the last step's column maxima are complete inside the timed region
    e_end.record()
    ranks.barrier(dev)
    w1 = time.perf_counter()
    launches = launch_count() - l0
    total_ms = e_begin.elapsed_ms(e_end)
    ns = len(evs)
    t_y = sum(e[0].elapsed_ms(e[1]) for e in evs.values()) / ns
    t_z = sum(e[1].elapsed_ms(e[2]) for e in evs.values()) / ns
    t_t = sum(e[2].elapsed_ms(e[3]) for e in evs.values()) / ns
    # the same three kernels each on its own (20 launches back to back, outside the timed region): inside the
    # step a kernel also pays for the dirty L2 lines its predecessor left behind
    alone_ms = {}
    if n == 1:                # (with several ranks the column reduce may carry its collective: never launched by one rank alone)
        for name, kern_, ins_, out_ in (("y_fused_row_sum", ky, [b0, bx, b1], by), ("z_col_max", kz, [bx], bz), ("t_transpose", kt, [bx], bt)):
            alone_ms[name] = time_kernel(dev, kern_, ins_, [out_], reps=20, warm=3)

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
        for i in range(steps):
            sl = i & 1
            if i >= 2:                         # the kernels that last read this slot must be done
                dev.wait_event(ev_k[sl], up)
            xs[sl].write_on(up, x_host.ptr, x_host.nbytes)
            ev_up[sl].record(up)
            dev.wait_event(ev_up[sl])          # compute stream: kernels of batch i wait for its upload
            if i >= 2:
                dev.wait_event(ev_down[sl])    # ... and for the previous results of this slot to have left
            oy, oz, ot = outs[sl]
            step(xs[sl], oy, oz, ot)
            if z_mode == "async":
                comm.join()                    # z leaves the device with this step's results
            ev_k[sl].record()
            dev.wait_event(ev_k[sl], down)     # download batch i's results
            oy.read_on(down, y_host.ptr, y_host.nbytes)
            oz.read_on(down, z_host.ptr, z_host.nbytes)
            ot.read_on(down, t_host.ptr, t_host.nbytes)
            ev_down[sl].record(down)
        down.synchronize()                     # the caller holds every result
        dev.synchronize()
    e2e_run(2)
    ranks.barrier(dev)
    ea, eb = dev.event(), dev.event()
    w2 = time.perf_counter()
    ea.record()
    e2e_run(KE)
    eb.record()
    ranks.barrier(dev)
    w3 = time.perf_counter()
    e2e_ms = ea.elapsed_ms(eb)
    sampler.stop()

    # the other way of combining the column maxima, for the record (multi-GPU runs only)
    z_other = None
    if comm is not None:
        other = "fused" if z_mode == "async" else "async"
        kz2 = reg.compile_ast(dev, W.cfg2_z())
        if other == "fused":
            comm.attach(kz2)

        def step_other():
            ky.execute([b0, bx, b1], [by])
            if other == "async":
                comm.join()
            kz2.execute([bx], [bz])
            if other == "async":
                comm.allreduce(bz, D.R_MAX, side_stream=True)
            kt.execute([bx], [bt])
        for _ in range(3):
            step_other()
        ranks.barrier(dev)
        dev.timer_begin()
        for _ in range(K):
            step_other()
        comm.join()
        ms_other = ranks.max([dev.timer_end() / K])[0]
        z_other = {"z_allreduce": other, "ms_per_step": ms_other, "value_gbs": BYTES_STEP * n / (ms_other * 1e-3) / 1e9}
        ranks.barrier(dev)

    # release the config 2 buffers, then time the other configurations
    extra = None
    if not args.no_extra:
        for b_ in (bx, by, bz, bt, xs[1], outs[1][0], outs[1][1], outs[1][2]):
            b_.release()
        for h_ in (y_host, z_host, t_host):
            h_.free()
        extra = extra_measurements(reg, dev, ranks, comm, quick=args.steps < 20)
        if "cfg2_single_pass" in extra:
            extra["cfg2_single_pass"]["speedup_over_three_kernels"] = (total_ms / K) / extra["cfg2_single_pass"]["ms_per_step"]
        if z_other:
            extra["cfg2_z_allreduce_other_way"] = z_other
    total_ms, e2e_ms, t_y, t_z, t_t = ranks.max([total_ms, e2e_ms, t_y, t_z, t_t])
    comm_info = comm.info() if comm is not None else None
    if rank != 0:
        ranks.close()
        return

    peak, peak_tf, peak_kind = measured_peaks()
    value = BYTES_STEP * n * K / (total_ms * 1e-3) / 1e9
    e2e = BYTES_STEP * n * KE / (e2e_ms * 1e-3) / 1e9
    kernels = {}
    for name, impl, b, ms in (("y_fused_row_sum", ky.impl, BYTES_Y, t_y), ("z_col_max", kz.impl, BYTES_Z, t_z),
                              ("t_transpose", kt.impl, BYTES_T, t_t)):
        gbs = b / (ms * 1e-3) / 1e9
        kernels[name] = {"impl": impl, "ms": ms, "algo_bytes": b, "achieved_gbs": gbs, "frac_of_" + peak_kind: gbs / peak}
        if name in alone_ms:
            kernels[name]["alone_ms"] = alone_ms[name]
            kernels[name]["alone_frac_of_" + peak_kind] = b / (alone_ms[name] * 1e-3) / 1e9 / peak
    top = max(kernels.items(), key=lambda kv: kv[1]["ms"])
    traffic = NCU_TRAFFIC.get("transpose_copy" if top[0] == "t_transpose" else
                              ("reduce_outer" if top[0] == "z_col_max" else "reduce_inner"))
    roofline = {"bound": "hbm", "kernel": top[1]["impl"], "achieved": top[1]["achieved_gbs"], "peak": peak,
                "peak_source": f"{peak_kind} copy bandwidth (MEASURED_PEAKS.json)" if peak_kind == "measured" else "fallback 6650 GB/s",
                "unit": "GB/s", "frac": top[1]["achieved_gbs"] / peak, "traffic": traffic,
                "time_share": top[1]["ms"] / (t_y + t_z + t_t),
                "step_frac": BYTES_STEP / (total_ms / K * 1e-3) / 1e9 / peak}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "l2": "inputs larger than L2 (x is 256 MiB, L2 126 MB)",
                   "per_gpu": "every GPU holds its own [8192,8192] block (seed 2 + rank)",
                   "sharding": ("row blocks of a global [8192*N, 8192] tensor; MAX all-reduce of the 32 KB column-max partials: " +
                                ("one-shot NVLink kernel on a side stream, overlapped with the transposing copy" if z_mode == "async"
                                 else "pushed to the peers by the pass that folds the split reduce's partials")) if n > 1 else "single GPU",
                   "algo_bytes_per_step_per_gpu": BYTES_STEP,
                   "kernel_events": f"per-kernel durations from events on every {SAMPLE}th timed step ({ns} of {K})"},
        "roofline": roofline, "kernels": kernels,
        "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(x_host.nbytes),
                "d2h_bytes_per_step": int(4 * ROWS + 4 * COLS + 4 * ROWS * COLS), "steps": KE,
                "ms_per_step": e2e_ms / KE},
        "gpu_launches": int(launches),
        "clocks": sampler.summary([(w0, w1), (w2, w3)]),
    }
    if comm_info is not None:
        line["comm"] = comm_info
    if n == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(x_host.array)
    if extra is not None:
        line["extra"] = extra
    print(json.dumps(line))
    ranks.close()


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


def kernel_table(dev, prog, reps=10):
    """Device time of every kernel of a program on its own: `reps` launches of the kernel recorded
    into a CUDA graph and replayed (so host launch cost stays out of it; the figure includes the
    ~1-2 us gap between dependent launches, as the captured step does):
    [impl, us, algorithmic MB, algorithmic GFLOP] per kernel, in launch order."""
    rows = []
    for i, d, kern, srcs in prog.kernels:
        ins, out = [prog._b(s_) for s_ in srcs], [prog.buf[prog.where[i][0]]]
        dev.synchronize()
        dev.graph_begin()
        try:
            for _ in range(reps):
                kern.execute(ins, out)
        finally:
            graph = dev.graph_end()
        graph.launch()
        dev.synchronize()
        dev.timer_begin()
        graph.launch()
        ms = dev.timer_end() / reps
        rows.append([kern.impl, round(ms * 1e3, 2), round(kern.algo_bytes / 1e6, 3), round(kern.algo_flops / 1e9, 4)])
    return rows


def step_bound_ms(prog, hbm_gbs, tf32_tflops):
    """Lower bound of a step from its kernels' algorithmic work: each kernel can go no faster than its
    bytes over the HBM copy bandwidth or its flops over the tensor peak of its arithmetic mode."""
    from harp_b200 import desc as D
    t = 0.0
    for _, d, kern, _ in prog.kernels:
        three = d.gemm_mode != D.GEMM_TF32
        t += max(kern.algo_bytes / (hbm_gbs * 1e9), kern.algo_flops * (3 if three else 1) / (tf32_tflops * 1e12))
    return t * 1e3


def extra_measurements(reg, dev, ranks, comm, quick=False):
    """The other configurations, timed with CUDA events on the library's stream, every
    rank working on its shard (max over ranks): dense contractions (config 1 on rank 0;
    config 5 with A and C split by rows and B replicated, the batched form split by batch
    index), the MLP step (config 3) and the CNN step (config 4) batch-sharded with the
    gradient all-reduce fused into the update, config 2 split by rows of ONE tensor, and on
    one GPU the convolution layers and the remaining kernel classes alone."""
    from harp_b200 import desc as D
    from harp_b200 import parallel
    from harp_b200 import workloads as W
    from harp_b200.frontend import B200Executor, Program
    rank, world = ranks.rank, ranks.world
    hbm, bf16_tf, peak_kind = measured_peaks()
    tf32_peak = bf16_tf / 2.0
    out = {"peaks": {"hbm_gbs": hbm, "tf32_tflops": tf32_peak, "source": peak_kind + " (TF32 taken as half the dense bf16 figure)"}}
    rng = np.random.default_rng(5)
    w = D.Ast.w

    # ---- configs 1 and 5: dense contractions ------------------------------------------------
    gemm = {}
    shapes = [("cfg1_512", 512, 512, 512, 0, False), ("cfg5_8192", 8192, 8192, 8192, 0, True),
              ("cfg5_batched_64x1024", 1024, 1024, 1024, 64, True)]
    for name, m, k_, n, batch, sharded in shapes:
        if not sharded and rank != 0:
            continue
        if batch:
            lo, hi = parallel.batch_shard(batch, rank, world)
            bs, ml = hi - lo, m
        else:
            sh = parallel.gemm_row_shard(m, k_, n, rank, world) if sharded else {"m_local": m}
            bs, ml = 1, sh["m_local"]
        ba = reg.allocate_buffer(dev, [bs * ml * k_]); bb = reg.allocate_buffer(dev, [bs * k_ * n])
        bo = reg.allocate_buffer(dev, [bs * ml * n])
        ba.write_vec(rng.uniform(-1, 1, bs * ml * k_).astype(np.float32))
        bb.write_vec(rng.uniform(-1, 1, bs * k_ * n).astype(np.float32))       # B: replicated in this GPU's own memory
        for mode, mname in ((D.GEMM_TF32, "tf32"), (D.GEMM_3XTF32, "3xtf32")):
            kern = reg.compile_ast(dev, W.matmul_desc(ml, k_, n, batch=bs if batch else 0, mode=mode))
            if sharded:
                ranks.barrier(dev)
            ms = time_kernel(dev, kern, [ba, bb], [bo], reps=3 if quick else 10)
            if sharded:
                ms = ranks.max([ms])[0]
            flops = 2.0 * max(batch, 1) * m * k_ * n
            tf = flops / ms / 1e9
            gemm[f"{name}_{mname}"] = {"impl": kern.impl, "ms": ms, "tflops": tf,
                                       "frac_of_tf32_peak": tf * (3 if mode == D.GEMM_3XTF32 else 1) / (tf32_peak * (world if sharded else 1)),
                                       "per_gpu": f"A,C rows {ml} of {m}, B replicated" if not batch else f"batches {bs} of {batch}",
                                       "n_gpus": world if sharded else 1}
        for b_ in (ba, bb, bo):
            b_.release()
    out["matmul"] = gemm

    # ---- config 2 split by rows of ONE [8192, 8192] tensor (strong scaling) -----------------
    if world > 1:
        lo, hi = parallel.shard_range(ROWS, rank, world)
        rl = hi - lo
        x = W.cfg2_input(ROWS, COLS)[lo:hi]
        c0, c1 = W.cfg2_consts()
        bx = reg.allocate_buffer(dev, [rl, COLS]); bx.write_vec(x)
        b0 = reg.allocate_buffer(dev, [1]); b0.write_vec(c0)
        b1 = reg.allocate_buffer(dev, [1]); b1.write_vec(c1)
        by, bz, bt = reg.allocate_buffer(dev, [rl]), reg.allocate_buffer(dev, [COLS]), reg.allocate_buffer(dev, [COLS * rl])
        ky, kz, kt = (reg.compile_ast(dev, f(rl, COLS)) for f in (W.cfg2_y, W.cfg2_z, W.cfg2_t))

        def strong_step():
            ky.execute([b0, bx, b1], [by])
            comm.join()
            kz.execute([bx], [bz])
            comm.allreduce(bz, D.R_MAX, side_stream=True)
            kt.execute([bx], [bt])
        for _ in range(3):
            strong_step()
        ranks.barrier(dev)
        steps = 20 if quick else 100
        dev.timer_begin()
        for _ in range(steps):
            strong_step()
        comm.join()
        ms = ranks.max([dev.timer_end() / steps])[0]
        out["cfg2_strong"] = {"ms_per_step": ms, "value_gbs": BYTES_STEP / (ms * 1e-3) / 1e9, "rows_per_gpu": rl,
                              "sharding": "rows [r*8192/g, (r+1)*8192/g) of ONE [8192,8192] tensor; y and t stay sharded, z by a 32 KB MAX all-reduce",
                              "algo_bytes_per_step_total": BYTES_STEP}
        for b_ in (bx, by, bz, bt):
            b_.release()

    if world == 1:
        # config 2's three roots from ONE pass over x (sibling fusion): read x once, write t once
        c0, c1 = W.cfg2_consts()
        bx = reg.allocate_buffer(dev, [ROWS * COLS]); bx.write_vec(W.cfg2_input(ROWS, COLS))
        b0 = reg.allocate_buffer(dev, [1]); b0.write_vec(c0)
        b1 = reg.allocate_buffer(dev, [1]); b1.write_vec(c1)
        ks = reg.compile_ast(dev, W.cfg2_siblings())
        bo = reg.allocate_buffer(dev, [int(ks.desc.output.numel)])
        ms = time_kernel(dev, ks, [b0, bx, b1], [bo], reps=5 if quick else 20)
        single = 4 * ROWS * COLS + 4 * ROWS * COLS + 4 * ROWS + 4 * COLS          # x once in, t once out, y and z
        out["cfg2_single_pass"] = {"impl": ks.impl, "ms_per_step": ms, "algo_bytes_per_step": single,
                                   "value_gbs": single / ms / 1e6, "frac_of_hbm": single / ms / 1e6 / hbm,
                                   "accounting": "one fused pass: 4*8192^2 read + 4*8192^2 written + y + z = 536 936 448 B "
                                                 "(the headline line charges the three separate kernels 1 073 807 368 B)",
                                   "speedup_over_three_kernels": None}
        for b_ in (bx, b0, b1, bo):
            b_.release()
        out["conv2d"] = conv_measurements(reg, dev, rng, quick)
        out["kernels_alone"] = misc_kernel_measurements(reg, dev, rng, hbm, quick)

    # ---- configs 3 and 4: training steps, batch-sharded, whole step as one CUDA graph -------
    one_shot = comm is None or comm.info()["one_shot"]

    def train_step(build, n_global, lr, steps, tables=False):
        ex = B200Executor(dev, reg)
        n_local = n_global // world
        loss, ps, grads, _ = build(n_local)
        prog = Program([loss], ex, sgd=list(zip(ps, grads)), lr=lr / world, persistent=True, flat=True,
                       comm=comm, overlap=one_shot)
        # with the one-shot transport the collective is part of the recorded step; a communicator that
        # fell back to NCCL keeps its collective outside the graph
        prog.capture(include_update=one_shot)
        for _ in range(3):
            prog.run()
        ranks.barrier(dev)
        dev.timer_begin()
        for _ in range(steps):
            prog.run()
        ms = ranks.max([dev.timer_end() / steps])[0]
        res = {"ms_per_step": ms, "global_batch": n_global, "per_gpu_batch": n_local,
               "kernels_per_step": len(prog.kernels) + (len(prog.sgd_kernels) if comm is None else 1 + len(prog.buckets)),
               "all_specialised": all(k.specialised for _, _, k, _ in prog.kernels),
               "allreduce_bytes_per_step": 4 * prog.cnumel[-1] if comm is not None else 0,
               "overlapped_bucket": [list(b) for b in prog.buckets],
               "loss_after": float(prog.fetch(loss)), "steps": steps + 3 + 1}
        bound = step_bound_ms(prog, hbm, tf32_peak)
        res["roofline"] = {"bound_ms": bound, "frac": bound / ms,
                           "how": "sum over the step's kernels of max(algorithmic bytes / HBM copy bandwidth, executed flops / TF32 peak)"}
        if tables and rank == 0:
            res["kernel_table_us"] = kernel_table(dev, prog)
        return res, prog

    steps = 20 if quick else 100
    res, prog = train_step(lambda nl: W.mlp_graph(nl, 256, seed=3 + rank), 65536, 1e-3, steps, tables=True)
    res["samples_per_s"] = 65536 / res["ms_per_step"] * 1e3
    res["derived_tflops"] = 2.597e10 / res["ms_per_step"] / 1e9
    out["mlp_cfg3"] = res
    del prog
    # "cnn_cfg4": this backend's forms of the same functions (one implicit-GEMM kernel per
    # convolution / input gradient / weight gradient, pools over strided views);
    # "cnn_cfg4_reference_spelling" (one GPU only): eclat's own composition of them.
    res, prog = train_step(lambda nl: W.cnn_graph(nl, seed=4 + rank, fused_conv=True), 4096, 1e-2, 5 if quick else 20, tables=True)
    res["img_per_s"] = 4096 / res["ms_per_step"] * 1e3
    out["cnn_cfg4"] = res
    del prog
    if world == 1:
        # the 8-GPU shard size on one GPU: what does not shrink with the shard shows here
        res, prog = train_step(lambda nl: W.cnn_graph(512, seed=4, fused_conv=True), 512, 1e-2, 5 if quick else 20, tables=True)
        res["img_per_s"] = 512 / res["ms_per_step"] * 1e3
        out["cnn_cfg4_shard_512"] = res
        del prog
        res, prog = train_step(lambda nl: W.cnn_graph(nl, seed=4, fused_conv=False), 4096, 1e-2, 3 if quick else 10, tables=True)
        res["img_per_s"] = 4096 / res["ms_per_step"] * 1e3
        out["cnn_cfg4_reference_spelling"] = res
        del prog
    return out


def W_matmul(m, k, n):
    from harp_b200 import workloads as W
    return W.matmul_desc(m, k, n)


def misc_kernel_measurements(reg, dev, rng, hbm, quick=False):
    """Kernel classes that no configuration's headline covers, each alone on inputs larger
    than L2: scans, optimizer updates, scatter-add, a plain elementwise add."""
    from harp_b200 import desc as D
    w = D.Ast.w
    res = {}

    def run(name, kd, sizes, out_size, dtypes=None, in_place=None):
        bufs = []
        for j, sz in enumerate(sizes):
            dt = dtypes[j] if dtypes else D.F32
            b = reg.allocate_buffer(dev, [sz], dt)
            if dt == D.F32:
                b.write_vec(rng.uniform(-1, 1, sz).astype(np.float32))
            elif dt in (D.F16, D.BF16):
                x = rng.uniform(-1, 1, sz).astype(np.float32)
                b.write_vec(x.astype(np.float16) if dt == D.F16 else D.bf16_bits(x))
            bufs.append(b)
        bo = bufs[in_place] if in_place is not None else reg.allocate_buffer(dev, [out_size], kd.output.dtype)
        kern = reg.compile_ast(dev, kd)
        ms = time_kernel(dev, kern, bufs, [bo], reps=3 if quick else 10)
        gbs = kern.algo_bytes / ms / 1e6
        res[name] = {"impl": kern.impl, "ms": ms, "algo_bytes": kern.algo_bytes, "gbs": gbs, "frac_of_hbm": gbs / hbm}
        for b in bufs + ([] if in_place is not None else [bo]):
            b.release()
    n = 1 << 26                      # 256 MiB per operand
    run("ew_add", D.elementwise([n], [D.contiguous([n])] * 2, w(0) + w(1)), [n, n], n)
    run("cumsum_rows_8192x8192", D.scan([8192, 8192], [D.contiguous([8192, 8192])], w(0), D.R_SUM, 1), [n], n)
    run("cumsum_rows_65536x1024", D.scan([65536, 1024], [D.contiguous([65536, 1024])], w(0), D.R_SUM, 1), [n], n)
    run("cumsum_4_long_rows", D.scan([4, n // 4], [D.contiguous([4, n // 4])], w(0), D.R_SUM, 1), [n], n)
    run("sgd_update", D.KernelDesc(D.K_SGD, [n], [D.contiguous([n])] * 2, D.contiguous([n]), scalar=0.01), [n, n], n, in_place=0)
    run("sgd_momentum_update", D.sgd_momentum(n, 0.01, 0.9), [n, n, n], n, in_place=0)
    run("adam_update", D.adam(n, 1e-3), [n, n, n, n, 1], n, dtypes=[D.F32] * 4 + [D.I32], in_place=0)
    # fold of 3x3 windows, the scatter-add the reference reaches through unfold's gradient: [512,32,11,11,3,3] -> [512,32,13,13]
    from harp_b200.frontend import View
    src_shape, dst_shape = [512, 32, 11, 11, 3, 3], [512, 32, 13, 13]
    dst = View.contiguous(dst_shape).unfold([2, 3], [3, 3], [1, 1], [1, 1])
    kd = D.KernelDesc(D.K_SCATTER, src_shape, [D.contiguous(src_shape)], dst.operand(int(np.prod(dst_shape)), D.F32), None)
    run("scatter_add_fold3x3", kd, [int(np.prod(src_shape))], int(np.prod(dst_shape)))
    # a bias gradient: column sums of [2.77 M, 32] (few kept elements: column threads x row lanes)
    rows = 4096 * 676
    run("bias_grad_colsum_2768896x32", D.reduce([rows, 32], [D.contiguous([rows, 32])], w(0), D.R_SUM, 0), [rows * 32], 32)
    # a first-layer weight gradient as a contraction: dW[32, 9] over 2.77 M positions (one output tile, long K)
    a = D.Operand([32, 1, 0], 0, D.F32, rows * 32)
    b = D.Operand([9, 0, 1], 0, D.F32, rows * 9)
    run("tall_wgrad_32x9_over_2768896", D.reduce([rows, 32, 9], [a, b], w(0) * w(1), D.R_SUM, 0), [rows * 32, rows * 9], 32 * 9)
    # a contraction on the f32 FFMA kernel (row stride not a multiple of 16 bytes: TMA cannot address it)
    run("gemm_simt_2048x1022x2048", W_matmul(2048, 1022, 2048), [2048 * 1022, 1022 * 2048], 2048 * 2048)
    # ReLU + 2x2 max-pool of config 4's first layer at batch 4096, forward and gradient, one kernel each
    planes = 4096 * 32
    run("relu_maxpool2_fwd_131072x26x26", D.maxpool2d(planes, 26, 26, 2, relu=True), [planes * 676], planes * 169)
    run("relu_maxpool2_grad_131072x26x26", D.maxpool2d(planes, 26, 26, 2, relu=True, grad=True),
        [planes * 169, planes * 676, planes * 169], planes * 676)
    # 16-bit storage: elements widen to f32 in registers, 64-bit accesses
    run("ew_add_bf16", D.elementwise([2 * n], [D.contiguous([2 * n], D.BF16)] * 2, w(0) + w(1), out_dtype=D.BF16), [2 * n, 2 * n], 2 * n,
        dtypes=[D.BF16, D.BF16])
    # 16-bit contractions on tcgen05 kind::f16 (x @ W^T form, f32 accumulate, f32 result)
    for dt, tag in ((D.BF16, "bf16"), (D.F16, "f16")):
        for m_, n_, k_ in ((8192, 8192, 8192),) if not quick else ((2048, 2048, 2048),):
            a = D.Operand([k_, 0, 1], 0, dt, m_ * k_)
            b = D.Operand([0, k_, 1], 0, dt, n_ * k_)
            kd = D.reduce([m_, n_, k_], [a, b], w(0) * w(1), D.R_SUM, 2, out=D.Operand([n_, 1, 0], 0, D.F32, m_ * n_))
            name = f"gemm_{tag}_{m_}x{n_}x{k_}"
            run(name, kd, [m_ * k_, n_ * k_], m_ * n_, dtypes=[dt, dt])
            res[name]["tflops"] = 2.0 * m_ * n_ * k_ / res[name]["ms"] / 1e9
            res[name]["frac_of_bf16_peak"] = res[name]["tflops"] / measured_peaks()[1]
            del res[name]["gbs"], res[name]["frac_of_hbm"]
    return res


def run_only_small(args):
    """`--only gemm`: the tensor-core contraction on a 4096 x 2048 x 4096 case; `--only cfg2`: the
    config 2 kernels and the one-pass sibling form on a [4096, 8192] block; `--only kernels`: the
    kernel classes of misc_kernel_measurements; `--only gemm16`: a 4096^3 bf16 / f16 contraction; `--only pool`: the
    fused ReLU + max-pool kernels and a bf16 elementwise add; `--only mlp` / `--only cnn`: the kernels of one training
    step of config 3 / of config 4's 512-image shard (small cases for profiler captures)."""
    from harp_b200 import desc as D
    from harp_b200 import workloads as W
    from harp_b200.backend import B200BackendRegistry
    reg = B200BackendRegistry()
    dev = reg.create_device(0)
    rng = np.random.default_rng(5)
    hbm, _, _ = measured_peaks()
    if args.only == "gemm":
        res = {}
        m, k_, n = 4096, 2048, 4096          # 256 pair tiles: the persistent two-CTA kernel; 64 + 32 + 64 MiB
        ba, bb, bo = reg.allocate_buffer(dev, [m * k_]), reg.allocate_buffer(dev, [k_ * n]), reg.allocate_buffer(dev, [m * n])
        ba.write_vec(rng.uniform(-1, 1, m * k_).astype(np.float32)); bb.write_vec(rng.uniform(-1, 1, k_ * n).astype(np.float32))
        for mode, mname in ((D.GEMM_TF32, "tf32"), (D.GEMM_3XTF32, "3xtf32")):
            kern = reg.compile_ast(dev, W.matmul_desc(m, k_, n, mode=mode))
            ms = time_kernel(dev, kern, [ba, bb], [bo], reps=2, warm=1)
            res[mname] = {"impl": kern.impl, "ms": ms, "tflops": 2.0 * m * k_ * n / ms / 1e9}
        print(json.dumps({"only": "gemm", "gemm_4096x2048x4096": res}))
        return
    if args.only == "cfg2":
        # the config 2 kernels on a [4096, 8192] block (128 MiB, larger than L2), plus the one-pass sibling form
        rows = 4096
        c0, c1 = W.cfg2_consts()
        bx = reg.allocate_buffer(dev, [rows * COLS]); bx.write_vec(W.cfg2_input(rows, COLS))
        b0 = reg.allocate_buffer(dev, [1]); b0.write_vec(c0)
        b1 = reg.allocate_buffer(dev, [1]); b1.write_vec(c1)
        res = {}
        for name, kd, ins in (("y", W.cfg2_y(rows, COLS), [b0, bx, b1]), ("z", W.cfg2_z(rows, COLS), [bx]),
                              ("t", W.cfg2_t(rows, COLS), [bx]), ("siblings", W.cfg2_siblings(rows, COLS), [b0, bx, b1])):
            kern = reg.compile_ast(dev, kd)
            bo = reg.allocate_buffer(dev, [int(kd.output.numel)])
            ms = time_kernel(dev, kern, ins, [bo], reps=3, warm=2)
            res[name] = {"impl": kern.impl, "ms": ms, "gbs": kern.algo_bytes / ms / 1e6}
            bo.release()
        print(json.dumps({"only": "cfg2", "rows": rows, "kernels": res}))
        return
    if args.only == "gemm16":
        # bf16 / f16 contraction 4096^3 on the persistent pair kernel (32 MiB per operand, 64 MiB result)
        res = {}
        m = k_ = n = 4096
        for dt, tag in ((D.BF16, "bf16"), (D.F16, "f16")):
            x = rng.uniform(-1, 1, m * k_).astype(np.float32)
            ba, bb = reg.allocate_buffer(dev, [m * k_], dt), reg.allocate_buffer(dev, [n * k_], dt)
            ba.write_vec(x.astype(np.float16) if dt == D.F16 else D.bf16_bits(x)); bb.write_vec(x.astype(np.float16) if dt == D.F16 else D.bf16_bits(x))
            bo = reg.allocate_buffer(dev, [m * n])
            kd = D.reduce([m, n, k_], [D.Operand([k_, 0, 1], 0, dt, m * k_), D.Operand([0, k_, 1], 0, dt, n * k_)], D.Ast.w(0) * D.Ast.w(1),
                          D.R_SUM, 2, out=D.Operand([n, 1, 0], 0, D.F32, m * n))
            kern = reg.compile_ast(dev, kd)
            ms = time_kernel(dev, kern, [ba, bb], [bo], reps=2, warm=1)
            res[tag] = {"impl": kern.impl, "ms": ms, "tflops": 2.0 * m * k_ * n / ms / 1e9}
        print(json.dumps({"only": "gemm16", "gemm_4096x4096x4096": res}))
        return
    if args.only == "pool":
        # ReLU + 2x2 max-pool of config 4's first layer at batch 1024 (88 MiB in), forward and gradient, and a bf16 add
        planes = 1024 * 32
        res = {}
        bx = reg.allocate_buffer(dev, [planes * 676]); bx.write_vec(rng.standard_normal(planes * 676).astype(np.float32))
        by, bg, bgx = reg.allocate_buffer(dev, [planes * 169]), reg.allocate_buffer(dev, [planes * 169]), reg.allocate_buffer(dev, [planes * 676])
        bg.write_vec(rng.standard_normal(planes * 169).astype(np.float32))
        for name, kd, ins, out in (("fwd", D.maxpool2d(planes, 26, 26, 2, relu=True), [bx], by),
                                   ("grad", D.maxpool2d(planes, 26, 26, 2, relu=True, grad=True), [bg, bx, by], bgx)):
            kern = reg.compile_ast(dev, kd)
            ms = time_kernel(dev, kern, ins, [out], reps=3, warm=2)
            res[name] = {"impl": kern.impl, "ms": ms, "gbs": kern.algo_bytes / ms / 1e6}
        n16 = 1 << 26
        x = rng.uniform(-1, 1, n16).astype(np.float32)
        ba, bb, bo = (reg.allocate_buffer(dev, [n16], D.BF16) for _ in range(3))
        ba.write_vec(D.bf16_bits(x)); bb.write_vec(D.bf16_bits(x))
        kern = reg.compile_ast(dev, D.elementwise([n16], [D.contiguous([n16], D.BF16)] * 2, D.Ast.w(0) + D.Ast.w(1), out_dtype=D.BF16))
        ms = time_kernel(dev, kern, [ba, bb], [bo], reps=3, warm=2)
        res["ew_add_bf16"] = {"impl": kern.impl, "ms": ms, "gbs": kern.algo_bytes / ms / 1e6}
        print(json.dumps({"only": "pool", "kernels": res}))
        return
    if args.only in ("mlp", "cnn"):
        # one training step of config 3 (batch 65536) / config 4 (batch 512), kernel by kernel, no graph:
        # every buffer is at most 67 MB, so a profiler capture of a few launches stays small
        from harp_b200.frontend import B200Executor, Program
        ex = B200Executor(dev, reg)
        loss, ps, grads, _ = W.mlp_graph(65536, 256) if args.only == "mlp" else W.cnn_graph(512, fused_conv=True)
        prog = Program([loss], ex, sgd=list(zip(ps, grads)), lr=1e-3, persistent=True, flat=True)
        for _ in range(2):
            prog.run()
        dev.synchronize()
        print(json.dumps({"only": args.only, "kernels": [k.impl for _, _, k, _ in prog.kernels], "table_us": kernel_table(dev, prog, reps=3),
                          "loss": float(prog.fetch(loss))}))
        return
    print(json.dumps({"only": "kernels", "kernels": misc_kernel_measurements(reg, dev, rng, hbm, quick=True)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="only config 2 (skip matmul / MLP / CNN measurements)")
    ap.add_argument("--z-allreduce", default="async", choices=["async", "fused"],
                    help="multi-GPU: how the column-max partials are combined (side-stream all-reduce, or fused into the reduce's finish pass)")
    ap.add_argument("--only", default="", choices=["", "conv2d", "conv2d_grad", "gemm", "gemm16", "pool", "kernels", "cfg2", "mlp", "cnn"],
                    help="run one small kernel case alone (profiler captures); prints no bench line")
    args = ap.parse_args()
    if args.only in ("conv2d", "conv2d_grad"):
        run_only_conv(args)
    elif args.only:
        run_only_small(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
