"""Host-side mirror of eclat's backend plugin surface for the B200 backend.

Same names, argument meaning and error behaviour as the Rust traits a backend
crate implements, so code (and tests) written against the reference's
``BackendRegistry`` / ``Device`` / ``Buffer`` / ``Kernel`` read the same here:

* ``B200BackendRegistry`` -- ``BackendRegistry`` (src/backend/device.rs:83-171)
* ``B200Device``          -- ``Device``          (src/backend/traits.rs:273-306)
* ``B200Buffer``          -- ``Buffer``/``TypedBuffer`` (src/backend/traits.rs:312-482)
* ``B200Kernel``          -- ``Kernel``          (src/backend/traits.rs:531-587)

Where the reference passes a lowered ``AstNode::Program`` holding one
``Kernel`` to ``compile_ast``, this mirror passes the equivalent
``harp_b200.desc.KernelDesc``.  Everything executes through ``libeb200.so``.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Sequence

import numpy as np

from . import capi
from . import desc as D


class DeviceError(RuntimeError):
    """DeviceError (src/backend/device.rs:30-60)."""


class B200Device:
    """One B200 with its stream and stream-ordered memory pool."""

    def __init__(self, handle: C.c_void_p, index: int):
        self._h = handle
        self.index = index
        props = D.CDeviceProps()
        capi.call("eb200_device_get_props", self._h, C.byref(props))
        self.name = props.name.decode()
        self.sm_count = props.sm_count
        self.cc = (props.cc_major, props.cc_minor)
        self.total_mem_bytes = props.total_mem_bytes
        self.l2_bytes = props.l2_bytes

    @staticmethod
    def is_available() -> bool:
        return B200BackendRegistry().is_available()

    def profile(self) -> dict:
        """DeviceProfile (src/backend/traits.rs:163-199)."""
        return {"device_type": "Gpu", "compute_units": self.sm_count, "max_work_group_size": 1024,
                "warp_size": 32, "preferred_tile_sizes": [64, 128], "local_memory_size": 227 * 1024}

    def synchronize(self):
        capi.call("eb200_device_sync", self._h)

    def stream(self) -> int:
        s = C.c_void_p()
        capi.call("eb200_device_stream", self._h, C.byref(s))
        return s.value or 0

    def timer_begin(self):
        capi.call("eb200_timer_begin", self._h)

    def timer_end(self) -> float:
        ms = C.c_float()
        capi.call("eb200_timer_end", self._h, C.byref(ms))
        return ms.value

    def event(self) -> "B200Event":
        return B200Event(self)

    def copy_stream(self) -> "B200Stream":
        """A side stream for host<->device copies that overlap compute."""
        return B200Stream(self)

    def wait_event(self, ev: "B200Event", stream: "B200Stream" = None):
        """Make `stream` (default: this device's compute stream) wait for `ev`."""
        capi.call("eb200_stream_wait", self._h, stream._h if stream else None, ev._h)

    def graph_begin(self):
        """Start recording launches on this device into a CUDA graph."""
        capi.call("eb200_graph_begin", self._h)

    def graph_end(self) -> "B200Graph":
        h = C.c_void_p()
        capi.call("eb200_graph_end", self._h, C.byref(h))
        return B200Graph(h)

    def mem_stats(self) -> dict:
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        capi.call("eb200_device_mem_stats", self._h, C.byref(a), C.byref(b), C.byref(c))
        return {"in_use": a.value, "peak": b.value, "n_allocs": c.value}

    def close(self):
        if self._h:
            capi.call("eb200_device_close", self._h)
            self._h = None


class B200Stream:
    def __init__(self, device: "B200Device"):
        self.device = device
        self._h = C.c_void_p()
        capi.call("eb200_stream_create", device._h, C.byref(self._h))

    def synchronize(self):
        capi.call("eb200_stream_sync", self._h)

    def __del__(self):
        try:
            if self._h:
                capi.call("eb200_stream_destroy", self._h)
                self._h = None
        except Exception:
            pass


class B200Graph:
    """A recorded step; ``launch`` replays it with one submission."""

    def __init__(self, handle):
        self._h = handle

    def launch(self):
        capi.call("eb200_graph_launch", self._h)

    def __del__(self):
        try:
            if self._h:
                capi.call("eb200_graph_release", self._h)
                self._h = None
        except Exception:
            pass


class B200Event:
    """A timing point on the device stream."""

    def __init__(self, device: "B200Device"):
        self._h = C.c_void_p()
        capi.call("eb200_event_create", device._h, C.byref(self._h))

    def record(self, stream: "B200Stream" = None):
        if stream is None:
            capi.call("eb200_event_record", self._h)
        else:
            capi.call("eb200_event_record_on", self._h, stream._h)

    def elapsed_ms(self, later: "B200Event") -> float:
        ms = C.c_float()
        capi.call("eb200_event_elapsed_ms", self._h, later._h, C.byref(ms))
        return ms.value

    def __del__(self):
        try:
            if self._h:
                capi.call("eb200_event_destroy", self._h)
                self._h = None
        except Exception:
            pass


class B200Buffer:
    """Device buffer.  ``write_from_host`` rejects a size mismatch like
    CBuffer (crates/backend-c/src/buffer.rs:151-160); ``clone_buffer`` is a
    value copy (shared storage, copy-on-write)."""

    def __init__(self, device: B200Device, handle: C.c_void_p, shape: Sequence[int], dtype: int):
        self.device = device
        self._h = handle
        self._shape = [int(s) for s in shape]
        self._dtype = dtype

    @classmethod
    def allocate(cls, device: B200Device, shape: Sequence[int], dtype: int = D.F32,
                 zero: bool = True) -> "B200Buffer":
        n = math.prod(shape) if len(shape) else 1
        h = C.c_void_p()
        capi.call("eb200_buffer_alloc" if zero else "eb200_buffer_alloc_uninit",
                  device._h, n * D.DTYPE_SIZE[dtype], C.byref(h))
        return cls(device, h, shape, dtype)

    def shape(self) -> List[int]:
        return list(self._shape)

    def dtype(self) -> int:
        return self._dtype

    def numel(self) -> int:
        return math.prod(self._shape) if self._shape else 1

    def byte_len(self) -> int:
        return self.numel() * D.DTYPE_SIZE[self._dtype]

    def write_from_host(self, data: bytes):
        buf = (C.c_char * len(data)).from_buffer_copy(data) if not isinstance(data, C.Array) else data
        capi.call("eb200_buffer_write", self._h, buf, len(data))

    def read_to_host(self) -> bytes:
        out = (C.c_char * self.byte_len())()
        capi.call("eb200_buffer_read", self._h, out, self.byte_len())
        return bytes(out)

    # TypedBuffer::write_vec / read_vec with numpy arrays
    def write_vec(self, a: np.ndarray):
        a = np.ascontiguousarray(a, dtype=D.DTYPE_NP[self._dtype])
        capi.call("eb200_buffer_write", self._h, a.ctypes.data_as(C.c_void_p), a.nbytes)

    def read_vec(self) -> np.ndarray:
        out = np.empty(self.numel(), dtype=D.DTYPE_NP[self._dtype])
        capi.call("eb200_buffer_read", self._h, out.ctypes.data_as(C.c_void_p), out.nbytes)
        return out

    def write_async(self, host_ptr: int, nbytes: int):
        """Copy from pinned host memory; completes at device.synchronize()."""
        capi.call("eb200_buffer_write_async", self._h, C.c_void_p(host_ptr), nbytes)

    def read_async(self, host_ptr: int, nbytes: int):
        capi.call("eb200_buffer_read_async", self._h, C.c_void_p(host_ptr), nbytes)

    def write_on(self, stream: "B200Stream", host_ptr: int, nbytes: int):
        capi.call("eb200_buffer_write_on", self._h, C.c_void_p(host_ptr), nbytes, stream._h)

    def read_on(self, stream: "B200Stream", host_ptr: int, nbytes: int):
        capi.call("eb200_buffer_read_on", self._h, C.c_void_p(host_ptr), nbytes, stream._h)

    def to_ndarray(self) -> np.ndarray:
        return self.read_vec().reshape(self._shape)

    def clone_buffer(self) -> "B200Buffer":
        h = C.c_void_p()
        capi.call("eb200_buffer_clone", self._h, C.byref(h))
        return B200Buffer(self.device, h, self._shape, self._dtype)

    def device_ptr(self) -> int:
        p = C.c_void_p()
        capi.call("eb200_buffer_device_ptr", self._h, C.byref(p))
        return p.value or 0

    def release(self):
        if self._h:
            capi.call("eb200_buffer_release", self._h)
            self._h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class KernelConfig:
    """KernelConfig (src/backend/traits.rs:486-528)."""

    def __init__(self, entry_point: str):
        self.entry_point = entry_point
        self.global_work_size = [1, 1, 1]
        self.local_work_size = None
        self.shape_vars = {}


class B200Kernel:
    def __init__(self, device: B200Device, handle: C.c_void_p, kdesc: D.KernelDesc):
        self.device = device
        self._h = handle
        self.desc = kdesc
        self._config = KernelConfig(kdesc.name)
        info = D.CKernelInfo()
        capi.call("eb200_kernel_get_info", self._h, C.byref(info))
        self.impl = info.impl.decode()
        self.launches = info.launches
        self.specialised = bool(info.specialised)
        self.scratch_bytes = info.scratch_bytes
        self.algo_bytes = info.algo_bytes
        self.algo_flops = info.algo_flops

    def config(self) -> KernelConfig:
        return self._config

    def device_kind(self) -> str:
        return "B200"

    def clone_kernel(self) -> "B200Kernel":
        return B200BackendRegistry().compile_ast(self.device, self.desc)

    def execute(self, inputs: Sequence[B200Buffer], outputs: Sequence[B200Buffer]):
        """Inputs first, then outputs, in parameter order
        (src/backend/traits.rs:545-550).  Asynchronous; a following
        ``read_to_host`` orders after it."""
        for b in list(inputs) + list(outputs):
            if not isinstance(b, B200Buffer):
                # the C backend panics on a foreign buffer (crates/backend-c/src/kernel.rs:196-210)
                raise TypeError("B200Kernel requires B200Buffer arguments")
        ins = (C.c_void_p * max(1, len(inputs)))(*[b._h for b in inputs])
        outs = (C.c_void_p * max(1, len(outputs)))(*[b._h for b in outputs])
        capi.call("eb200_kernel_launch", self._h, ins, len(inputs), outs, len(outputs))

    def execute_with_sizes(self, inputs, outputs, grid_size=None, local_size=None):
        # grid and block are chosen by the hand-written kernel, not by the caller
        self.execute(inputs, outputs)

    def release(self):
        if self._h:
            capi.call("eb200_kernel_release", self._h)
            self._h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class B200BackendRegistry:
    """BackendRegistry (src/backend/device.rs:83-171)."""

    def kind(self) -> str:
        return "B200"

    def name(self) -> str:
        return "B200 (sm_100a, hand-written kernels)"

    def is_available(self) -> bool:
        try:
            return len(self.list_devices()) > 0
        except (capi.Eb200Error, RuntimeError):
            return False

    def list_devices(self) -> List[str]:
        n = C.c_int()
        st = capi.load().eb200_device_count(C.byref(n))
        if st != capi.OK:
            return []
        return [f"b200:{i}" for i in range(n.value)]

    def supports_runtime(self) -> bool:
        return True

    def create_device(self, index: int = 0) -> B200Device:
        h = C.c_void_p()
        try:
            capi.call("eb200_device_open", index, C.byref(h))
        except capi.Eb200Error as e:
            raise DeviceError(str(e)) from e
        return B200Device(h, index)

    def allocate_buffer(self, device: B200Device, shape: Sequence[int], dtype: int = D.F32) -> B200Buffer:
        return B200Buffer.allocate(device, shape, dtype)

    def compile_ast(self, device: B200Device, program: D.KernelDesc, signature=None) -> B200Kernel:
        h = C.c_void_p()
        cdesc = program.to_c()
        capi.call("eb200_kernel_create", device._h, C.byref(cdesc), C.byref(h))
        return B200Kernel(device, h, program)

    def supports_binary_cache(self) -> bool:
        return False


class B200Comm:
    """Communicator over the GPUs of one box (``eb200_comm_*``): one process per
    GPU.  Rank 0 calls ``B200Comm.unique_id()`` and hands the 128 bytes to the
    other ranks over whatever channel the host program has; every rank then
    constructs its communicator.  The reference has nothing like it (no
    distributed code); it serves batch-sharded training and row-sharded
    reductions."""

    COMM_ID_BYTES = 128

    def __init__(self, device: B200Device, rank: int, nranks: int, unique_id: Optional[bytes] = None):
        self.device, self.rank, self.nranks = device, rank, nranks
        self._h = C.c_void_p()
        idbuf = None
        if nranks > 1:
            assert unique_id is not None and len(unique_id) == self.COMM_ID_BYTES
            idbuf = (C.c_char * self.COMM_ID_BYTES).from_buffer_copy(unique_id)
        capi.call("eb200_comm_init", device._h, rank, nranks, idbuf, C.byref(self._h))

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_char * B200Comm.COMM_ID_BYTES)()
        capi.call("eb200_comm_unique_id", buf)
        return bytes(buf)

    def info(self) -> dict:
        r, n, o = C.c_int(), C.c_int(), C.c_int()
        a, b = C.c_int64(), C.c_int64()
        capi.call("eb200_comm_info", self._h, C.byref(r), C.byref(n), C.byref(o), C.byref(a), C.byref(b))
        return {"rank": r.value, "nranks": n.value, "one_shot": bool(o.value), "calls_one_shot": a.value, "calls_nccl": b.value}

    def allreduce(self, buf: B200Buffer, op: int = D.R_SUM, offset: int = 0, count: Optional[int] = None, side_stream: bool = False):
        n = buf.numel() - offset if count is None else count
        capi.call("eb200_comm_allreduce_async" if side_stream else "eb200_comm_allreduce", self._h, buf._h, offset, n, op)

    def allreduce_sgd(self, params: B200Buffer, grads: B200Buffer, lr: float, offset: int = 0, count: Optional[int] = None,
                      side_stream: bool = False):
        """params -= lr * (sum of grads over the ranks), one kernel."""
        n = params.numel() - offset if count is None else count
        capi.call("eb200_comm_allreduce_sgd_async" if side_stream else "eb200_comm_allreduce_sgd",
                  self._h, params._h, grads._h, offset, n, lr)

    def join(self):
        """The compute stream waits for what was issued with ``side_stream=True``."""
        capi.call("eb200_comm_join", self._h)

    def attach(self, kernel: B200Kernel):
        """The reduce kernel's output becomes the all-reduce over the ranks of its local result."""
        capi.call("eb200_kernel_set_allreduce", kernel._h, self._h)

    def destroy(self):
        if self._h:
            capi.call("eb200_comm_destroy", self._h)
            self._h = None


class PinnedArray:
    """A numpy array over page-locked host memory (staging for async copies)."""

    def __init__(self, shape, dtype=np.float32):
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        self._p = C.c_void_p()
        capi.call("eb200_host_alloc", self.nbytes, C.byref(self._p))
        buf = (C.c_char * self.nbytes).from_address(self._p.value)
        self.array = np.frombuffer(buf, dtype=dtype).reshape(shape)
        self.ptr = self._p.value

    def free(self):
        if self._p:
            self.array = None
            capi.call("eb200_host_free", self._p)
            self._p = None


def launch_count() -> int:
    n = C.c_int64()
    capi.call("eb200_launch_count", C.byref(n))
    return n.value
