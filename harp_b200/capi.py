"""ctypes binding of ``libeb200.so`` (the C ABI in ``include/eb200.h``).

This is the same FFI surface the Rust backend crate binds; Python uses it for
the tests, the benchmark and the host-side mirror in ``harp_b200.backend``.
Loading fails loudly when the library has not been built: there is no other
execution path.
"""
from __future__ import annotations

import ctypes as C
import os

from . import desc as D

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libeb200.so")

# eb200_status
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_OOM, ERR_BOUNDS, ERR_COMM, ERR_TIMEOUT, ERR_NO_DEVICE = range(9)
STATUS_NAME = {
    OK: "OK", ERR_INVALID: "INVALID", ERR_UNSUPPORTED: "UNSUPPORTED", ERR_CUDA: "CUDA",
    ERR_OOM: "OOM", ERR_BOUNDS: "BOUNDS", ERR_COMM: "COMM", ERR_TIMEOUT: "TIMEOUT",
    ERR_NO_DEVICE: "NO_DEVICE",
}


class Eb200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"eb200 error {STATUS_NAME.get(status, status)}: {message}")
        self.status = status
        self.message = message


_p = C.c_void_p
_pp = C.POINTER(C.c_void_p)

# name -> argtypes; every function returns int (status) unless noted
SIGNATURES = {
    "eb200_device_count": [C.POINTER(C.c_int)],
    "eb200_device_open": [C.c_int, _pp],
    "eb200_device_close": [_p],
    "eb200_device_sync": [_p],
    "eb200_device_get_props": [_p, C.POINTER(D.CDeviceProps)],
    "eb200_device_stream": [_p, _pp],
    "eb200_timer_begin": [_p],
    "eb200_timer_end": [_p, C.POINTER(C.c_float)],
    "eb200_event_create": [_p, _pp],
    "eb200_event_record": [_p],
    "eb200_event_elapsed_ms": [_p, _p, C.POINTER(C.c_float)],
    "eb200_event_destroy": [_p],
    "eb200_stream_create": [_p, _pp],
    "eb200_stream_destroy": [_p],
    "eb200_stream_sync": [_p],
    "eb200_stream_wait": [_p, _p, _p],
    "eb200_event_record_on": [_p, _p],
    "eb200_buffer_write_on": [_p, _p, C.c_size_t, _p],
    "eb200_buffer_read_on": [_p, _p, C.c_size_t, _p],
    "eb200_graph_begin": [_p],
    "eb200_graph_end": [_p, _pp],
    "eb200_graph_launch": [_p],
    "eb200_graph_release": [_p],
    "eb200_device_mem_stats": [_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)],
    "eb200_buffer_alloc": [_p, C.c_size_t, _pp],
    "eb200_buffer_alloc_uninit": [_p, C.c_size_t, _pp],
    "eb200_buffer_retain": [_p],
    "eb200_buffer_release": [_p],
    "eb200_buffer_bytes": [_p, C.POINTER(C.c_size_t)],
    "eb200_buffer_write": [_p, _p, C.c_size_t],
    "eb200_buffer_read": [_p, _p, C.c_size_t],
    "eb200_buffer_write_async": [_p, _p, C.c_size_t],
    "eb200_buffer_read_async": [_p, _p, C.c_size_t],
    "eb200_buffer_clone": [_p, _pp],
    "eb200_buffer_device_ptr": [_p, _pp],
    "eb200_host_alloc": [C.c_size_t, _pp],
    "eb200_host_free": [_p],
    "eb200_kernel_create": [_p, C.POINTER(D.CKernelDesc), _pp],
    "eb200_kernel_get_info": [_p, C.POINTER(D.CKernelInfo)],
    "eb200_kernel_query": [C.POINTER(D.CKernelDesc), C.c_int, C.POINTER(D.CKernelInfo)],
    "eb200_abi_sizes": [C.POINTER(C.c_size_t)] * 4,
    "eb200_kernel_launch": [_p, _pp, C.c_int, _pp, C.c_int],
    "eb200_kernel_release": [_p],
    "eb200_reduce_cols_static": [_p, C.c_int64, C.c_int64, C.c_int, _p, _p],
    "eb200_launch_count": [C.POINTER(C.c_int64)],
    "eb200_comm_unique_id": [_p],
    "eb200_comm_init": [_p, C.c_int, C.c_int, _p, _pp],
    "eb200_comm_info": [_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int64), C.POINTER(C.c_int64)],
    "eb200_comm_allreduce": [_p, _p, C.c_int64, C.c_int64, C.c_int],
    "eb200_comm_allreduce_async": [_p, _p, C.c_int64, C.c_int64, C.c_int],
    "eb200_comm_join": [_p],
    "eb200_comm_allreduce_sgd": [_p, _p, _p, C.c_int64, C.c_int64, C.c_float],
    "eb200_comm_allreduce_sgd_async": [_p, _p, _p, C.c_int64, C.c_int64, C.c_float],
    "eb200_kernel_set_allreduce": [_p, _p],
    "eb200_comm_destroy": [_p],
}

_lib = None


def load() -> C.CDLL:
    """Load the library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m harp_b200._build`. "
            "harp_b200 has no CPU execution path.")
    lib = C.CDLL(LIB_PATH)
    lib.eb200_abi_version.restype = C.c_int
    lib.eb200_abi_version.argtypes = []
    lib.eb200_last_error.restype = C.c_char_p
    lib.eb200_last_error.argtypes = []
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int):
    if status != OK:
        raise Eb200Error(status, load().eb200_last_error().decode(errors="replace"))


def call(name: str, *args):
    check(getattr(load(), name)(*args))
