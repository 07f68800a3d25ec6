"""eb200_reduce_cols_static: the column reduce for callers that may not allocate.

Some users of this library hold device memory but cannot ask for more: a serving
loop that must never hit the device-wide synchronisation inside cudaMalloc, or a
host application whose own arena already owns the GPU's memory.  For them the
library keeps the reduce's partial-result scratch in a fixed array of its own.
This test drives that entry point through the C ABI with raw device pointers and
checks it against the regular kernel path (eb200_kernel_create/launch) on two
calls in a row, so stale partials from the first call would show in the second.
"""
import ctypes as C

import numpy as np
import pytest

from harp_b200 import capi
from harp_b200 import desc as D
from harp_b200 import workloads as W

pytestmark = pytest.mark.gpu


def regular_path(registry, dev, x, op):
    rows, cols = x.shape
    k = D.reduce([rows, cols], [D.contiguous([rows, cols])], D.Ast.w(0), op, 0)
    bx = registry.allocate_buffer(dev, [rows, cols]); bx.write_vec(x)
    bo = registry.allocate_buffer(dev, [cols])
    kern = registry.compile_ast(dev, k)
    kern.execute([bx], [bo])
    return bo.read_vec(), bx


def static_path(dev, bx, rows, cols, op, registry):
    bo = registry.allocate_buffer(dev, [cols])          # the caller's own memory
    before = dev.mem_stats()["n_allocs"]
    capi.call("eb200_reduce_cols_static", C.c_void_p(bx.device_ptr()), rows, cols, op,
              C.c_void_p(bo.device_ptr()), C.c_void_p(dev.stream()))
    assert dev.mem_stats()["n_allocs"] == before          # the call took nothing from the pool
    return bo.read_vec()


# besides a regular shape: a ragged one (cols not a multiple of 4: scalar path), one column of many
# rows (every split holds one partial), and one row (nothing to reduce; the copy must still be exact)
@pytest.mark.parametrize("rows,cols", [(4096, 512), (777, 130), (200000, 1), (1, 4096), (5000, 130)])
def test_static_scratch_reduce_matches_regular_path_twice(dev, registry, rows, cols):
    rng = np.random.default_rng(99)
    for call in range(2):                                 # two calls in a row share the scratch
        x = rng.standard_normal((rows, cols)).astype(np.float32) * (call + 1)
        ref_max, bx = regular_path(registry, dev, x, D.R_MAX)
        got_max = static_path(dev, bx, rows, cols, D.R_MAX, registry)
        assert (got_max == ref_max).all() and (got_max == x.max(axis=0)).all()
        ref_sum, _ = regular_path(registry, dev, x, D.R_SUM)
        got_sum = static_path(dev, bx, rows, cols, D.R_SUM, registry)
        tol = 1e-5 * np.abs(x.astype(np.float64)).sum(axis=0)
        assert (np.abs(got_sum.astype(np.float64) - ref_sum) <= tol).all()


def test_static_scratch_limit_is_a_clear_error(dev, registry):
    # 296 row-splits x 2048 columns of partials exceed the 2 MiB the library carries;
    # the call must refuse before launching anything (the buffers here are tiny)
    rows, cols = 8192, 2048
    bx = registry.allocate_buffer(dev, [8])
    bo = registry.allocate_buffer(dev, [8])
    with pytest.raises(capi.Eb200Error) as e:
        capi.call("eb200_reduce_cols_static", C.c_void_p(bx.device_ptr()), rows, cols, D.R_SUM,
                  C.c_void_p(bo.device_ptr()), C.c_void_p(dev.stream()))
    assert e.value.status == capi.ERR_UNSUPPORTED and "scratch" in e.value.message
