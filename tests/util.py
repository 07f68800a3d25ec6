"""Shared helpers for the parity tests: run a KernelDesc on the GPU through the
backend mirror, run it on the CPU oracle, compare."""
import numpy as np

from harp_b200 import desc as D
from harp_b200.backend import B200BackendRegistry, B200Buffer


def run_gpu(dev, k: D.KernelDesc, inputs, out_init=None):
    reg = B200BackendRegistry()
    bufs = []
    for a, o in zip(inputs, k.inputs):
        a = np.ascontiguousarray(a, dtype=D.DTYPE_NP[o.dtype]).reshape(-1)
        assert a.size == o.numel, (a.size, o.numel)
        b = reg.allocate_buffer(dev, [a.size], o.dtype)
        b.write_vec(a)
        bufs.append(b)
    out = reg.allocate_buffer(dev, [int(k.output.numel)], k.output.dtype)
    if out_init is not None:
        out.write_vec(out_init)
    kern = reg.compile_ast(dev, k)
    kern.execute(bufs, [out])
    res = out.read_vec()
    return res, kern


def sum_tolerance(k: D.KernelDesc, inputs, rel=1e-5):
    """Cancellation-safe bound for sums: |gpu - cpu| <= rel * sum|terms| per
    output (any summation order of f32 terms stays within it), else rel*|cpu|."""
    from oracle import c_emit as O
    absk = D.KernelDesc(k.kclass, k.shape, k.inputs, k.output, k.map, k.reduce_op, k.reduce_axis)
    terms = O.eval_f64(D.KernelDesc(D.K_ELEMENTWISE, k.shape, k.inputs, D.contiguous(k.shape), k.map), inputs)
    terms = np.abs(terms).reshape(k.shape)
    return rel * terms.sum(axis=k.reduce_axis).reshape(-1)


def assert_close(got, ref, rel=1e-5, abs_tol=None, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    tol = rel * np.abs(ref)
    if abs_tol is not None:
        tol = np.maximum(tol, abs_tol)
    tol = np.maximum(tol, 1e-30)
    bad = np.abs(got - ref) > tol
    both_nan = np.isnan(got) & np.isnan(ref)
    bad &= ~both_nan
    same_inf = np.isinf(ref) & (got == ref)
    bad &= ~same_inf
    if bad.any():
        i = int(np.argmax(bad))
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} differ; first at {i}: got {got.reshape(-1)[i]!r} ref {ref.reshape(-1)[i]!r}")
