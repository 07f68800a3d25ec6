"""Scan (P_) kernels and the device-resident optimizer steps against the oracle:
the reference's scan loop nest (src/lowerer/loop_gen.rs:237-327) as emitted C,
and the host loops of crates/nn/src/optim/{sgd,adam}.rs as strict-IEEE C."""
import numpy as np
import pytest

from harp_b200 import desc as D
from harp_b200.backend import B200BackendRegistry
from harp_b200.desc import Ast
from oracle import c_emit as O
from util import run_gpu

pytestmark = pytest.mark.gpu
w = Ast.w


def _scan_check(dev, k, inputs, exact):
    got, kern = run_gpu(dev, k, inputs)
    ref = O.run(k, inputs)
    if exact:
        assert got.tobytes() == ref.tobytes(), kern.impl
    else:
        # every prefix is a sum of f32 terms in some order: within 1e-5 of the sum of their magnitudes
        terms = O.eval_f64(D.KernelDesc(D.K_ELEMENTWISE, k.shape, k.inputs, D.contiguous(k.shape), k.map), inputs)
        ax = k.reduce_axis
        t = np.abs(terms).reshape(k.shape)
        outer = int(np.prod(k.shape[:ax])) if ax else 1
        bound = 1e-5 * np.cumsum(t.reshape(outer, -1), axis=1).reshape(-1) + 1e-30
        assert (np.abs(got.astype(np.float64) - ref.astype(np.float64)) <= bound).all(), kern.impl
    return kern


@pytest.mark.parametrize("shape,axis", [((7, 33), 1), ((300, 1024), 1), ((4, 5000), 1), ((3, 100000), 1), ((64, 129), 1),
                                        ((5, 6, 7), 1), ((9, 4, 8), 0), ((2, 3, 4, 5), 2), ((1, 1), 1), ((513,), 0)])
def test_cumsum_and_cummax_match_the_reference_loop_nest(dev, shape, axis):
    rng = np.random.default_rng(sum(shape) + axis)
    x = rng.standard_normal(shape).astype(np.float32)
    for op, exact in ((D.R_SUM, False), (D.R_MAX, True), (D.R_MIN, True)):
        _scan_check(dev, D.scan(list(shape), [D.contiguous(list(shape))], w(0), op, axis), [x], exact)


def test_cumprod_and_fused_map(dev):
    rng = np.random.default_rng(1)
    x = rng.uniform(0.9, 1.1, (37, 260)).astype(np.float32)
    k = D.scan([37, 260], [D.contiguous([37, 260])], w(0), D.R_PROD, 1)
    got, _ = run_gpu(dev, k, [x])
    np.testing.assert_allclose(got, O.run(k, [x]), rtol=1e-4)
    # a map in front of the scan (exp of a scaled input) and a broadcast second operand
    y = rng.standard_normal(260).astype(np.float32)
    k = D.scan([37, 260], [D.contiguous([37, 260]), D.Operand([0, 1], 0, D.F32, 260)], (w(0) * w(1)).exp(), D.R_SUM, 1)
    _scan_check(dev, k, [x, y], False)


def test_scan_through_views_and_masks(dev):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((40, 24)).astype(np.float32)
    # scan along the rows of the transposed view (strided loads), output contiguous
    src = D.Operand([1, 24], 0, D.F32, 40 * 24)
    _scan_check(dev, D.scan([24, 40], [src], w(0), D.R_SUM, 1), [x], False)
    _scan_check(dev, D.scan([24, 40], [src], w(0), D.R_MAX, 1), [x], True)
    # padded view: two columns of zeros on each side
    padded = D.Operand([24, 1], -2, D.F32, 40 * 24, [D.Bound([0, 1], 0, 2, 26)])
    _scan_check(dev, D.scan([40, 28], [padded], w(0), D.R_SUM, 1), [x], False)


def test_long_rows_take_the_tiled_form(dev, registry):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 1 << 18)).astype(np.float32)
    kern = _scan_check(dev, D.scan([3, 1 << 18], [D.contiguous([3, 1 << 18])], w(0), D.R_SUM, 1), [x], False)
    assert kern.impl == "scan_tiles_v4" and kern.launches == 2
    _scan_check(dev, D.scan([3, 1 << 18], [D.contiguous([3, 1 << 18])], w(0), D.R_MAX, 1), [x], True)
    # not a multiple of the tile or of 4
    x = rng.standard_normal((2, 70001)).astype(np.float32)
    kern = _scan_check(dev, D.scan([2, 70001], [D.contiguous([2, 70001])], w(0), D.R_SUM, 1), [x], False)
    assert kern.impl == "scan_tiles_v1"


def _run_optimizer(dev, k, arrays, steps, grads):
    """Runs `steps` launches of the optimizer kernel on the GPU and on the oracle;
    arrays = [p, g, state...]; returns both sides' final arrays."""
    reg = B200BackendRegistry()
    bufs = []
    for a, o in zip(arrays, k.inputs):
        b = reg.allocate_buffer(dev, [a.size], o.dtype)
        b.write_vec(a)
        bufs.append(b)
    kern = reg.compile_ast(dev, k)
    host = [a.copy() for a in arrays]
    ok = O.OracleKernel(k)
    for s in range(steps):
        bufs[1].write_vec(grads[s])
        kern.execute(bufs, [bufs[0]])                   # in place: the output is the parameter buffer
        host[1] = grads[s].copy()
        host[0] = ok(host)
    return [b.read_vec() for b in bufs], host, kern


def test_sgd_momentum_is_bit_identical_to_the_host_loop(dev):
    n = 225034
    rng = np.random.default_rng(4)
    p, v = rng.standard_normal(n).astype(np.float32), np.zeros(n, np.float32)
    grads = [rng.standard_normal(n).astype(np.float32) for _ in range(4)]
    got, ref, kern = _run_optimizer(dev, D.sgd_momentum(n, 1e-2, 0.9), [p, grads[0], v], 4, grads)
    assert kern.impl == "sgd_momentum_update"
    assert got[0].tobytes() == ref[0].tobytes() and got[2].tobytes() == ref[2].tobytes()


def test_adam_is_bit_identical_to_the_host_loop_and_counts_steps_on_the_device(dev):
    n = 66561
    rng = np.random.default_rng(5)
    p = rng.standard_normal(n).astype(np.float32)
    m, v, t = np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(1, np.int32)
    grads = [rng.standard_normal(n).astype(np.float32) * 0.1 for _ in range(5)]
    got, ref, kern = _run_optimizer(dev, D.adam(n, 1e-3), [p, grads[0], m, v, t], 5, grads)
    assert kern.impl == "adam_update"
    assert int(got[4][0]) == 5 and int(ref[4][0]) == 5
    for i in (0, 2, 3):
        assert got[i].tobytes() == ref[i].tobytes(), i


def test_program_with_momentum_and_adam_tracks_the_oracle(dev, registry):
    from harp_b200 import workloads as W
    from harp_b200.frontend import B200Executor, Program
    from oracle.executor import OracleExecutor
    for opt, kw in (("momentum", {"momentum": 0.9}), ("adam", {})):
        runs = []
        for ex, fuse in ((B200Executor(dev, registry), "chains"), (OracleExecutor(), "reference")):
            loss, ps, grads, _ = W.mlp_graph(256, 32)
            prog = Program([loss], ex, fuse=fuse, sgd=list(zip(ps, grads)), lr=0.01, persistent=True, flat=True, optimizer=opt, **kw)
            hist = []
            for _ in range(10):
                prog.run()
                hist.append(float(prog.fetch(loss)))
            runs.append(hist)
        assert runs[0][-1] < runs[0][0]
        np.testing.assert_allclose(runs[0], runs[1], rtol=2e-3)


@pytest.mark.parametrize("n,c", [(4096, 10), (512, 10), (37, 5), (3, 1000), (1, 1), (70000, 3)])
def test_softmax_cross_entropy_forward_and_backward_in_one_kernel(dev, n, c):
    """Loss and logits gradient against the oracle's restatement of the reference's composition
    (log_softmax, multiply by the one-hot targets, sums, scale) and against float64."""
    rng = np.random.default_rng(n + c)
    x = (rng.standard_normal((n, c)) * 3).astype(np.float32)
    t = np.eye(c, dtype=np.float32)[rng.integers(0, c, n)]
    k = D.softmax_xent(n, c, -1.0 / n)
    got, kern = run_gpu(dev, k, [x, t])
    ref = O.run(k, [x, t])
    assert kern.impl == "softmax_xent_fwd_bwd" and kern.launches == 1
    x64 = x.astype(np.float64)
    z = x64 - x64.max(axis=1, keepdims=True)
    logp = z - np.log(np.exp(z).sum(axis=1, keepdims=True))
    loss64 = -(t * logp).sum() / n
    grad64 = -(t - np.exp(logp) * t.sum(axis=1, keepdims=True)) / n
    assert abs(got[0] - ref[0]) <= 1e-5 * abs(ref[0]) + 1e-7 and abs(got[0] - loss64) <= 1e-5 * abs(loss64) + 1e-7
    g, r = got[D.XENT_GRAD_OFFSET:].reshape(n, c), ref[D.XENT_GRAD_OFFSET:].reshape(n, c)
    scale = np.abs(grad64).max()
    assert np.abs(g - r).max() <= 1e-5 * scale and np.abs(g - grad64).max() <= 1e-5 * scale


@pytest.mark.parametrize("rows,cols", [(64, 64), (256, 512), (1024, 192), (8192, 8192)])
def test_sibling_fusion_reads_x_once_for_y_z_and_t(dev, rows, cols):
    """Config 2's three roots from one pass over x: y against the oracle's row sum (and float64),
    z and t bit-exact against the oracle's column max and transposing copy."""
    from harp_b200 import workloads as W
    x = W.cfg2_input(rows, cols)
    c0, c1 = W.cfg2_consts()
    k = W.cfg2_siblings(rows, cols)
    got, kern = run_gpu(dev, k, [c0, x, c1])
    assert kern.impl == "siblings_rowsum_colmax_transpose" and kern.specialised and kern.launches == 2
    pad = lambda v: (v + 63) // 64 * 64
    y, z, t = got[:rows], got[pad(rows):pad(rows) + cols], got[pad(rows) + pad(cols):]
    y_ref = O.run(W.cfg2_y(rows, cols), [c0, x, c1])
    terms = np.abs(np.exp(0.5 * x.astype(np.float64) + 1.0) * x).sum(axis=1)
    exact = (np.exp(0.5 * x.astype(np.float64) + 1.0) * x).sum(axis=1)
    assert (np.abs(y.astype(np.float64) - y_ref) <= 1e-5 * terms).all() and (np.abs(y - exact) <= 1e-5 * terms).all()
    assert z.tobytes() == O.run(W.cfg2_z(rows, cols), [x]).tobytes()
    assert t.tobytes() == np.ascontiguousarray(x.T).tobytes()
