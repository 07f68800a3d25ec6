"""Seeded differential sweep: random loop nests (shapes with size-1 axes, odd
extents, permuted and broadcast operands, offsets, padded views, random maps
and reduce axes) on the GPU against the emitted-C oracle."""
import numpy as np
import pytest

from harp_b200 import desc as D
from harp_b200.desc import Ast
from oracle import c_emit as O

from util import run_gpu

pytestmark = pytest.mark.gpu
w = Ast.w


def random_view(rng, shape):
    """A random operand over `shape`: permuted storage, some broadcast axes, an offset."""
    nd = len(shape)
    bcast = [rng.random() < 0.25 for _ in range(nd)]
    store_shape = [1 if b else s for b, s in zip(bcast, shape)]
    perm = list(rng.permutation(nd))
    phys = [store_shape[p] for p in perm]                      # storage order
    pst = D.contiguous_strides(phys)
    strides = [0] * nd
    for pos, p in enumerate(perm):
        strides[p] = 0 if bcast[p] or shape[p] == 1 else pst[pos]
    off = int(rng.integers(0, 5))
    numel = int(np.prod(phys)) + off
    return D.Operand(strides, off, D.F32, numel)


def random_expr(rng, nin, depth=0):
    r = rng.random()
    if depth > 3 or r < 0.25:
        return w(int(rng.integers(0, nin))) if rng.random() < 0.8 else Ast.const(float(rng.uniform(-2, 2)))
    a = random_expr(rng, nin, depth + 1)
    b = random_expr(rng, nin, depth + 1)
    pick = rng.integers(0, 9)
    if pick == 0: return a + b
    if pick == 1: return a * b
    if pick == 2: return a.maximum(b)
    if pick == 3: return a - b
    if pick == 4: return Ast.select(a.lt(b), a, b)
    if pick == 5: return (a * Ast.const(0.25)).exp()
    if pick == 6: return (a * a + Ast.const(1.0)).sqrt()
    if pick == 7: return (a * a + Ast.const(0.5)).recip()
    return (a * Ast.const(0.5)).sin()


def case(seed):
    rng = np.random.default_rng(seed)
    nd = int(rng.integers(1, 5))
    shape = [int(rng.choice([1, 2, 3, 4, 5, 7, 8, 12, 16, 33, 64])) for _ in range(nd)]
    nin = int(rng.integers(1, 4))
    ops = [random_view(rng, shape) for _ in range(nin)]
    expr = random_expr(rng, nin)
    used = expr.wildcards()
    if not used:
        expr = expr + w(0)
    data = [rng.uniform(-1.5, 1.5, o.numel).astype(np.float32) for o in ops]
    if rng.random() < 0.5:
        return D.elementwise(shape, ops, expr), data
    op = int(rng.choice([D.R_SUM, D.R_MAX, D.R_MIN]))
    return D.reduce(shape, ops, expr, op, int(rng.integers(0, nd))), data


@pytest.mark.parametrize("seed", range(80))
def test_random_loop_nest_matches_oracle(dev, seed):
    k, data = case(seed)
    got, kern = run_gpu(dev, k, data)
    ref = O.run(k, data)
    if k.kclass == D.K_REDUCE and k.reduce_op == D.R_SUM:
        terms = np.abs(O.eval_f64(D.KernelDesc(D.K_ELEMENTWISE, k.shape, k.inputs, D.contiguous(k.shape), k.map), data))
        tol = 1e-5 * terms.reshape(k.shape).sum(axis=k.reduce_axis).reshape(-1) + 1e-6
        assert (np.abs(got.astype(np.float64) - ref) <= tol).all(), (seed, kern.impl)
    else:
        tol = 1e-5 * np.abs(ref) + 2e-6
        assert (np.abs(got.astype(np.float64) - ref) <= tol).all(), (seed, kern.impl, k.map.key())


@pytest.mark.parametrize("seed", range(12))
def test_random_padded_gather_is_bit_exact(dev, seed):
    rng = np.random.default_rng(1000 + seed)
    h, wd = int(rng.integers(3, 20)), int(rng.integers(3, 20))
    pt, pb, pl, pr = (int(v) for v in rng.integers(0, 4, 4))
    x = rng.standard_normal((h, wd)).astype(np.float32)
    op = D.Operand([wd, 1], -pt * wd - pl, D.F32, x.size,
                   [D.Bound([1, 0], 0, pt, pt + h), D.Bound([0, 1], 0, pl, pl + wd)], float(rng.integers(-2, 3)))
    k = D.copy([h + pt + pb, wd + pl + pr], op)
    got, _ = run_gpu(dev, k, [x])
    assert got.tobytes() == O.run(k, [x]).tobytes()


# ---- convolutions: forward, input gradient, weight gradient, every kernel form -----------------------

def conv_case(seed):
    rng = np.random.default_rng(1000 + seed)
    k = int(rng.choice([1, 2, 3, 3, 3, 5]))
    pad = int(rng.integers(0, k))                      # 0 .. k-1
    c = int(rng.choice([1, 2, 3, 8, 16, 32, 64]))
    co = int(rng.choice([4, 8, 12, 20, 32, 64, 96, 132]))
    top = 15 if seed % 3 else 41          # every third layer is large enough to leave the whole-image staging path
    h = int(rng.integers(max(k - 2 * pad, 1), top)) + (2 if k == 5 else 0)
    wd = int(rng.integers(max(k - 2 * pad, 1), top)) + (2 if k == 5 else 0)
    n = int(rng.integers(1, 6))
    while c * k * k > 2048:
        c //= 2
    return n, c, h, wd, co, k, pad


@pytest.mark.parametrize("seed", range(int(__import__("os").environ.get("EB200_TEST_CONV_SEEDS", "24"))))
def test_random_convolutions_all_forms(dev, seed):
    """Seeded random layers through whichever kernel the library picks (tensor cores with
    TMA / bulk / cp.async patch staging or direct gathers, channel-blocked or table k order,
    the streaming f32 kernels for tiny reductions): forward with bias and ReLU in both
    output layouts, the input gradient, the weight gradient where a one-kernel form is
    served.  Reference: the oracle's loop nests; bound 1e-5 * sum |terms| (3xTF32 / f32)."""
    n, c, h, wd, co, k, pad = conv_case(seed)
    ho, wo = h + 2 * pad - k + 1, wd + 2 * pad - k + 1
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, (n, c, h, wd)).astype(np.float32)
    w_ = rng.uniform(-1, 1, (co, c, k, k)).astype(np.float32)
    b = rng.uniform(-1, 1, co).astype(np.float32)
    g = rng.uniform(-1, 1, (n, co, ho, wo)).astype(np.float32)
    bound = 1e-5 * (c * k * k + 1)                       # |x|, |w|, |b| <= 1: sum |terms| <= K + 1
    for nchw in (False, True):
        kd = D.conv2d(n, c, h, wd, co, k, k, pad=pad, relu=True, nchw=nchw)
        got, kern = run_gpu(dev, kd, [x, w_, b])
        assert kern.impl.startswith("conv2d_"), kern.impl
        assert np.abs(got - O.run(kd, [x, w_, b])).max() <= bound, (kern.impl, n, c, h, wd, co, k, pad)
    # input gradient: the same class over flipped weights (pad' = k-1-pad >= 0 by construction)
    from harp_b200 import capi
    kd = D.conv2d(n, co, ho, wo, c, k, k, pad=k - 1 - pad, bias=False, flip=True, nchw=True)
    if co % 32 == 0 or co * k * k <= 2048:               # else the per-k table would not fit: composed form instead
        got, kern = run_gpu(dev, kd, [g, w_])
        assert kern.impl.endswith("_dgrad"), kern.impl
        assert np.abs(got - O.run(kd, [g, w_])).max() <= 1e-5 * (co * k * k + 1), kern.impl
    else:
        with pytest.raises(capi.Eb200Error) as e:
            run_gpu(dev, kd, [g, w_])
        assert e.value.status == capi.ERR_UNSUPPORTED
    # weight gradient: rows layout always, planes layout for tiny reductions
    grows = np.ascontiguousarray(g.transpose(0, 2, 3, 1)).reshape(n * ho * wo, co)
    for g_nchw, gin in ((False, grows), (True, g)):
        kd = D.conv2d_wgrad(n, c, h, wd, co, k, k, pad=pad, g_nchw=g_nchw)
        try:
            got, kern = run_gpu(dev, kd, [x, gin])
        except capi.Eb200Error as e:                     # planes too large for shared memory, Co % 4 != 0, ...: composed form instead
            assert e.status == capi.ERR_UNSUPPORTED
            continue
        assert kern.impl.endswith("_wgrad"), kern.impl
        assert np.abs(got - O.run(kd, [x, gin])).max() <= 1e-5 * (n * ho * wo + 1), kern.impl
    dev.synchronize()
