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
