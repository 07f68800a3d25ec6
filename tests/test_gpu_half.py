"""f16 / bf16 storage on the GPU against the oracle's `_Float16` / `__bf16` kernels.

Tolerance: one unit in the last place of the STORED type for an elementwise result (the reference's
C computes the chain in the 16-bit type's promoted arithmetic, this library in f32 with one rounding
at the store), 1e-5 of the sum of magnitudes for f32-accumulated sums; comparisons, selections,
maxima and plain casts are exact."""
import numpy as np
import pytest

from harp_b200 import desc as D
from harp_b200.desc import Ast
from oracle import c_emit as O
from test_half import as_f32, half_inputs, ulp
from util import run_gpu

pytestmark = pytest.mark.gpu
w = Ast.w


def close(got, ref, dt, what, tol_dt=None):
    g, r = as_f32(got, dt).astype(np.float64), as_f32(ref, dt).astype(np.float64)
    assert (np.abs(g - r) <= ulp(tol_dt if tol_dt is not None else dt) * np.abs(r) + 1e-30).all(), what


@pytest.mark.parametrize("shape", [(512, 1024), (37, 1023), (4, 6, 260), (2048, 4096)])
@pytest.mark.parametrize("dts", [(D.F16, D.F16, D.F16), (D.BF16, D.BF16, D.BF16), (D.BF16, D.F32, D.F16), (D.F16, D.BF16, D.F32)])
def test_elementwise_over_16_bit_storage(dev, shape, dts):
    da, db, do = dts
    a, b = half_inputs(shape, da, 1), half_inputs(shape, db, 2)
    shape = list(shape)
    for name, m in (("add", w(0) + w(1)), ("fused", (w(0) * w(1) + 0.5).maximum(w(0))), ("select", Ast.select(w(0).lt(w(1)), w(0), w(1)))):
        k = D.KernelDesc(D.K_ELEMENTWISE, shape, [D.contiguous(shape, da), D.contiguous(shape, db)], D.contiguous(shape, do), m)
        got, kern = run_gpu(dev, k, [a, b])
        assert kern.impl == ("ew_chain_v4" if int(np.prod(shape)) % 4 == 0 else "ew_chain_v1")     # contiguous operands collapse to one dim
        ref = O.run(k, [a, b])
        if name == "select" and da == db:
            assert got.tobytes() == ref.tobytes(), (name, dts)
        elif da == db or do != D.F32:
            close(got, ref, do, (name, dts))
        else:
            # one f16 and one bf16 operand: the reference's C converts both to ONE 16-bit type before it compares or
            # adds them, this library widens each exactly: up to two roundings of the coarser type apart
            if name == "select":        # defined here as: widen both exactly, then compare and pick
                af, bf = as_f32(a, da).reshape(-1), as_f32(b, db).reshape(-1)
                assert got.tobytes() == np.where(af < bf, af, bf).astype(np.float32).tobytes()
                continue
            g, r = got.astype(np.float64), ref.astype(np.float64)
            assert (np.abs(g - r) <= 2 * ulp(D.BF16) * np.abs(r) + 1e-30).all(), (name, dts)


@pytest.mark.parametrize("dt", [D.F16, D.BF16])
def test_broadcast_strided_and_masked_16_bit_operands(dev, dt):
    x, bias = half_inputs((96, 200), dt, 3), half_inputs((200,), dt, 4)
    # bias broadcast along rows, x read transposed, output f32
    k = D.KernelDesc(D.K_ELEMENTWISE, [200, 96], [D.Operand([1, 200], 0, dt, 96 * 200), D.Operand([1, 0], 0, dt, 200)],
                     D.contiguous([200, 96]), w(0) + w(1))
    got, _ = run_gpu(dev, k, [x, bias])
    ref = (as_f32(x, dt).reshape(96, 200).T + as_f32(bias, dt)[:, None]).astype(np.float32)
    assert got.tobytes() == O.run(k, [x, bias]).tobytes() == ref.reshape(-1).tobytes()     # one f32 addition of exactly widened values
    # padded view: zeros around a [96, 200] block
    src = D.Operand([200, 1], -(2 * 200 + 3), dt, 96 * 200,
                    bounds=[D.Bound([1, 0], -2, 0, 96), D.Bound([0, 1], -3, 0, 200)])
    k = D.KernelDesc(D.K_ELEMENTWISE, [100, 208], [src], D.contiguous([100, 208], dt), w(0) * 2.0)
    got, _ = run_gpu(dev, k, [x])
    assert got.tobytes() == O.run(k, [x]).tobytes()          # doubling is exact


@pytest.mark.parametrize("dt", [D.F16, D.BF16])
def test_reductions_accumulate_in_f32(dev, dt):
    x = half_inputs((300, 1000), dt, 5)
    xf = as_f32(x, dt).reshape(300, 1000).astype(np.float64)
    for axis in (0, 1):
        k = D.reduce([300, 1000], [D.contiguous([300, 1000], dt)], w(0) * w(0), D.R_SUM, axis)
        got, kern = run_gpu(dev, k, [x])
        ref = O.run(k, [x])
        bound = 1e-5 * (xf * xf).sum(axis)
        assert (np.abs(got - ref) <= bound).all() and (np.abs(got - (xf * xf).sum(axis)) <= bound).all(), kern.impl
        # max keeps the storage type and is exact
        kept = [1 if d == axis else e for d, e in enumerate([300, 1000])]
        st = D.contiguous_strides(kept)
        st[axis] = 0
        k = D.reduce([300, 1000], [D.contiguous([300, 1000], dt)], w(0), D.R_MAX, axis, out=D.Operand(st, 0, dt, 1000 if axis == 0 else 300))
        got, _ = run_gpu(dev, k, [x])
        assert (as_f32(got, dt) == as_f32(x, dt).reshape(300, 1000).max(axis)).all()


def test_cast_rounds_like_the_storage_type(dev):
    x = np.random.default_rng(6).standard_normal(4096).astype(np.float32) * 100
    for dt in (D.F16, D.BF16):
        k = D.KernelDesc(D.K_ELEMENTWISE, [4096], [D.contiguous([4096])], D.contiguous([4096]), w(0).cast(dt))
        got, _ = run_gpu(dev, k, [x])
        ref = x.astype(np.float16).astype(np.float32) if dt == D.F16 else D.bf16_value(D.bf16_bits(x))
        assert got.tobytes() == ref.tobytes()
        # and storing through a 16-bit output is the same rounding
        k = D.KernelDesc(D.K_ELEMENTWISE, [4096], [D.contiguous([4096])], D.contiguous([4096], dt), w(0) * 1.0)
        got, _ = run_gpu(dev, k, [x])
        assert as_f32(got, dt).tobytes() == ref.tobytes()


@pytest.mark.parametrize("m,n,k,batch", [(256, 256, 128, 1), (300, 200, 72, 1), (1024, 512, 4096, 1), (128, 256, 64, 4), (1, 8, 8, 1),
                                         (2048, 2048, 2048, 1)])
@pytest.mark.parametrize("dt", [D.F16, D.BF16])
def test_16_bit_contraction_on_the_tensor_cores(dev, m, n, k, batch, dt):
    """tcgen05 kind::f16: exact products of the 16-bit operands, f32 accumulation.  Against float64: within
    1e-5 of the sum of magnitudes (plus one rounding of the stored type when C is 16-bit).  The oracle's loop
    (the reference's 3-loop MatMul fallback, src/lowerer/lower.rs:834-984) rounds every product to the 16-bit
    type before adding it, so it is held to the looser 2^-9 of the same sum."""
    from test_half import half_matmul_desc
    a, b = half_inputs((batch, m, k), dt, 11), half_inputs((batch, n, k), dt, 12)
    af, bf = as_f32(a, dt).reshape(batch, m, k).astype(np.float64), as_f32(b, dt).reshape(batch, n, k).astype(np.float64)
    exact = np.einsum("bmk,bnk->bmn", af, bf).reshape(-1)
    mag = np.einsum("bmk,bnk->bmn", np.abs(af), np.abs(bf)).reshape(-1)
    for out_dt in (D.F32, dt):
        kd = half_matmul_desc(m, n, k, dt, out_dt, batch)
        got, kern = run_gpu(dev, kd, [a, b])
        if m > 1:         # (an extent-1 row dim is dropped before classification: a matrix-vector product stays a reduce)
            assert kern.impl == ("gemm_tcgen05_f16_kk" if dt == D.F16 else "gemm_tcgen05_bf16_kk"), kern.impl
        g = as_f32(got, out_dt).astype(np.float64)
        tol = 1e-5 * mag + (ulp(out_dt) * np.abs(exact) if out_dt != D.F32 else 0.0)
        assert (np.abs(g - exact) <= tol + 1e-30).all(), (out_dt, float(np.abs(g - exact).max()))
        if m * n * k * batch <= 1 << 24:
            ref = as_f32(O.run(kd, [a, b], openmp=True), out_dt).astype(np.float64)
            assert (np.abs(ref - exact) <= 2.0 ** -9 * mag + ulp(out_dt) * np.abs(exact) + 1e-30).all()
