"""Pins the CPU oracle: the reference's own known-answer vectors for this path,
replayed through the C the oracle emits, plus cross-checks of the emitted loop
nests against numpy.  Runs without a GPU."""
import numpy as np
import pytest

from harp_b200 import desc as D
from harp_b200 import workloads as W
from harp_b200.desc import Ast
from oracle import c_emit as O

w = Ast.w


def test_ref_vector_add_1d():
    # crates/backend-c/src/lib.rs:181-202  [1,2,3,4]+[5,6,7,8] = [6,8,10,12]
    k = D.elementwise([4], [D.contiguous([4])] * 2, w(0) + w(1))
    out = O.run(k, [np.array([1, 2, 3, 4.]), np.array([5, 6, 7, 8.])])
    assert out.tolist() == [6.0, 8.0, 10.0, 12.0]


def test_ref_vector_mul_1d():
    # crates/backend-c/src/lib.rs:204-224  [1,2,3,4]*[2,3,4,5] = [2,6,12,20]
    k = D.elementwise([4], [D.contiguous([4])] * 2, w(0) * w(1))
    out = O.run(k, [np.array([1, 2, 3, 4.]), np.array([2, 3, 4, 5.])])
    assert out.tolist() == [2.0, 6.0, 12.0, 20.0]


def test_ref_vector_add_2d_sevens():
    # crates/backend-c/src/lib.rs:226-245  2x3: [1..6] + [6..1] = six 7.0s
    k = D.elementwise([2, 3], [D.contiguous([2, 3])] * 2, w(0) + w(1))
    out = O.run(k, [np.arange(1, 7.), np.arange(6, 0, -1.)])
    assert out.tolist() == [7.0] * 6


def test_ref_vector_openmp_10000():
    # crates/backend-openmp/src/lib.rs:207-231  i + (10000-i) = 10000
    k = D.elementwise([10000], [D.contiguous([10000])] * 2, w(0) + w(1))
    i = np.arange(10000, dtype=np.float32)
    out = O.run(k, [i, 10000 - i], openmp=True)
    assert (out == 10000.0).all()


def unfold_2x2_s2_descs():
    """unfold(2x2, stride 2) of a 4x4 tensor and the fold (scatter) back:
    window gather C_ kernel (src/lowerer/lower.rs:355-359) and S_ kernel."""
    # output [oh, ow, kh, kw] = in[(oh*2+kh)*4 + ow*2+kw]
    src = D.Operand([8, 2, 4, 1], 0, D.F32, 16)
    unfold = D.copy([2, 2, 2, 2], src)
    fold = D.KernelDesc(D.K_SCATTER, [2, 2, 2, 2], [D.contiguous([2, 2, 2, 2])],
                        D.Operand([8, 2, 4, 1], 0, D.F32, 16))
    return unfold, fold


def test_ref_vector_unfold_fold_preserves_sum():
    # crates/backend-c/src/lib.rs:298-339: unfold(2x2,s2) -> fold keeps sum of 0..15
    unfold, fold = unfold_2x2_s2_descs()
    x = np.arange(16, dtype=np.float32)
    u = O.run(unfold, [x])
    assert u.reshape(2, 2, 2, 2)[1, 0].tolist() == [[8.0, 9.0], [12.0, 13.0]]
    f = O.run(fold, [u])
    assert f.sum() == x.sum() == 120.0
    assert (f == x).all()   # non-overlapping windows: fold inverts unfold


def test_emitted_text_matches_renderer_conventions():
    k = W.cfg2_y(4, 8)
    src = O.emit_kernel_c(k)
    assert "for (long long ridx0 = 0; ridx0 < 4; ridx0 += 1) {" in src
    assert "float acc;" in src and "acc = 0.0f;" in src
    assert "exp2f(" in src and "1.442695f" in src
    assert src.startswith("/* Generated C code by Harp */")
    assert "void kernel(float* buf0, float* buf1, float* buf2, float* out)" in src
    z = O.emit_kernel_c(W.cfg2_z(4, 8))
    assert "acc = (-INFINITY);" in z and "fmaxf(acc, " in z
    # reduce over axis 0: kept axis outside, reduce loop innermost
    assert z.index("ridx1 < 8") < z.index("ridx0 < 4")
    omp = O.emit_kernel_c(k, openmp=True)
    assert "#pragma omp parallel for" in omp and "#include <omp.h>" in omp


def test_f32_literals():
    assert O.f32_literal(1.0) == "1.0f"
    assert O.f32_literal(-1.0) == "-1.0f"
    assert O.f32_literal(0.5) == "0.5f"
    assert O.f32_literal(D.LOG2_E) == "1.442695f"
    assert O.f32_literal(float("-inf")) == "(-INFINITY)"
    assert O.f32_literal(1e-7) == "0.0000001f"


@pytest.mark.parametrize("openmp", [False, True])
def test_cfg2_small_against_numpy(openmp):
    x = W.cfg2_input(37, 64)
    c0, c1 = W.cfg2_consts()
    y = O.run(W.cfg2_y(37, 64), [c0, x, c1], openmp=openmp)
    np.testing.assert_allclose(y, (np.exp(0.5 * x.astype(np.float64) + 1) * x).sum(1), rtol=2e-5, atol=1e-4)
    z = O.run(W.cfg2_z(37, 64), [x], openmp=openmp)
    assert (z == x.max(0)).all()
    t = O.run(W.cfg2_t(37, 64), [x], openmp=openmp)
    assert (t.reshape(64, 37) == x.T).all()


def test_matmul_forms_against_numpy():
    a, b = W.uniform_pm1((17, 9), 0), W.uniform_pm1((9, 13), 1)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    for fma in (False, True):
        c = O.run(W.matmul_desc(17, 9, 13), [a, b], fma=fma)
        np.testing.assert_allclose(c.reshape(17, 13), ref, rtol=1e-5, atol=1e-5)
    x, wt = W.uniform_pm1((5, 9), 2), W.uniform_pm1((7, 9), 3)
    c = O.run(W.linear_desc(5, 9, 7), [x, wt])
    np.testing.assert_allclose(c.reshape(5, 7), x.astype(np.float64) @ wt.T.astype(np.float64), rtol=1e-5, atol=1e-5)


def test_padded_load_select():
    # 1-D pad by (1, 2): out[i] = (1 <= i < 5) ? x[i-1] : 0
    op = D.Operand([1], -1, D.F32, 4, [D.Bound([1], 0, 1, 5)], 0.0)
    k = D.elementwise([7], [op], w(0))
    out = O.run(k, [np.array([1, 2, 3, 4.])])
    assert out.tolist() == [0, 1, 2, 3, 4, 0, 0]
    assert "?" in O.emit_kernel_c(k)


def test_eval_f64_agrees_with_compiled_c():
    x = W.cfg2_input(16, 32)
    c0, c1 = W.cfg2_consts()
    k = W.cfg2_y(16, 32)
    np.testing.assert_allclose(O.run(k, [c0, x, c1]), O.eval_f64(k, [c0, x, c1]), rtol=1e-5, atol=1e-5)
