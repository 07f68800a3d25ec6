"""Parity of the CUDA kernels with the CPU oracle, through the C ABI.

Bit-exact for copies/permutes/gathers and exact ops (add, mul, max, compare);
1e-5 relative for f32 maps with transcendentals; sums are compared with the
cancellation-safe bound |gpu - cpu| <= 1e-5 * sum|terms| (any order of adding the
same f32 terms stays inside it) and against a float64 evaluation.
"""
import numpy as np
import pytest

from harp_b200 import capi
from harp_b200 import desc as D
from harp_b200 import workloads as W
from harp_b200.chains import CHAINS
from harp_b200.desc import Ast
from oracle import c_emit as O

from util import assert_close, run_gpu, sum_tolerance

pytestmark = pytest.mark.gpu
w = Ast.w


def rnd(shape, seed, lo=-1.0, hi=1.0):
    return np.random.default_rng(seed).uniform(lo, hi, shape).astype(np.float32)


# ---- the reference's own known-answer vectors, through the GPU path ------------------

def test_ref_vectors_add_mul(dev):
    k = D.elementwise([4], [D.contiguous([4])] * 2, w(0) + w(1))
    out, kern = run_gpu(dev, k, [np.array([1, 2, 3, 4.]), np.array([5, 6, 7, 8.])])
    assert out.tolist() == [6.0, 8.0, 10.0, 12.0]
    k = D.elementwise([4], [D.contiguous([4])] * 2, w(0) * w(1))
    out, _ = run_gpu(dev, k, [np.array([1, 2, 3, 4.]), np.array([2, 3, 4, 5.])])
    assert out.tolist() == [2.0, 6.0, 12.0, 20.0]
    k = D.elementwise([2, 3], [D.contiguous([2, 3])] * 2, w(0) + w(1))
    out, _ = run_gpu(dev, k, [np.arange(1, 7.), np.arange(6, 0, -1.)])
    assert out.tolist() == [7.0] * 6
    k = D.elementwise([10000], [D.contiguous([10000])] * 2, w(0) + w(1))
    i = np.arange(10000, dtype=np.float32)
    out, _ = run_gpu(dev, k, [i, 10000 - i])
    assert (out == 10000.0).all()


def test_ref_vector_unfold_fold(dev):
    src = D.Operand([8, 2, 4, 1], 0, D.F32, 16)
    unfold = D.copy([2, 2, 2, 2], src)
    fold = D.KernelDesc(D.K_SCATTER, [2, 2, 2, 2], [D.contiguous([2, 2, 2, 2])],
                        D.Operand([8, 2, 4, 1], 0, D.F32, 16))
    x = np.arange(16, dtype=np.float32)
    u, _ = run_gpu(dev, unfold, [x])
    assert (u == O.run(unfold, [x])).all()
    f, _ = run_gpu(dev, fold, [u], out_init=np.full(16, 7.0, np.float32))  # scatter zero-fills first
    assert f.sum() == 120.0 and (f == x).all()


# ---- buffers ----------------------------------------------------------------------------

def test_buffer_semantics(dev, registry):
    b = registry.allocate_buffer(dev, [5, 3])
    assert b.shape() == [5, 3] and b.byte_len() == 60
    assert (b.read_vec() == 0).all()                      # zero-initialised like CBuffer
    with pytest.raises(capi.Eb200Error) as e:             # size mismatch is an error
        b.write_from_host(b"\0" * 59)
    assert e.value.status == capi.ERR_INVALID and "mismatch" in e.value.message
    data = np.arange(15, dtype=np.float32)
    b.write_vec(data)
    assert b.read_to_host() == data.tobytes()
    c = b.clone_buffer()                                   # value copy (copy-on-write)
    b.write_vec(data * 2)
    assert (c.read_vec() == data).all() and (b.read_vec() == data * 2).all()
    # a kernel writing into a clone must not disturb the original
    d = b.clone_buffer()
    k = registry.compile_ast(dev, D.elementwise([15], [D.contiguous([15])], w(0) * Ast.const(3.0)))
    k.execute([c], [d])
    assert (d.read_vec() == data * 3).all() and (b.read_vec() == data * 2).all()
    with pytest.raises(TypeError):
        k.execute([np.zeros(15)], [d])
    st = dev.mem_stats()
    assert st["in_use"] > 0 and st["peak"] >= st["in_use"]


def test_side_stream_copies_ordered_by_events(dev, registry):
    """Upload on one side stream, kernel on the compute stream, download on
    another side stream, ordered only by events; two rounds reuse the buffers."""
    from harp_b200.backend import PinnedArray
    n = 1 << 20
    src, dst = PinnedArray((n,)), PinnedArray((n,))
    a, o = registry.allocate_buffer(dev, [n]), registry.allocate_buffer(dev, [n])
    k = registry.compile_ast(dev, D.elementwise([n], [D.contiguous([n])], w(0) * Ast.const(2.0)))
    up, down = dev.copy_stream(), dev.copy_stream()
    e_up, e_k, e_down = dev.event(), dev.event(), dev.event()
    for rnd_ in range(2):
        src.array[...] = np.arange(n, dtype=np.float32) + rnd_
        if rnd_:
            dev.wait_event(e_k, up)            # the kernel that read `a` is done
        a.write_on(up, src.ptr, src.nbytes); e_up.record(up)
        dev.wait_event(e_up)
        if rnd_:
            dev.wait_event(e_down)             # the previous download of `o` is done
        k.execute([a], [o]); e_k.record()
        dev.wait_event(e_k, down)
        o.read_on(down, dst.ptr, dst.nbytes); e_down.record(down)
        down.synchronize()
        assert (dst.array == 2 * (np.arange(n, dtype=np.float32) + rnd_)).all()
    src.free(); dst.free()


def test_launch_rejects_short_buffers(dev, registry):
    k = registry.compile_ast(dev, D.elementwise([16], [D.contiguous([16])], w(0)))
    a = registry.allocate_buffer(dev, [8])
    o = registry.allocate_buffer(dev, [16])
    with pytest.raises(capi.Eb200Error) as e:
        k.execute([a], [o])
    assert e.value.status == capi.ERR_BOUNDS


# ---- elementwise -------------------------------------------------------------------------

@pytest.mark.parametrize("name,expr", CHAINS, ids=[n for n, _ in CHAINS])
def test_every_compiled_chain_matches_oracle(dev, name, expr):
    nin = max(expr.wildcards()) + 1 if expr.wildcards() else 1
    shape = [37, 20]
    positive = any(t in expr.key() for t in ("log2", "sqrt", "recip"))
    ins = [rnd(shape, 100 + i, 0.5 if positive else -2.0, 2.0) for i in range(nin)]
    k = D.elementwise(shape, [D.contiguous(shape)] * nin, expr)
    got, kern = run_gpu(dev, k, ins)
    assert kern.specialised, name
    ref = O.run(k, ins)
    assert_close(got, ref, rel=1e-5, abs_tol=2e-6, what=name)


def test_interpreter_matches_oracle_and_compiled(dev):
    shape = [33, 7]
    a, b = rnd(shape, 1, 0.1, 3.0), rnd(shape, 2, 0.1, 3.0)
    e = Ast.select((w(0).sin() * w(1).sqrt() + w(0)).floor().lt(w(1)), w(0).log2(), w(1).exp2().recip())
    k = D.elementwise(shape, [D.contiguous(shape)] * 2, e)
    got, kern = run_gpu(dev, k, [a, b])
    assert not kern.specialised
    assert_close(got, O.run(k, [a, b]), rel=1e-5, abs_tol=2e-6)
    # a chain that has a compiled functor, forced through the interpreter by
    # adding a no-op: both evaluators must agree
    chain = ((w(0) * Ast.const(0.5)) + Ast.const(1.0)).exp() * w(0)
    slow = chain + Ast.const(0.0) * w(0)
    k1 = D.elementwise(shape, [D.contiguous(shape)], chain)
    k2 = D.elementwise(shape, [D.contiguous(shape)], slow)
    g1, kn1 = run_gpu(dev, k1, [a])
    g2, kn2 = run_gpu(dev, k2, [a])
    assert kn1.specialised and not kn2.specialised
    assert_close(g2, g1, rel=1e-6)


@pytest.mark.parametrize("shape", [[1], [3], [4], [5, 1, 7], [128, 32], [2, 3, 4, 5, 6], [1, 1, 1024], [257, 129]])
def test_elementwise_shapes_and_broadcasts(dev, shape):
    nd = len(shape)
    a = rnd(shape, 3)
    # operand 1 broadcasts along every other axis (stride 0), like an expanded bias
    bshape = [s if d % 2 == nd % 2 else 1 for d, s in enumerate(shape)]
    b = rnd(bshape, 4)
    bst = [st if bshape[d] != 1 else 0 for d, st in enumerate(D.contiguous_strides(bshape))]
    opb = D.Operand(bst, 0, D.F32, b.size)
    k = D.elementwise(shape, [D.contiguous(shape), opb], (w(0) + w(1)).maximum(Ast.const(0.0)))
    got, _ = run_gpu(dev, k, [a, b])
    assert (got == O.run(k, [a, b])).all()     # add + max are exact


def test_bool_output_and_input(dev):
    shape = [19, 5]
    a, b = rnd(shape, 5), rnd(shape, 6)
    k = D.elementwise(shape, [D.contiguous(shape)] * 2, w(0).lt(w(1)), out_dtype=D.BOOL)
    mask, _ = run_gpu(dev, k, [a, b])
    assert mask.dtype == np.uint8 and (mask == (a < b).reshape(-1)).all()
    k2 = D.elementwise(shape, [D.contiguous(shape, D.BOOL), D.contiguous(shape), D.contiguous(shape)],
                       Ast.select(w(0), w(1), w(2)))
    got, _ = run_gpu(dev, k2, [mask, a, b])
    assert (got == np.where(a < b, a, b).reshape(-1)).all()


def test_padded_view_loads(dev):
    # 2-D pad (1,2)x(2,1) of a 5x6 tensor: View::padded (src/graph/shape/view.rs:980-1054)
    x = rnd([5, 6], 7)
    op = D.Operand([6, 1], -1 * 6 - 2, D.F32, 30,
                   [D.Bound([1, 0], 0, 1, 6), D.Bound([0, 1], 0, 2, 8)], -3.0)
    k = D.elementwise([8, 9], [op], w(0) * Ast.const(2.0))
    got, _ = run_gpu(dev, k, [x])
    assert (got == O.run(k, [x])).all()
    ref = np.full((8, 9), -3.0, np.float32)
    ref[1:6, 2:8] = x
    assert (got.reshape(8, 9) == ref * 2).all()


def test_gather_copy_unfold_windows(dev):
    # im2col of a [2,3,8,8] tensor with 3x3 windows, stride 1: C_ kernel (lower.rs:355-359)
    x = rnd([2, 3, 8, 8], 8)
    src = D.Operand([192, 64, 8, 1, 8, 1], 0, D.F32, x.size)
    k = D.copy([2, 3, 6, 6, 3, 3], src)
    got, _ = run_gpu(dev, k, [x])
    assert got.tobytes() == O.run(k, [x]).tobytes()


# ---- reductions -----------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 10), (50, 4), (9, 64), (33, 100), (5, 1024), (3, 4100), (2, 8192), (300, 17)])
@pytest.mark.parametrize("op", [D.R_SUM, D.R_MAX, D.R_MIN, D.R_PROD])
def test_reduce_inner_axis(dev, rows, cols, op):
    lo, hi = (0.9, 1.1) if op == D.R_PROD else (-1.0, 1.0)
    x = rnd([rows, cols], rows * 1000 + cols, lo, hi)
    k = D.reduce([rows, cols], [D.contiguous([rows, cols])], w(0), op, 1)
    got, _ = run_gpu(dev, k, [x])
    ref = O.run(k, [x])
    if op in (D.R_MAX, D.R_MIN):
        assert (got == ref).all()
    elif op == D.R_SUM:
        assert (np.abs(got.astype(np.float64) - ref) <= sum_tolerance(k, [x]) + 1e-30).all()
    else:
        assert_close(got, ref, rel=1e-4)


@pytest.mark.parametrize("rows,cols", [(4096, 256), (5000, 68), (4100, 508), (8192, 128)])
def test_reduce_inner_short_rows_eight_lanes_per_row(dev, rows, cols):
    """Many short rows: eight lanes per row, four rows per warp; with a second operand that repeats for
    every row (a layer's weight vector) and one value per row (a broadcast column)."""
    x, wv, col = rnd([rows, cols], rows + cols), rnd([cols], 5), rnd([rows], 6)
    ins = [D.contiguous([rows, cols]), D.Operand([0, 1], 0, D.F32, cols), D.Operand([1, 0], 0, D.F32, rows)]
    for op, m in ((D.R_SUM, w(0) * w(1) + w(2)), (D.R_MAX, w(0) * w(2))):
        k = D.reduce([rows, cols], ins, m, op, 1)
        got, kern = run_gpu(dev, k, [x, wv, col])
        assert kern.impl == "reduce_inner_t8_v4"
        ref = O.run(k, [x, wv, col])
        if op == D.R_MAX:
            assert (got == ref).all()
        else:
            assert (np.abs(got.astype(np.float64) - ref) <= sum_tolerance(k, [x, wv, col]) + 1e-30).all()


@pytest.mark.parametrize("rows,cols", [(1, 1), (10, 7), (64, 4), (1000, 12), (4096, 64), (513, 130), (70, 1024)])
@pytest.mark.parametrize("op", [D.R_SUM, D.R_MAX])
def test_reduce_outer_axis(dev, rows, cols, op):
    x = rnd([rows, cols], rows * 7 + cols)
    k = D.reduce([rows, cols], [D.contiguous([rows, cols])], w(0), op, 0)
    got, _ = run_gpu(dev, k, [x])
    ref = O.run(k, [x])
    if op == D.R_MAX:
        assert (got == ref).all()
    else:
        assert (np.abs(got.astype(np.float64) - ref) <= sum_tolerance(k, [x]) + 1e-30).all()


@pytest.mark.parametrize("rows,cols,op", [(100000, 32, D.R_SUM), (5000, 36, D.R_SUM), (300, 512, D.R_MAX), (70001, 8, D.R_MAX), (4096, 64, D.R_SUM)])
def test_reduce_outer_narrow_outputs_use_row_lanes(dev, rows, cols, op):
    """Few kept columns (bias gradients): a CTA is (cols / 4) column threads x row lanes.
    Same results as the thread-per-vector kernel (flag 16) and as the oracle; with a
    pre-map and an operand broadcast along the rows."""
    x, b = rnd([rows, cols], rows + 3 * cols), rnd([cols], 9)
    bo = D.Operand([0, 1], 0, D.F32, cols)
    expr = w(0) * w(1) if op == D.R_SUM else w(0) + w(1)
    k = D.reduce([rows, cols], [D.contiguous([rows, cols]), bo], expr, op, 0)
    got, kern = run_gpu(dev, k, [x, b])
    assert kern.impl.startswith("reduce_outer_narrow_v4"), kern.impl
    k.flags = 16
    plain, kern2 = run_gpu(dev, k, [x, b])
    assert kern2.impl.startswith("reduce_outer_v4"), kern2.impl
    ref = O.run(k, [x, b])
    if op == D.R_MAX:
        assert (got == ref).all() and (plain == ref).all()
    else:
        tol = sum_tolerance(k, [x, b]) + 1e-30
        assert (np.abs(got.astype(np.float64) - ref) <= tol).all()
        assert (np.abs(plain.astype(np.float64) - ref) <= tol).all()


@pytest.mark.parametrize("rows,cols,op", [(300, 2048, D.R_SUM), (1000, 4100, D.R_SUM), (160, 8192, D.R_MAX), (500, 2052, D.R_SUM)])
def test_reduce_inner_bulk_copy_staged_variant(dev, rows, cols, op):
    """Descriptor flag 32: rows staged through shared memory by cp.async.bulk with
    per-slot mbarriers; same results as the direct-load kernel."""
    x = rnd([rows, cols], rows + cols)
    m = rnd([rows], 7)
    mb = D.Operand([1, 0], 0, D.F32, rows)
    expr = (w(0) - w(1)).exp() if op == D.R_SUM else w(0) * w(1)
    k = D.reduce([rows, cols], [D.contiguous([rows, cols]), mb], expr, op, 1)
    base, _ = run_gpu(dev, k, [x, m])
    k.flags = 32
    got, kern = run_gpu(dev, k, [x, m])
    dev.synchronize()
    if op == D.R_MAX:
        assert (got == base).all()
    else:
        assert_close(got, base, rel=2e-6)
        assert (np.abs(got.astype(np.float64) - O.run(k, [x, m])) <= sum_tolerance(k, [x, m])).all()


def test_reduce_middle_axis_with_map_and_broadcast(dev):
    shape = [6, 50, 20]
    a = rnd(shape, 11)
    b = rnd([6, 1, 20], 12)
    opb = D.Operand([20, 0, 1], 0, D.F32, 120)
    k = D.reduce(shape, [D.contiguous(shape), opb], (w(0) - w(1)) * (w(0) - w(1)), D.R_SUM, 1)
    got, _ = run_gpu(dev, k, [a, b])
    assert (np.abs(got.astype(np.float64) - O.run(k, [a, b])) <= sum_tolerance(k, [a, b])).all()


def test_long_single_row_split_sum(dev):
    n = 1 << 22
    x = rnd([1, n], 13)
    k = D.reduce([1, n], [D.contiguous([1, n])], w(0) * w(0), D.R_SUM, 1)
    got, kern = run_gpu(dev, k, [x])
    assert kern.launches == 2 and kern.scratch_bytes > 0
    exact = float((x.astype(np.float64) ** 2).sum())
    assert abs(got[0] - exact) <= 1e-5 * exact
    assert abs(O.run(k, [x])[0] - exact) <= 1e-3 * exact   # the sequential f32 loop drifts more


def test_reduce_with_padded_input(dev):
    x = rnd([6, 10], 14)
    op = D.Operand([10, 1], -2, D.F32, 60, [D.Bound([0, 1], 0, 2, 12)], 0.0)
    k = D.reduce([6, 14], [op], w(0), D.R_SUM, 1)
    got, _ = run_gpu(dev, k, [x])
    assert_close(got, O.run(k, [x]), rel=1e-5, abs_tol=1e-5)


def test_softmax_pieces_over_ten_classes(dev):
    # log_softmax (crates/nn/src/functional/activation.rs:174-187): max, sub+exp+sum
    logits = rnd([512, 10], 15, -4, 4)
    kmax = D.reduce([512, 10], [D.contiguous([512, 10])], w(0), D.R_MAX, 1)
    m, _ = run_gpu(dev, kmax, [logits])
    assert (m == logits.max(1)).all()
    mb = D.Operand([1, 0], 0, D.F32, 512)
    ksum = D.reduce([512, 10], [D.contiguous([512, 10]), mb], (w(0) - w(1)).exp(), D.R_SUM, 1)
    s, _ = run_gpu(dev, ksum, [logits, m])
    assert_close(s, O.run(ksum, [logits, m]), rel=1e-5)


# ---- transposes -----------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(16, 16), (64, 64), (65, 63), (17, 300), (1000, 33), (512, 2048)])
def test_transpose_bit_exact(dev, rows, cols):
    x = rnd([rows, cols], rows + cols)
    x.reshape(-1)[::97] = np.nan        # payload bits must survive too
    k = W.cfg2_t(rows, cols)
    got, kern = run_gpu(dev, k, [x])
    assert kern.impl == "transpose_copy"
    assert got.tobytes() == np.ascontiguousarray(x.T).tobytes()
    assert got.tobytes() == O.run(k, [x]).tobytes()


def test_batched_and_inner_permutes_bit_exact(dev):
    x = rnd([3, 40, 5, 48], 16)
    for perm in [(0, 3, 2, 1), (3, 0, 1, 2), (1, 0, 3, 2), (2, 3, 0, 1), (0, 2, 1, 3)]:
        st = D.contiguous_strides(x.shape)
        shape = [x.shape[p] for p in perm]
        src = D.Operand([st[p] for p in perm], 0, D.F32, x.size)
        k = D.elementwise(shape, [src], w(0))
        got, _ = run_gpu(dev, k, [x])
        assert got.tobytes() == np.ascontiguousarray(x.transpose(perm)).tobytes(), perm


def test_conv_patch_permute_bit_exact(dev):
    # [N,C,Ho,Wo,kh,kw] -> [N,Ho,Wo,C,kh,kw] (crates/nn/src/functional/conv.rs:150-158)
    x = rnd([4, 8, 11, 11, 3, 3], 17)
    perm = (0, 2, 3, 1, 4, 5)
    st = D.contiguous_strides(x.shape)
    shape = [x.shape[p] for p in perm]
    k = D.elementwise(shape, [D.Operand([st[p] for p in perm], 0, D.F32, x.size)], w(0))
    got, _ = run_gpu(dev, k, [x])
    assert got.tobytes() == np.ascontiguousarray(x.transpose(perm)).tobytes()


# ---- dense contraction ------------------------------------------------------------------------

def gemm_check(dev, k, a, b, ref64, rel):
    got, kern = run_gpu(dev, k, [a, b])
    if min(k.shape) > 1:    # degenerate extents collapse into plain reduces
        assert kern.impl.startswith("gemm")
    scale = np.abs(a.astype(np.float64)).max() * np.abs(b.astype(np.float64)).max() * k.shape[k.reduce_axis]
    err = np.abs(got.astype(np.float64) - ref64.reshape(-1)).max()
    assert err <= rel * scale, (err, scale)
    return got, kern


def test_cfg1_matmul_512(dev):
    """Config 1: A, B uniform[-1,1] from seed 0 (A first), 512^3."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    b = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    k = W.matmul_desc(512, 512, 512)
    got, kern = gemm_check(dev, k, a, b, a.astype(np.float64) @ b.astype(np.float64), 1e-6)
    assert kern.impl.startswith("gemm_tcgen05_3xtf32_kn")
    bound = 1e-5 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)).reshape(-1)
    for fma in (False, True):           # both forms the reference's C backend can take
        ref = O.run(k, [a, b], fma=fma)
        assert (np.abs(got.astype(np.float64) - ref) <= bound).all()
    # the f32 FFMA kernel on the same contraction agrees with the C loop much more tightly
    k2 = W.matmul_desc(512, 512, 512); k2.flags = 8
    got2, kern2 = run_gpu(dev, k2, [a, b])
    assert kern2.impl.startswith("gemm_simt_f32")
    assert_close(got2, O.run(k2, [a, b]), rel=1e-5, abs_tol=1e-5 * np.sqrt(512) * 0.34)


@pytest.mark.parametrize("m,k_,n", [(1, 1, 1), (5, 7, 3), (64, 16, 64), (65, 17, 66), (200, 300, 10), (1000, 9, 32)])
def test_gemm_odd_shapes_all_forms(dev, m, k_, n):
    a, b = rnd([m, k_], 20), rnd([k_, n], 21)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    gemm_check(dev, W.matmul_desc(m, k_, n), a, b, ref, 1e-6)
    # linear form: x[M,K] . W[N,K]^T
    wt = np.ascontiguousarray(b.T)
    gemm_check(dev, W.linear_desc(m, k_, n), a, wt, ref, 1e-6)


def test_gemm_batched(dev):
    a, b = rnd([6, 33, 20], 22), rnd([6, 20, 41], 23)
    ref = np.einsum("bmk,bkn->bmn", a.astype(np.float64), b.astype(np.float64))
    gemm_check(dev, W.matmul_desc(33, 20, 41, batch=6), a, b, ref, 1e-6)


def test_gemm_weight_gradient_form(dev):
    # dW[o,i] = sum_b dy[b,o] * x[b,i]  (VJP of linear: src/grad/rules.rs:196-222): reduce over axis 0
    dy, x = rnd([50, 12], 24), rnd([50, 30], 25)
    a = D.Operand([12, 1, 0], 0, D.F32, dy.size)
    b = D.Operand([30, 0, 1], 0, D.F32, x.size)
    k = D.reduce([50, 12, 30], [a, b], w(0) * w(1), D.R_SUM, 0)
    gemm_check(dev, k, dy, x, dy.astype(np.float64).T @ x.astype(np.float64), 1e-6)


@pytest.mark.parametrize("mode,tol", [(D.GEMM_TF32, 1e-2), (D.GEMM_3XTF32, 1e-5)])
@pytest.mark.parametrize("m,k_,n", [(128, 128, 128), (256, 96, 384), (300, 1000, 200), (129, 68, 260), (1024, 512, 64)])
def test_gemm_tensor_core_modes_and_layouts(dev, mode, tol, m, k_, n):
    """tcgen05 path: TF32 within 1e-2, 3xTF32 within 1e-5 of the float64 product,
    relative to sum_k |a_ik b_kj| (the bound that holds for any summation order;
    elementwise-relative is meaningless where a dot product cancels), for N-major B
    (matmul_demo form) and K-major B (linear form), including ragged M/N/K tails."""
    a, b = rnd([m, k_], 30), rnd([k_, n], 31)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    for form in ("nn", "tn"):
        if form == "nn":
            kd = W.matmul_desc(m, k_, n, mode=mode); got, kern = run_gpu(dev, kd, [a, b])
        else:
            kd = W.linear_desc(m, k_, n, mode=mode); got, kern = run_gpu(dev, kd, [a, np.ascontiguousarray(b.T)])
        assert kern.impl.startswith("gemm_tcgen05"), kern.impl
        err = np.abs(got.reshape(m, n) - ref)
        assert (err <= tol * scale).all(), (form, err.max(), float((err / scale).max()))
    dev.synchronize()     # would raise TIMEOUT had any bounded wait in the kernel run out


def test_gemm_tensor_core_batched_and_strided_views(dev):
    # batch of 5; A rows are a window [.., 0:64] of a wider [96, 80] matrix (lda = 80)
    a_full, b = rnd([5, 96, 80], 32), rnd([5, 64, 160], 33)
    a_op = D.Operand([96 * 80, 80, 1, 0], 0, D.F32, a_full.size)
    b_op = D.Operand([64 * 160, 0, 160, 1], 0, D.F32, b.size)
    kd = D.reduce([5, 96, 64, 160], [a_op, b_op], w(0) * w(1), D.R_SUM, 2)
    got, kern = run_gpu(dev, kd, [a_full, b])
    assert kern.impl.startswith("gemm_tcgen05")
    ref = np.einsum("bmk,bkn->bmn", a_full[:, :, :64].astype(np.float64), b.astype(np.float64))
    assert np.abs(got.reshape(ref.shape) - ref).max() <= 1e-5 * np.abs(ref).max()
    # B shared across the batch (stride 0 on the batch dim)
    b1 = rnd([64, 160], 34)
    b_op = D.Operand([0, 0, 160, 1], 0, D.F32, b1.size)
    kd = D.reduce([5, 96, 64, 160], [a_op, b_op], w(0) * w(1), D.R_SUM, 2)
    got, kern = run_gpu(dev, kd, [a_full, b1])
    ref = np.einsum("bmk,kn->bmn", a_full[:, :, :64].astype(np.float64), b1.astype(np.float64))
    assert np.abs(got.reshape(ref.shape) - ref).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("b_,o_,i_", [(4096, 128, 256), (20000, 64, 288), (3000, 32, 9), (1000, 10, 128)])
def test_gemm_weight_gradient_split_k(dev, b_, o_, i_):
    """dW = dy^T x: M-major A, long K, split over CTAs with partials in scratch."""
    dy, x = rnd([b_, o_], 37), rnd([b_, i_], 38)
    a = D.Operand([o_, 1, 0], 0, D.F32, dy.size)
    b = D.Operand([i_, 0, 1], 0, D.F32, x.size)
    k = D.reduce([b_, o_, i_], [a, b], w(0) * w(1), D.R_SUM, 0)
    got, kern = run_gpu(dev, k, [dy, x])
    assert "splitk" in kern.impl and kern.scratch_bytes > 0
    ref = dy.astype(np.float64).T @ x.astype(np.float64)
    bound = 1e-5 * (np.abs(dy).astype(np.float64).T @ np.abs(x).astype(np.float64))
    assert (np.abs(got.reshape(o_, i_) - ref) <= bound).all(), kern.impl
    dev.synchronize()


@pytest.mark.parametrize("b_,o_,i_", [(40000, 32, 9), (100001, 10, 32), (65536, 7, 5), (300000, 32, 27)])
def test_gemm_tall_skinny_weight_gradient(dev, b_, o_, i_):
    """dW[o, i] = sum_b dy[b, o] * x[b, i] with a one-tile output and a very long
    reduction (conv1's weight gradient): lane per output row, warp-uniform loads of
    x's row, partials per CTA summed in order.  Against float64 and the split-K f32 kernel."""
    dy, x = rnd([b_, o_], 47), rnd([b_, i_], 48)
    a = D.Operand([o_, 1, 0], 0, D.F32, dy.size)
    b = D.Operand([i_, 0, 1], 0, D.F32, x.size)
    k = D.reduce([b_, o_, i_], [a, b], w(0) * w(1), D.R_SUM, 0)
    got, kern = run_gpu(dev, k, [dy, x])
    assert kern.impl == "gemm_tall_f32_splitk", kern.impl
    ref = dy.astype(np.float64).T @ x.astype(np.float64)
    bound = 1e-5 * (np.abs(dy).astype(np.float64).T @ np.abs(x).astype(np.float64))
    assert (np.abs(got.reshape(o_, i_) - ref) <= bound).all()
    k.flags = 16
    other, kern2 = run_gpu(dev, k, [dy, x])
    assert kern2.impl.startswith("gemm_simt_f32")
    assert (np.abs(other.reshape(o_, i_) - ref) <= bound).all()


@pytest.mark.parametrize("form", ["nn", "tn", "wgrad"])
def test_gemm_3xtf32_split_in_the_kernel_equals_split_beforehand(dev, form):
    """3xTF32 either splits the operands into hi / lo copies with two passes beforehand (large,
    compute-bound contractions) or inside the kernel after the TMA load (everything below 200
    flop per operand byte).  Same hi / lo values, same MMAs: the results are equal bit for bit."""
    m, k_, n = 384, 200, 320
    a, b = rnd([m, k_], 55), rnd([k_, n], 56)
    if form == "nn":
        kd, ins = W.matmul_desc(m, k_, n), [a, b]
    elif form == "tn":
        kd, ins = W.linear_desc(m, k_, n), [a, np.ascontiguousarray(b.T)]
    else:
        dy, x = rnd([4096, 64], 57), rnd([4096, 96], 58)
        kd = D.reduce([4096, 64, 96], [D.Operand([64, 1, 0], 0, D.F32, dy.size), D.Operand([96, 0, 1], 0, D.F32, x.size)],
                      w(0) * w(1), D.R_SUM, 0)
        ins = [dy, x]
    outs = {}
    for mode in ("1", "0"):
        kd.flags = 8192 if mode == "1" else 4096       # descriptor flags: split inside the kernel / by a pre-pass
        got, kern = run_gpu(dev, kd, ins)
        assert kern.impl.startswith("gemm_tcgen05_3xtf32"), kern.impl
        assert (kern.scratch_bytes == 0) == (mode == "1" and "splitk" not in kern.impl) or "splitk" in kern.impl
        outs[mode] = got
    assert np.array_equal(outs["1"], outs["0"])
    dev.synchronize()


def test_gemm_misaligned_layout_stays_on_f32_kernel(dev):
    # lda = 30 floats is not a multiple of 16 bytes: TMA cannot address it
    a, b = rnd([64, 30], 35), rnd([30, 64], 36)
    kd = W.matmul_desc(64, 30, 64)
    got, kern = run_gpu(dev, kd, [a, b])
    assert kern.impl == "gemm_simt_f32"
    assert np.abs(got.reshape(64, 64) - a.astype(np.float64) @ b.astype(np.float64)).max() <= 1e-5


# ---- scatter / sgd ---------------------------------------------------------------------------------

def test_scatter_add_overlapping_windows(dev):
    # fold of 3x3 stride-1 windows over [2,4,9,9] -> overlapping accumulation; served as a gather over the output,
    # which adds the terms in the order of the reference's sequential loop nest: bit-identical to the plain C oracle
    n, c, h = 2, 4, 9
    oh = h - 2
    cols = rnd([n, c, oh, oh, 3, 3], 26)
    out = D.Operand([c * h * h, h * h, h, 1, h, 1], 0, D.F32, n * c * h * h)
    k = D.KernelDesc(D.K_SCATTER, list(cols.shape), [D.contiguous(cols.shape)], out)
    got, kern = run_gpu(dev, k, [cols])
    assert kern.impl == "scatter_add_as_gather"
    assert got.tobytes() == O.run(k, [cols]).tobytes()


@pytest.mark.parametrize("case", ["overlap_rows_only", "permuted_input", "strided_dilated", "one_plane", "many_planes_merged"])
def test_fold_as_gather_matches_the_sequential_loop_bit_for_bit(dev, case):
    from harp_b200.frontend import View
    if case == "overlap_rows_only":     # 3x2 windows, stride 2: rows overlap, columns do not; row 11 / column 10 stay zero
        src_shape, dst_shape, uf = [3, 5, 5, 5, 3, 2], [3, 5, 12, 11], ([2, 3], [3, 2], [2, 2], [1, 1])
        src = D.contiguous(src_shape)
    elif case == "permuted_input":      # the [n, ho, wo, c, kh, kw] rows a convolution-as-GEMM produces
        src_shape, dst_shape, uf = [4, 6, 11, 11, 3, 3], [4, 6, 13, 13], ([2, 3], [3, 3], [1, 1], [1, 1])
        src = D.Operand([11 * 11 * 6 * 9, 9, 11 * 6 * 9, 6 * 9, 3, 1], 0, D.F32, int(np.prod(src_shape)))
    elif case == "strided_dilated":     # stride 3, dilation 2 (columns overlap, some rows no window reaches)
        src_shape, dst_shape, uf = [2, 3, 4, 5, 2, 3], [2, 3, 12, 17], ([2, 3], [2, 3], [3, 3], [2, 2])
        src = D.contiguous(src_shape)
    elif case == "many_planes_merged":  # row-disjoint windows over planes that collapse into ONE plane of 1 M rows
        src_shape, dst_shape, uf = [262200, 1, 2, 2, 2, 3], [262200, 1, 4, 5], ([2, 3], [2, 3], [2, 2], [1, 1])
        src = D.contiguous(src_shape)
    else:
        src_shape, dst_shape, uf = [1, 1, 30, 30, 3, 3], [1, 1, 32, 32], ([2, 3], [3, 3], [1, 1], [1, 1])
        src = D.contiguous(src_shape)
    x = rnd([int(np.prod(src_shape))], 77)
    dst = View.contiguous(dst_shape).unfold(*uf)
    assert list(dst.shape) == src_shape
    k = D.KernelDesc(D.K_SCATTER, src_shape, [src], dst.operand(int(np.prod(dst_shape)), D.F32), None)
    got, kern = run_gpu(dev, k, [x])
    assert kern.impl == "scatter_add_as_gather" and kern.launches == 2
    assert got.tobytes() == O.run(k, [x]).tobytes()


def test_fold_of_disjoint_windows_keeps_the_atomic_kernel(dev):
    # a pooling gradient: 2x2 windows, stride 2, over 11x11 planes -- at most one term per element, exact in any order
    from harp_b200.frontend import View
    src_shape, dst_shape = [3, 5, 5, 5, 2, 2], [3, 5, 11, 11]
    x = rnd([int(np.prod(src_shape))], 79)
    dst = View.contiguous(dst_shape).unfold([2, 3], [2, 2], [2, 2], [1, 1])
    k = D.KernelDesc(D.K_SCATTER, src_shape, [D.contiguous(src_shape)], dst.operand(int(np.prod(dst_shape)), D.F32), None)
    got, kern = run_gpu(dev, k, [x])
    assert kern.impl == "scatter_add"
    assert got.tobytes() == O.run(k, [x]).tobytes()


def test_scatter_that_is_not_a_fold_keeps_the_atomic_kernel(dev):
    # planes that overlap each other (stride 5 between planes of 9 elements): no output element owns its terms
    x = rnd([6, 2, 2, 2, 2], 78)
    out = D.Operand([5, 3, 1, 3, 1], 0, D.F32, 40)
    k = D.KernelDesc(D.K_SCATTER, [6, 2, 2, 2, 2], [D.contiguous([6, 2, 2, 2, 2])], out)
    got, kern = run_gpu(dev, k, [x])
    assert kern.impl == "scatter_add"
    assert_close(got, O.run(k, [x]), rel=1e-5, abs_tol=1e-5)


@pytest.mark.parametrize("n", [1, 5, 4096, 225034])
def test_sgd_update_bit_exact(dev, n):
    p, g = rnd([n], 27), rnd([n], 28)
    k = D.KernelDesc(D.K_SGD, [n], [D.contiguous([n]), D.contiguous([n])], D.contiguous([n]), scalar=1e-2)
    got, _ = run_gpu(dev, k, [p, g])
    lr = np.float32(1e-2)
    assert got.tobytes() == (p - lr * g).astype(np.float32).tobytes()


# ---- config 2 at full size -------------------------------------------------------------------

def test_cfg2_full_size(dev, registry):
    x = W.cfg2_input()
    c0, c1 = W.cfg2_consts()
    ky, kz, kt = W.cfg2_y(), W.cfg2_z(), W.cfg2_t()
    y, kern_y = run_gpu(dev, ky, [c0, x, c1])
    z, kern_z = run_gpu(dev, kz, [x])
    t, kern_t = run_gpu(dev, kt, [x])
    assert kern_y.impl.startswith("reduce_inner") and kern_y.specialised
    assert kern_z.impl == "reduce_outer_v4_split" and kern_t.impl == "transpose_copy"
    # oracle at full size (OpenMP form, same arithmetic per row)
    y_ref = O.run(ky, [c0, x, c1], openmp=True)
    tol = sum_tolerance(ky, [c0, x, c1])
    assert (np.abs(y.astype(np.float64) - y_ref) <= tol).all()
    y64 = O.eval_f64(ky, [c0, x, c1])
    assert (np.abs(y - y64) <= tol).all() and (np.abs(y_ref - y64) <= tol).all()
    assert (z == x.max(axis=0)).all()
    assert t.tobytes() == np.ascontiguousarray(x.T).tobytes()
    # size-independent properties: transposing twice is the identity; the max of
    # the column maxima is the global max
    tt, _ = run_gpu(dev, kt, [t])
    assert tt.tobytes() == x.tobytes()
    assert z.max() == x.max()


# ---- conv2d as one implicit-GEMM kernel --------------------------------------------------------------

def _conv_ref64(x, w_, b, pad, relu):
    """float64 direct convolution in NHWC-flattened [M, Co] order, plus sum |terms|."""
    n, c, h, wd = x.shape
    co, _, kh, kw = w_.shape
    xp = np.zeros((n, c, h + 2 * pad, wd + 2 * pad)); xp[:, :, pad:pad + h, pad:pad + wd] = x
    ho, wo = h + 2 * pad - kh + 1, wd + 2 * pad - kw + 1
    win = np.lib.stride_tricks.sliding_window_view(xp, (kh, kw), axis=(2, 3))       # [n, c, ho, wo, kh, kw]
    cols = win.transpose(0, 2, 3, 1, 4, 5).reshape(n * ho * wo, c * kh * kw)
    wm = w_.reshape(co, -1).astype(np.float64)
    ref = cols @ wm.T
    scale = np.abs(cols) @ np.abs(wm).T
    if b is not None:
        ref = ref + b.astype(np.float64)[None, :]
        scale = scale + np.abs(b.astype(np.float64))[None, :]
    if relu:
        ref = np.maximum(ref, 0.0)
    return ref, scale


@pytest.mark.parametrize("mode,tol", [(D.GEMM_TF32, 1e-2), (D.GEMM_3XTF32, 1e-5)])
@pytest.mark.parametrize("shape", [
    (4, 1, 28, 28, 32, 3, 3, 0),       # first CNN layer: K = 9 padded to one 32-wide block
    (3, 32, 13, 13, 64, 3, 3, 0),      # second CNN layer: K = 288, nine blocks
    (2, 3, 17, 19, 20, 3, 3, 1),       # zero padding, ragged M (not a multiple of 128) and Co (not of 32)
    (1, 8, 9, 9, 130, 5, 5, 2),        # Co spans two 128-wide column tiles, 5x5 window
    (2, 5, 6, 7, 7, 1, 1, 0),          # 1x1 window
    (2, 64, 10, 12, 48, 3, 3, 1),      # channel-blocked k order (C % 32 == 0) with padding
    (300, 1, 28, 28, 32, 3, 3, 0),     # 1585 row tiles: every persistent CTA walks several tiles
    (32, 32, 40, 40, 140, 3, 3, 1),    # 400 x 2 tiles, channel-blocked, two column tiles
    (1, 32, 16, 16, 8, 7, 7, 3),       # 49 taps: the table without tap bits
])
def test_conv2d_implicit_gemm_matches_direct_convolution(dev, mode, tol, shape):
    n, c, h, wd, co, kh, kw, pad = shape
    x, w_, b = rnd([n, c, h, wd], 60), rnd([co, c, kh, kw], 61), rnd([co], 62)
    ho, wo = h + 2 * pad - kh + 1, wd + 2 * pad - kw + 1
    for bias, relu, nchw in ((True, True, False), (False, False, True)):
        kd = D.conv2d(n, c, h, wd, co, kh, kw, pad=pad, bias=bias, relu=relu, mode=mode, nchw=nchw)
        kd.flags |= D.FLAG_TENSOR_CORE       # layers with C*KH*KW <= 32 would otherwise take the streaming f32 kernel
        ins = [x, w_, b] if bias else [x, w_]
        got, kern = run_gpu(dev, kd, ins)
        assert kern.impl.startswith("conv2d_igemm"), kern.impl
        ref, scale = _conv_ref64(x, w_, b if bias else None, pad, relu)
        cpu = O.run(kd, ins)
        if nchw:      # flag 512: [N, Co, Ho, Wo] instead of [N*Ho*Wo, Co]
            got = got.reshape(n, co, ho, wo).transpose(0, 2, 3, 1)
            cpu = cpu.reshape(n, co, ho, wo).transpose(0, 2, 3, 1)
        err = np.abs(got.reshape(ref.shape) - ref)
        assert (err <= tol * scale + 1e-30).all(), (shape, bias, float((err / np.maximum(scale, 1e-30)).max()))
        # and against the CPU oracle's loop nest (same bound: the summation orders differ)
        assert (np.abs(got.reshape(ref.shape) - cpu.reshape(ref.shape)) <= 2 * tol * scale + 1e-30).all()
    dev.synchronize()     # would raise TIMEOUT had a bounded wait in the kernel run out


def test_conv2d_fused_front_end_equals_composed_spelling(dev):
    """conv2d_fused (one kernel) against conv2d + relu spelled the reference's way
    (pad, unfold, permute, contiguous, GEMM, bias), both on the GPU."""
    from harp_b200 import frontend as F
    x, w_, b = rnd([3, 4, 12, 12], 63), rnd([6, 4, 3, 3], 64), rnd([6], 65)
    ex = F.B200Executor(dev)
    outs = []
    for fused in (True, False):
        X, Wt, B = F.Tensor.input(x), F.Tensor.input(w_), F.Tensor.input(b)
        y = X.conv2d_fused(Wt, B, padding=1, relu=True) if fused else X.conv2d(Wt, B, padding=1).relu()
        y = y.contiguous()
        p = F.Program([y], ex)
        p.run()
        outs.append(p.fetch(y))
        if fused:
            assert [d.kclass for d in p.kernel_descs()] == [D.K_CONV2D]      # the kernel writes NCHW itself
    assert outs[0].shape == (3, 6, 12, 12)
    assert np.abs(outs[0] - outs[1]).max() <= 1e-4


@pytest.mark.parametrize("mode,tol", [(D.GEMM_TF32, 1e-2), (D.GEMM_3XTF32, 1e-5)])
@pytest.mark.parametrize("shape", [(3, 32, 13, 13, 64, 3, 0), (2, 3, 9, 10, 5, 3, 1), (2, 8, 12, 12, 16, 5, 2)])
def test_conv2d_input_gradient_is_the_same_kernel_over_flipped_weights(dev, mode, tol, shape):
    """dX of y = conv2d(x, w, pad) is conv2d(dy, w', k-1-pad) with w'[c][co][kh][kw] =
    w[co][c][K-1-kh][K-1-kw] (descriptor flag 128 reads the forward weights that way):
    checked against the float64 adjoint of the forward convolution."""
    n, c, h, wd, co, k, pad = shape
    ho, wo = h + 2 * pad - k + 1, wd + 2 * pad - k + 1
    g, w_ = rnd([n, co, ho, wo], 70), rnd([co, c, k, k], 71)
    kd = D.conv2d(n, co, ho, wo, c, k, k, pad=k - 1 - pad, bias=False, flip=True, mode=mode)
    kd.flags |= D.FLAG_TENSOR_CORE
    got, kern = run_gpu(dev, kd, [g, w_])
    assert kern.impl.startswith("conv2d_igemm") and kern.impl.endswith("_dgrad"), kern.impl
    # adjoint in float64: scatter every dy element times its window of weights
    ref = np.zeros((n, c, h + 2 * pad, wd + 2 * pad)); scale = np.zeros_like(ref)
    for i in range(k):
        for j in range(k):
            t = np.einsum("nohw,oc->nchw", g.astype(np.float64), w_[:, :, i, j].astype(np.float64))
            ta = np.einsum("nohw,oc->nchw", np.abs(g).astype(np.float64), np.abs(w_[:, :, i, j]).astype(np.float64))
            ref[:, :, i:i + ho, j:j + wo] += t; scale[:, :, i:i + ho, j:j + wo] += ta
    sl = (slice(None), slice(None), slice(pad, pad + h), slice(pad, pad + wd))
    ref, scale = ref[sl].transpose(0, 2, 3, 1).reshape(-1, c), scale[sl].transpose(0, 2, 3, 1).reshape(-1, c)
    err = np.abs(got.reshape(ref.shape) - ref)
    assert (err <= tol * scale + 1e-30).all(), float((err / np.maximum(scale, 1e-30)).max())
    cpu = O.run(kd, [g, w_]).reshape(ref.shape)
    assert (np.abs(got.reshape(ref.shape) - cpu) <= 2 * tol * scale + 1e-30).all()
    dev.synchronize()


@pytest.mark.parametrize("mode,tol", [(D.GEMM_TF32, 1e-2), (D.GEMM_3XTF32, 1e-5)])
@pytest.mark.parametrize("shape", [
    (5, 1, 28, 28, 32, 3, 0),          # conv1 of config 4: K = 9, 676 positions per image (22 blocks, the last ragged)
    (6, 32, 13, 13, 64, 3, 0),         # conv2: K = 288 = three row tiles, 121 positions
    (3, 4, 9, 10, 20, 3, 1),           # padding, Co not a multiple of 32
    (400, 8, 6, 6, 8, 3, 1),           # more images than CTAs per row tile: every stream walks several images
    (2, 16, 8, 8, 128, 5, 2),          # 5x5 window, K = 400 (four row tiles), 128 output channels
])
def test_conv2d_weight_gradient_contracts_positions_on_the_tensor_cores(dev, mode, tol, shape):
    """dW[co, c, kh, kw] = sum_{n, oh, ow} g[n, oh, ow, co] x[n, c, oh+kh-p, ow+kw-p] as one kernel
    (flag 256) against float64 and against the oracle's loop nest."""
    n, c, h, wd, co, k, pad = shape
    ho, wo = h + 2 * pad - k + 1, wd + 2 * pad - k + 1
    x, g = rnd([n, c, h, wd], 80), rnd([n * ho * wo, co], 81)
    kd = D.conv2d_wgrad(n, c, h, wd, co, k, k, pad=pad, mode=mode)
    kd.flags |= D.FLAG_TENSOR_CORE
    got, kern = run_gpu(dev, kd, [x, g])
    assert kern.impl.startswith("conv2d_igemm") and kern.impl.endswith("_wgrad") and kern.launches == 2, kern.impl
    xp = np.zeros((n, c, h + 2 * pad, wd + 2 * pad)); xp[:, :, pad:pad + h, pad:pad + wd] = x
    win = np.lib.stride_tricks.sliding_window_view(xp, (k, k), axis=(2, 3))       # [n, c, ho, wo, k, k]
    cols = win.transpose(0, 2, 3, 1, 4, 5).reshape(n * ho * wo, c * k * k)
    ref = g.astype(np.float64).T @ cols
    scale = np.abs(g).astype(np.float64).T @ np.abs(cols)
    err = np.abs(got.reshape(ref.shape) - ref)
    assert (err <= tol * scale + 1e-30).all(), float((err / np.maximum(scale, 1e-30)).max())
    cpu = O.run(kd, [x, g]).reshape(ref.shape)
    assert (np.abs(got.reshape(ref.shape) - cpu) <= 2 * tol * scale + 1e-30).all()
    dev.synchronize()


@pytest.mark.parametrize("shape", [
    (5, 1, 28, 28, 32, 3, 3, 0),       # conv1 of config 4
    (3, 3, 9, 11, 20, 3, 3, 1),        # K = 27, padding, Co not a multiple of 4
    (2, 2, 8, 8, 7, 2, 4, 1),          # K = 16, rectangular window
    (300, 1, 12, 12, 5, 5, 5, 2),      # K = 25; more positions than one grid pass
])
def test_conv2d_tiny_reduction_streams_through_the_f32_kernel(dev, shape):
    """C*KH*KW <= 32: forward (both output layouts, bias, ReLU), the input gradient through
    flipped weights, and for K <= 12 the weight gradient (both gradient layouts) on the
    streaming FFMA kernels: within 1e-5 of sum |terms| of float64, like 3xTF32."""
    n, c, h, wd, co, kh, kw, pad = shape
    ho, wo = h + 2 * pad - kh + 1, wd + 2 * pad - kw + 1
    x, w_, b = rnd([n, c, h, wd], 90), rnd([co, c, kh, kw], 91), rnd([co], 92)
    for nchw in (False, True):
        kd = D.conv2d(n, c, h, wd, co, kh, kw, pad=pad, bias=True, relu=True, nchw=nchw)
        got, kern = run_gpu(dev, kd, [x, w_, b])
        assert kern.impl == "conv2d_direct_f32" and kern.launches == 1, kern.impl
        ref, scale = _conv_ref64(x, w_, b, pad, True)
        if nchw:
            got = got.reshape(n, co, ho, wo).transpose(0, 2, 3, 1)
        assert (np.abs(got.reshape(ref.shape) - ref) <= 1e-5 * scale + 1e-30).all()
    if c * kh * kw <= 12:
        g = rnd([n, co, ho, wo], 93)
        xp = np.zeros((n, c, h + 2 * pad, wd + 2 * pad)); xp[:, :, pad:pad + h, pad:pad + wd] = x
        cols = np.lib.stride_tricks.sliding_window_view(xp, (kh, kw), axis=(2, 3)).transpose(0, 2, 3, 1, 4, 5).reshape(n * ho * wo, -1)
        grows = g.transpose(0, 2, 3, 1).reshape(n * ho * wo, co)
        ref = grows.astype(np.float64).T @ cols
        scale = np.abs(grows).astype(np.float64).T @ np.abs(cols)
        for g_nchw, gin in ((True, g), (False, np.ascontiguousarray(grows))):
            kd = D.conv2d_wgrad(n, c, h, wd, co, kh, kw, pad=pad, g_nchw=g_nchw)
            got, kern = run_gpu(dev, kd, [x, gin])
            assert kern.impl == "conv2d_direct_f32_wgrad", kern.impl
            assert (np.abs(got.reshape(ref.shape) - ref) <= 1e-5 * scale + 1e-30).all()
            cpu = O.run(kd, [x, gin]).reshape(ref.shape)
            assert (np.abs(got.reshape(ref.shape) - cpu) <= 2e-5 * scale + 1e-30).all()
    if kh == kw and kh - 1 - pad >= 0 and co * kh * kw <= 32:
        g = rnd([n, co, ho, wo], 94)
        kd = D.conv2d(n, co, ho, wo, c, kh, kw, pad=kh - 1 - pad, bias=False, flip=True)
        got, kern = run_gpu(dev, kd, [g, w_])
        assert kern.impl == "conv2d_direct_f32_dgrad", kern.impl
        cpu = O.run(kd, [g, w_])
        assert np.abs(got - cpu).max() <= 1e-4 * max(1.0, np.abs(cpu).max())
