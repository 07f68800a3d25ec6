"""Graph front end on the CPU: view algebra, fusion, autograd and lowering,
executed through the oracle.  Pins the reference's autograd known-answer
vectors (crates/backend-metal/src/lib.rs:261-369, backend-agnostic semantics)
and the view-algebra facts of src/graph/shape/view.rs."""
import numpy as np
import pytest

from harp_b200 import desc as D
from harp_b200.frontend import Program, Tensor, View
from oracle.executor import OracleExecutor


def run(roots, fuse="chains"):
    p = Program(roots, OracleExecutor(), fuse=fuse)
    p.run()
    return [p.fetch(r) for r in roots], p


# ---- view algebra (src/graph/shape/view.rs:1437-1674, 2204-2348) ------------------------
def test_views_contiguous_permute_unsqueeze_expand():
    v = View.contiguous((2, 3, 4))
    assert v.strides == (12, 4, 1)
    assert v.permute((2, 0, 1)).strides == (1, 12, 4) and v.permute((2, 0, 1)).shape == (4, 2, 3)
    u = v.unsqueeze(1)
    assert u.shape == (2, 1, 3, 4) and u.strides == (12, 0, 4, 1)
    e = u.expand((2, 5, 3, 4))
    assert e.strides == (12, 0, 4, 1)
    assert v.reshape((6, 4)).strides == (4, 1) and v.permute((1, 0, 2)).reshape((6, 4)) is None


def test_unfold_shape_and_index():
    # [1,1,4,4] windows 2x2 stride 2 -> [1,1,2,2,2,2]; index = pos*stride + win*dilation
    v = View.contiguous((1, 1, 4, 4)).unfold([2, 3], [2, 2], [2, 2], [1, 1])
    assert v.shape == (1, 1, 2, 2, 2, 2) and v.strides == (16, 16, 8, 2, 4, 1)
    v = View.contiguous((8,)).unfold([0], [3], [1], [2])      # dilation 2
    assert v.shape == (4, 3) and v.strides == (1, 2)


def test_padded_view_bounds_survive_permute_and_unfold():
    v = View.contiguous((5, 6)).pad([(1, 2), (2, 1)])
    assert v.shape == (8, 9) and v.offset == -8 and len(v.bounds) == 2
    p = v.permute((1, 0))
    assert [tuple(b.coef) for b in p.bounds] == [(0, 1), (1, 0)]
    u = v.unfold([1], [3], [1], [1])                           # [8, 7, 3]
    assert tuple(u.bounds[1].coef) == (0, 1, 1)


# ---- the reference's autograd vectors -------------------------------------------------
def test_ref_autograd_square():
    x = Tensor.input([1, 2, 3, 4], requires_grad=True)
    (gx,), _ = run((x * x).sum().backward([x]))
    assert gx.tolist() == [2.0, 4.0, 6.0, 8.0]


def test_ref_autograd_mul():
    a = Tensor.input([1, 2, 3, 4], requires_grad=True)
    b = Tensor.input([2, 3, 4, 5], requires_grad=True)
    (ga, gb), _ = run((a * b).sum().backward([a, b]))
    assert ga.tolist() == [2.0, 3.0, 4.0, 5.0] and gb.tolist() == [1.0, 2.0, 3.0, 4.0]


def test_ref_autograd_add_same_tensor():
    x = Tensor.input([1, 2, 3, 4], requires_grad=True)
    (gx,), _ = run((x + x).sum().backward([x]))
    assert gx.tolist() == [2.0, 2.0, 2.0, 2.0]


def test_ref_unfold_fold_roundtrip():
    x = Tensor.input(np.arange(16).reshape(1, 1, 4, 4))
    f = x.unfold([2, 3], [2, 2], [2, 2], [1, 1]).fold((1, 1, 4, 4), [2, 3], [2, 2], [2, 2], [1, 1])
    (out,), p = run([f])
    assert out.sum() == 120.0 and (out == x.node.data).all()
    assert [d.kclass for d in p.kernel_descs()] == [D.K_COPY, D.K_SCATTER]


# ---- fusion levels ---------------------------------------------------------------------
def cfg2_graph(rows=16, cols=32):
    x = Tensor.input(np.random.default_rng(2).standard_normal((rows, cols)))
    c0, c1 = Tensor.input(np.float32(0.5)), Tensor.input(np.float32(1.0))    # D0 tensors
    bc = lambda c: c.unsqueeze(0).unsqueeze(1).expand(rows, cols)
    y = ((bc(c0) * x + bc(c1)).exp() * x).sum(1)
    z = x.max(0)
    t = x.permute(1, 0).contiguous()
    return x, [y, z, t]


def test_cfg2_kernel_counts_per_fusion_level():
    x, roots = cfg2_graph()
    ref = x.node.data.astype(np.float64)
    want = [(np.exp(0.5 * ref + 1) * ref).sum(1), ref.max(0), ref.T]
    counts = {}
    for fuse in ("none", "reference", "chains"):
        outs, p = run(roots, fuse)
        counts[fuse] = len(p.kernels)
        for o, wv in zip(outs, want):
            np.testing.assert_allclose(o, wv, rtol=2e-5, atol=1e-4)
    # eclat: mul, add, exp as E_ kernels + (mul fused into) R_ (src/lowerer/fusion.rs:28-56), + max + copy
    assert counts == {"none": 7, "reference": 6, "chains": 3}
    _, p = run(roots, "chains")
    y_desc = p.kernel_descs()[0]
    assert y_desc.kclass == D.K_REDUCE and len(y_desc.inputs) == 3
    # operand numbering depends on fusion order; the library renumbers by first use
    from harp_b200.csrc.gen_chains import canonical
    assert canonical(y_desc.map).key() == "mul(exp2(mul(add(mul(w0,w1),w2),c(0x3fb8aa3b))),w1)"


def test_matmul_lowers_to_the_broadcast_product_reduce():
    a = Tensor.input(np.ones((8, 12))); b = Tensor.input(np.ones((12, 16)))
    (c,), p = run([a.matmul(b)])
    assert (c == 12).all()
    (d,) = p.kernel_descs()
    assert d.kclass == D.K_REDUCE and d.shape == [8, 12, 16] and d.reduce_axis == 1
    assert list(d.inputs[0].strides) == [12, 1, 0] and list(d.inputs[1].strides) == [0, 16, 1]


# ---- whole models against an independent implementation (torch, CPU) -----------------------
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("fuse", ["none", "reference", "chains"])
def test_mlp_loss_and_gradients(fuse):
    rng = np.random.default_rng(3)
    X = rng.uniform(-np.pi, np.pi, (64, 1)).astype(np.float32)
    T = np.sin(X.astype(np.float64)).astype(np.float32)
    shapes = [(16, 1), (16,), (16, 16), (16,), (1, 16), (1,)]
    vals = [(rng.standard_normal(s) * 0.5).astype(np.float32) for s in shapes]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    x, t = Tensor.input(X), Tensor.input(T)
    h = x.linear(ps[0], ps[1]).tanh().linear(ps[2], ps[3]).tanh().linear(ps[4], ps[5])
    d = h - t
    loss = (d * d).sum() * (1.0 / 64)
    grads = loss.backward(ps)
    outs, _ = run([loss] + grads, fuse)
    tp = [torch.tensor(v, requires_grad=True) for v in vals]
    th = torch.tanh(torch.tanh(torch.tensor(X) @ tp[0].T + tp[1]) @ tp[2].T + tp[3]) @ tp[4].T + tp[5]
    tl = ((th - torch.tensor(T)) ** 2).mean()
    tl.backward()
    assert abs(float(outs[0]) - tl.item()) <= 1e-5 * abs(tl.item())
    for o, q in zip(outs[1:], tp):
        np.testing.assert_allclose(o, q.grad.numpy(), rtol=2e-4, atol=2e-6)


def test_cnn_loss_and_gradients():
    import torch.nn.functional as TF
    rng = np.random.default_rng(4)
    N = 3
    X = rng.uniform(0, 1, (N, 1, 12, 12)).astype(np.float32)
    vals = [(rng.standard_normal((4, 1, 3, 3)) * 0.3).astype(np.float32), np.full(4, 0.1, np.float32),
            (rng.standard_normal((6, 4, 3, 3)) * 0.2).astype(np.float32), np.zeros(6, np.float32),
            (rng.standard_normal((5, 6)) * 0.2).astype(np.float32), np.zeros(5, np.float32)]
    lab = rng.integers(0, 5, N)
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    h = Tensor.input(X).conv2d(ps[0], ps[1]).relu().max_pool2d(2)       # [N,4,5,5]
    h = h.conv2d(ps[2], ps[3]).relu().max_pool2d(2)                      # [N,6,1,1]
    logits = h.reshape(N, 6).linear(ps[4], ps[5])
    loss = -(logits.log_softmax(1) * Tensor.input(np.eye(5, dtype=np.float32)[lab])).sum() * (1.0 / N)
    grads = loss.backward(ps)
    outs, p = run([loss] + grads)
    tp = [torch.tensor(v, requires_grad=True) for v in vals]
    th = TF.max_pool2d(TF.relu(TF.conv2d(torch.tensor(X), tp[0], tp[1])), 2)
    th = TF.max_pool2d(TF.relu(TF.conv2d(th, tp[2], tp[3])), 2)
    tl = TF.cross_entropy(th.reshape(N, 6) @ tp[4].T + tp[5], torch.tensor(lab))
    tl.backward()
    assert abs(float(outs[0]) - tl.item()) <= 1e-5
    for o, q in zip(outs[1:], tp):
        np.testing.assert_allclose(o, q.grad.numpy(), rtol=2e-4, atol=2e-6)
    kinds = {d.kclass for d in p.kernel_descs()}
    assert {D.K_ELEMENTWISE, D.K_REDUCE, D.K_COPY, D.K_SCATTER} <= kinds


def test_sgd_step_updates_parameters_in_place():
    w0 = np.array([1.0, -2.0, 3.0], np.float32)
    wt = Tensor.input(w0, requires_grad=True)
    loss = (wt * wt).sum()
    (g,) = loss.backward([wt])
    p = Program([loss], OracleExecutor(), sgd=[(wt, g)], lr=0.1)
    p.run()
    assert np.allclose(p.ex.download(p.buffer_of(wt), 3), w0 - np.float32(0.1) * (2 * w0))
    p.run()
    assert np.allclose(p.ex.download(p.buffer_of(wt), 3), w0 * 0.8 * 0.8, rtol=1e-6)


def test_flat_parameter_and_gradient_buffers_change_nothing():
    from harp_b200 import workloads as W
    res = []
    for flat in (False, True):
        loss, ps, grads, _ = W.cnn_graph(2)
        p = Program([loss], OracleExecutor(), sgd=list(zip(ps, grads)), lr=0.05, persistent=True, flat=flat)
        for _ in range(2):
            p.run()
        res.append((float(p.fetch(loss)), [p.fetch(q).copy() for q in ps], len(p.sgd_kernels), len(p.grad_buffers())))
    assert res[0][0] == res[1][0] and res[0][2] == 8 and res[1][2] == 1 and res[1][3] == 1
    for a, b in zip(res[0][1], res[1][1]):
        assert (a == b).all()
