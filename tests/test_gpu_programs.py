"""Whole graphs on the B200 against the same graphs on the CPU oracle: the
front end lowers one kernel list, the CUDA library runs this backend's fused
form of it and the oracle runs eclat's form (fusion level "reference")."""
import numpy as np
import pytest

from harp_b200 import desc as D
from harp_b200.frontend import B200Executor, Program, Tensor
from oracle.executor import OracleExecutor

pytestmark = pytest.mark.gpu


def both(build, dev, registry):
    """build() -> (roots, extra); run on GPU (chains) and oracle (reference)."""
    roots, _ = build()
    pg = Program(roots, B200Executor(dev, registry), fuse="chains")
    pg.run()
    g = [pg.fetch(r) for r in roots]
    roots2, _ = build()
    po = Program(roots2, OracleExecutor(), fuse="reference")
    po.run()
    o = [po.fetch(r) for r in roots2]
    return g, o, pg, po


def test_ref_autograd_vectors_on_gpu(dev, registry):
    x = Tensor.input([1, 2, 3, 4], requires_grad=True)
    a = Tensor.input([1, 2, 3, 4], requires_grad=True)
    b = Tensor.input([2, 3, 4, 5], requires_grad=True)
    roots = (x * x).sum().backward([x]) + (a * b).sum().backward([a, b]) + (x + x).sum().backward([x])
    p = Program(roots, B200Executor(dev, registry))
    p.run()
    got = [p.fetch(r).tolist() for r in roots]
    assert got == [[2.0, 4.0, 6.0, 8.0], [2.0, 3.0, 4.0, 5.0], [1.0, 2.0, 3.0, 4.0], [2.0, 2.0, 2.0, 2.0]]


def test_cfg2_graph_through_the_tensor_api(dev, registry):
    def build():
        rows, cols = 512, 1024
        x = Tensor.input(np.random.default_rng(2).standard_normal((rows, cols)))
        c0, c1 = Tensor.input(np.float32(0.5)), Tensor.input(np.float32(1.0))
        bc = lambda c: c.unsqueeze(0).unsqueeze(1).expand(rows, cols)
        return [((bc(c0) * x + bc(c1)).exp() * x).sum(1), x.max(0), x.permute(1, 0).contiguous()], x
    g, o, pg, po = both(build, dev, registry)
    assert len(pg.kernels) == 3 and len(po.kernels) == 6
    assert [k.impl for _, _, k, _ in pg.kernels][2] == "transpose_copy"
    x = build()[1].node.data.astype(np.float64)
    tol = 1e-5 * np.abs(np.exp(0.5 * x + 1) * x).sum(1)
    assert (np.abs(g[0].astype(np.float64) - o[0]) <= tol).all()
    assert (g[1] == o[1]).all() and g[2].tobytes() == o[2].tobytes()


def mlp(batch, hidden, seed=3):
    rng = np.random.default_rng(seed)
    X = rng.uniform(-np.pi, np.pi, (batch, 1)).astype(np.float32)
    T = np.sin(X.astype(np.float64)).astype(np.float32)
    prng = np.random.default_rng(30)

    def xavier(o, i):
        b = np.sqrt(6.0 / (i + o))
        return prng.uniform(-b, b, (o, i)).astype(np.float32)
    vals = [xavier(hidden, 1), np.zeros(hidden, np.float32), xavier(hidden, hidden), np.zeros(hidden, np.float32),
            xavier(1, hidden), np.zeros(1, np.float32)]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    h = Tensor.input(X).linear(ps[0], ps[1]).tanh().linear(ps[2], ps[3]).tanh().linear(ps[4], ps[5])
    d = h - Tensor.input(T)
    loss = (d * d).sum() * (1.0 / batch)
    return loss, ps, loss.backward(ps)


def test_cfg3_mlp_step_matches_oracle(dev, registry):
    def build():
        loss, ps, grads = mlp(512, 64)
        return [loss] + grads, None
    g, o, pg, po = both(build, dev, registry)
    assert len(pg.kernels) < len(po.kernels)
    assert any(k.impl.startswith("gemm") for _, _, k, _ in pg.kernels)
    assert abs(float(g[0]) - float(o[0])) <= 1e-5 * abs(float(o[0]))
    for a, b in zip(g[1:], o[1:]):
        scale = np.abs(b).max() + 1e-12
        assert np.abs(a - b).max() <= 2e-4 * scale, (np.abs(a - b).max(), scale)


def test_cfg3_mlp_training_loss_decreases_and_tracks_oracle(dev, registry):
    runs = []
    for ex, fuse in ((B200Executor(dev, registry), "chains"), (OracleExecutor(), "reference")):
        loss, ps, grads = mlp(256, 32)
        p = Program([loss], ex, fuse=fuse, sgd=list(zip(ps, grads)), lr=0.05)
        hist = []
        for _ in range(20):
            p.run()
            hist.append(float(p.fetch(loss)))
        runs.append(hist)
    gpu, cpu = runs
    assert gpu[-1] < 0.8 * gpu[0]
    np.testing.assert_allclose(gpu, cpu, rtol=2e-3)


def cnn(n, seed=4):
    rng = np.random.default_rng(seed)
    X = rng.uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    lab = np.random.default_rng(40).integers(0, 10, n)
    prng = np.random.default_rng(41)

    def kaiming(*shape):
        fan_in = int(np.prod(shape[1:]))
        return (prng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    vals = [kaiming(32, 1, 3, 3), np.zeros(32, np.float32), kaiming(64, 32, 3, 3), np.zeros(64, np.float32),
            kaiming(128, 1600), np.zeros(128, np.float32), kaiming(10, 128), np.zeros(10, np.float32)]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    h = Tensor.input(X).conv2d(ps[0], ps[1]).relu().max_pool2d_unfold(2)
    h = h.conv2d(ps[2], ps[3]).relu().max_pool2d_unfold(2)
    h = h.reshape(n, 1600).linear(ps[4], ps[5]).relu().linear(ps[6], ps[7])
    onehot = Tensor.input(np.eye(10, dtype=np.float32)[lab])
    loss = -(h.log_softmax(1) * onehot).sum() * (1.0 / n)
    return loss, ps, loss.backward(ps)


def test_cfg4_cnn_step_matches_oracle(dev, registry):
    def build():
        loss, ps, grads = cnn(8)
        return [loss] + grads, None
    g, o, pg, po = both(build, dev, registry)
    impls = {k.impl.split("_v")[0] for _, _, k, _ in pg.kernels}
    assert "scatter_add_as_gather" in impls and any(i.startswith("gemm") for i in impls)
    assert abs(float(g[0]) - float(o[0])) <= 1e-5 * abs(float(o[0]))
    for a, b in zip(g[1:], o[1:]):
        scale = np.abs(b).max() + 1e-12
        assert np.abs(a - b).max() <= 2e-4 * scale, (np.abs(a - b).max(), scale)
    pg.ex.synchronize()


def test_cfg4_cnn_with_one_kernel_convolutions_matches_the_reference_spelling(dev, registry):
    """The CNN step with each convolution, conv2's input gradient and both weight
    gradients as one implicit-GEMM kernel each on the GPU, against the reference's spelling of the same
    graph on the CPU oracle: loss and all eight gradients."""
    from harp_b200 import workloads as W

    def run(fused, ex, fuse):
        loss, ps, grads, _ = W.cnn_graph(8, fused_conv=fused)
        p = Program([loss] + grads, ex, fuse=fuse)
        p.run()
        return [p.fetch(t) for t in [loss] + grads], p
    g, pg = run(True, B200Executor(dev, registry), "chains")
    o, _ = run(False, OracleExecutor(), "reference")
    impls = [k.impl for _, _, k, _ in pg.kernels]
    assert sum(i.startswith("conv2d_") for i in impls) == 5           # conv1 (K = 9) on the streaming f32 kernels, conv2 on tcgen05
    assert sum(i.endswith("_dgrad") for i in impls) == 1 and sum(i.endswith("_wgrad") for i in impls) == 2
    assert not any(d.kclass == D.K_SCATTER and len(d.shape) == 6 and d.shape[-1] == 3 for d in pg.kernel_descs())   # no 3x3 fold left
    assert abs(float(g[0]) - float(o[0])) <= 1e-5 * abs(float(o[0]))
    for a, b in zip(g[1:], o[1:]):
        scale = np.abs(b).max() + 1e-12
        assert np.abs(a - b).max() <= 2e-4 * scale, (np.abs(a - b).max(), scale)
    pg.ex.synchronize()
