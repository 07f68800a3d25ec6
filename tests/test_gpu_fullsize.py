"""Parity at the sizes the benchmark configurations are quoted on.

config 5: 8192^3 and 64 x [1024^2] contractions, TF32 and 3xTF32, on sampled rows
          against float64 and against the oracle's C triple loop (both fma forms);
config 3: one MLP step at batch 65536 / hidden 256 (loss + six gradients) against
          the OpenMP oracle program and float64;
config 4: EVERY kernel of the CNN step at batch 4096, one by one, against the
          oracle's loop nest for the same descriptor on the same inputs (sampled
          images for the convolutions' forward / input-gradient forms), and the
          whole step at the 8-GPU shard size (512 images) against the oracle;
plus the models as eclat's own Tensor API would build them (full-size ones /
zeros operands, sigmoid-1 "tanh", sum losses), GPU against oracle.

Tolerances: TF32 1e-2, 3xTF32 and f32 sums 1e-5, both times the sum of the
magnitudes of the terms of each output (an order-independent bound); maps with
transcendentals 1e-5 relative; copies, selects and max bit-exact."""
import numpy as np
import pytest

from harp_b200 import desc as D
from harp_b200 import workloads as W
from harp_b200.backend import B200BackendRegistry
from harp_b200.desc import Ast
from harp_b200.frontend import B200Executor, Program
from oracle import c_emit as O
from oracle.executor import OracleExecutor

pytestmark = pytest.mark.gpu
w = Ast.w
TOL = {D.GEMM_TF32: 1e-2, D.GEMM_3XTF32: 1e-5}


def _gemm_on_gpu(dev, k, a, b):
    reg = B200BackendRegistry()
    ba, bb = reg.allocate_buffer(dev, [a.size]), reg.allocate_buffer(dev, [b.size])
    ba.write_vec(a.reshape(-1)); bb.write_vec(b.reshape(-1))
    bo = reg.allocate_buffer(dev, [int(k.output.numel)])
    kern = reg.compile_ast(dev, k)
    kern.execute([ba, bb], [bo])
    out = bo.read_vec()
    for x in (ba, bb, bo):
        x.release()
    return out, kern


def test_cfg5_full_size_8192_cubed(dev):
    n = 8192
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    rows = np.sort(np.random.default_rng(55).choice(n, 64, replace=False))
    a_s = np.ascontiguousarray(a[rows])
    exact = a_s.astype(np.float64) @ b.astype(np.float64)
    mag = np.abs(a_s).astype(np.float64) @ np.abs(b).astype(np.float64)        # sum |a||b| per output
    # the reference's own loop nest on the sampled rows: an M = 64 descriptor of the same form
    small = W.matmul_desc(64, n, n)
    cpu = {fma: O.run(small, [a_s, b], openmp=True, fma=fma).reshape(64, n).astype(np.float64) for fma in (False, True)}
    for fma in (False, True):      # the oracle itself against float64 (f32 accumulation over K = 8192)
        assert (np.abs(cpu[fma] - exact) <= 1e-5 * mag).all()
    for mode in (D.GEMM_TF32, D.GEMM_3XTF32):
        c, kern = _gemm_on_gpu(dev, W.matmul_desc(n, n, n, mode=mode), a, b)
        assert kern.impl.startswith("gemm_tcgen05"), kern.impl
        got = c.reshape(n, n)[rows].astype(np.float64)
        assert (np.abs(got - exact) <= TOL[mode] * mag).all(), (mode, float((np.abs(got - exact) / mag).max()))
        for fma in (False, True):
            assert (np.abs(got - cpu[fma]) <= TOL[mode] * mag).all(), (mode, fma)
        # linearity in A as a size-independent check of the rows nobody sampled: C(2A) == 2 C(A) exactly
        if mode == D.GEMM_3XTF32:
            c2, _ = _gemm_on_gpu(dev, W.matmul_desc(n, n, n, mode=mode), a * 2.0, b)
            assert (c2 == 2.0 * c).all()


def test_cfg5_full_size_batched_64x1024(dev):
    bs, n = 64, 1024
    rng = np.random.default_rng(6)
    a = rng.uniform(-1, 1, (bs, n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (bs, n, n)).astype(np.float32)
    rows = np.sort(np.random.default_rng(66).choice(n, 8, replace=False))       # 8 rows of every batch: 512 rows in all
    a_s = np.ascontiguousarray(a[:, rows, :])
    exact = np.einsum("bmk,bkn->bmn", a_s.astype(np.float64), b.astype(np.float64))
    mag = np.einsum("bmk,bkn->bmn", np.abs(a_s).astype(np.float64), np.abs(b).astype(np.float64))
    small = W.matmul_desc(8, n, n, batch=bs)
    cpu = {fma: O.run(small, [a_s, b], openmp=True, fma=fma).reshape(bs, 8, n).astype(np.float64) for fma in (False, True)}
    for mode in (D.GEMM_TF32, D.GEMM_3XTF32):
        c, kern = _gemm_on_gpu(dev, W.matmul_desc(n, n, n, batch=bs, mode=mode), a, b)
        assert kern.impl.startswith("gemm_tcgen05"), kern.impl
        got = c.reshape(bs, n, n)[:, rows, :].astype(np.float64)
        assert (np.abs(got - exact) <= TOL[mode] * mag).all(), mode
        for fma in (False, True):
            assert (np.abs(got - cpu[fma]) <= TOL[mode] * mag).all(), (mode, fma)


def _mlp_f64(vals, X, T):
    """Loss and gradients of the 1-256-256-1 tanh MLP in float64 (mean squared error)."""
    W1, b1, W2, b2, W3, b3 = [v.astype(np.float64) for v in vals]
    X, T = X.astype(np.float64), T.astype(np.float64)
    h1 = np.tanh(X @ W1.T + b1); h2 = np.tanh(h1 @ W2.T + b2); y = h2 @ W3.T + b3
    d = y - T
    n = X.shape[0]
    loss = (d * d).sum() / n
    gy = 2.0 * d / n
    gW3, gb3 = gy.T @ h2, gy.sum(0)
    g2 = (gy @ W3) * (1 - h2 * h2)
    gW2, gb2 = g2.T @ h1, g2.sum(0)
    g1 = (g2 @ W2) * (1 - h1 * h1)
    gW1, gb1 = g1.T @ X, g1.sum(0)
    return loss, [gW1, gb1, gW2, gb2, gW3, gb3]


def test_cfg3_full_size_step(dev, registry):
    outs = []
    for ex, fuse in ((B200Executor(dev, registry), "chains"), (OracleExecutor(openmp=True), "reference")):
        loss, ps, grads, (x, t) = W.mlp_graph(65536, 256)
        p = Program([loss] + grads, ex, fuse=fuse)
        p.run()
        outs.append([np.array(p.fetch(r), np.float64) for r in [loss] + grads])
        if fuse == "chains":
            assert all(k.specialised for _, _, k, _ in p.kernels), [k.impl for _, _, k, _ in p.kernels if not k.specialised]
            vals = [p_.node.data for p_ in ps]
            X, T = x.node.data, t.node.data
        del p
    g, o = outs
    loss64, grads64 = _mlp_f64(vals, X, T)
    assert abs(g[0] - o[0]) <= 1e-5 * abs(o[0]) and abs(g[0] - loss64) <= 1e-5 * abs(loss64)
    for a, b, e in zip(g[1:], o[1:], grads64):
        scale = np.abs(e).max() + 1e-12
        # sums over 65536 samples: both sides within 1e-4 of the largest gradient entry of the exact result, and of each other
        assert np.abs(a.reshape(e.shape) - e).max() <= 1e-4 * scale, (np.abs(a.reshape(e.shape) - e).max(), scale)
        assert np.abs(b.reshape(e.shape) - e).max() <= 1e-4 * scale
        assert np.abs(a - b).max() <= 2e-4 * scale


def _abs_inputs(arrs):
    return [np.abs(a) for a in arrs]


def _oracle(d, ins, base):
    """The oracle's loop nest for `d`; elements the kernel does not write keep `base`
    (outputs may be slices of a larger buffer, e.g. the flat gradient buffer)."""
    return O.OracleKernel(d, openmp=True)(ins, base.copy())


def _check_kernel_against_oracle(d, ins, got, what):
    """One lowered kernel, GPU result `got` against the oracle on the same inputs."""
    zeros = np.zeros_like(got)
    if d.kclass == D.K_COPY or (d.kclass == D.K_ELEMENTWISE and set(_ops(d.map)) <= {"w", "const", "max", "lt", "select"}):
        assert got.tobytes() == _oracle(d, ins, got).tobytes(), what
        return "exact"
    if d.kclass == D.K_ELEMENTWISE:
        ref = _oracle(d, ins, got)
        assert np.allclose(got, ref, rtol=1e-5, atol=2e-6), (what, float(np.abs(got - ref).max()))
        return "1e-5"
    if d.kclass == D.K_REDUCE and d.reduce_op in (D.R_MAX, D.R_MIN):
        assert got.tobytes() == _oracle(d, ins, got).tobytes(), what
        return "exact"
    if d.kclass == D.K_REDUCE:
        ref = _oracle(d, ins, got)
        mag = _oracle(D.reduce(d.shape, d.inputs, d.map.maximum(-d.map), D.R_SUM, d.reduce_axis, out=d.output), ins, zeros)
        assert (np.abs(got.astype(np.float64) - ref) <= 1e-5 * mag + 1e-30).all(), (what, float(np.abs(got - ref).max()))
        return "1e-5 sum|terms|"
    if d.kclass == D.K_SCATTER:
        ref = O.run(d, ins)
        mag = O.run(d, _abs_inputs(ins))
        assert (np.abs(got.astype(np.float64) - ref) <= 1e-5 * mag + 1e-30).all(), what
        return "1e-5 sum|terms|"
    if d.kclass == D.K_MAXPOOL2D:
        assert got.tobytes() == _oracle(d, ins, got).tobytes(), what
        return "bit-exact"
    if d.kclass == D.K_SOFTMAX_XENT:
        ref = _oracle(d, ins, got)
        assert abs(float(got[0]) - float(ref[0])) <= 1e-5 * abs(float(ref[0])), what
        g, r = got[D.XENT_GRAD_OFFSET:], ref[D.XENT_GRAD_OFFSET:]
        assert np.abs(g - r).max() <= 1e-5 * np.abs(r).max(), what
        return "1e-5"
    raise AssertionError(f"unexpected kernel class {d.kclass} in the CNN step")


def _ops(ast):
    out = [ast.op]
    for a in ast.args:
        out += _ops(a)
    return out


def _check_conv(d, ins, got, what, n_sample=16):
    """The one-kernel convolution forms: forward / input gradient on sampled images (every
    image is independent), weight gradient over the whole batch."""
    n, c, h, w_, co, kh, kw, pad = d.shape
    ho, wo = h + 2 * pad - kh + 1, w_ + 2 * pad - kw + 1
    if d.flags & D.FLAG_WGRAD:
        ref = _oracle(d, ins, got)
        mag = _oracle(d, _abs_inputs(ins), np.zeros_like(got))
        assert (np.abs(got.astype(np.float64) - ref) <= 1e-5 * mag + 1e-30).all(), (what, float(np.abs(got - ref).max()))
        return
    pick = np.random.default_rng(n).choice(n, n_sample, replace=False)
    pick[:2] = (0, n - 1)                              # always the first and the last image
    pick = np.unique(pick)
    n_sample = len(pick)
    x = ins[0].reshape(n, -1)[pick]
    small = D.KernelDesc(D.K_CONV2D, [n_sample, c, h, w_, co, kh, kw, pad],
                         [D.Operand([0] * 8, 0, D.F32, x.size)] + [D.Operand([0] * 8, 0, D.F32, a.size) for a in ins[1:]],
                         D.Operand([0] * 8, 0, D.F32, n_sample * ho * wo * co), None, gemm_mode=d.gemm_mode, flags=d.flags)
    ref = O.run(small, [x] + list(ins[1:]), openmp=True).reshape(n_sample, -1)
    mag = O.run(small, _abs_inputs([x] + list(ins[1:])), openmp=True).reshape(n_sample, -1)
    sub = got.reshape(n, -1)[pick]
    assert (np.abs(sub.astype(np.float64) - ref) <= 1e-5 * mag + 1e-30).all(), (what, float(np.abs(sub - ref).max()))


@pytest.mark.parametrize("batch", [4096, 512])
def test_cfg4_every_kernel_at_batch_4096(dev, registry, batch):
    """Forward and backward of the CNN at the full batch (and at the 8-GPU shard size); then
    each kernel of the step is re-checked in isolation: its device inputs go through the
    oracle's loop nest for the same descriptor and must reproduce the device output."""
    loss, ps, grads, _ = W.cnn_graph(batch, fused_conv=True)
    prog = Program([loss] + grads, B200Executor(dev, registry), persistent=True)
    prog.run_forward()
    dev.synchronize()
    assert all(k.specialised for _, _, k, _ in prog.kernels), [k.impl for _, _, k, _ in prog.kernels if not k.specialised]
    seen = {}
    for pos, (i, d, kern, srcs) in enumerate(prog.kernels):
        ins = [prog._b(s_).read_vec() for s_ in srcs]
        got = prog.buf[prog.where[i][0]].read_vec()
        what = f"kernel {pos} {d.name} {kern.impl}"
        if d.kclass == D.K_CONV2D:
            _check_conv(d, ins, got, what, n_sample=16 if batch > 512 else 64)
            seen[kern.impl] = "1e-5 sum|terms|"
        else:
            # the oracle addresses whole buffers: inputs and output as the descriptor sees them
            ref_kind = _check_kernel_against_oracle(d, ins, got, what)
            seen[kern.impl] = ref_kind
    assert any(k.startswith("conv2d_igemm") for k in seen) and any(k.startswith("gemm_tcgen05") for k in seen), sorted(seen)
    assert np.isfinite(float(prog.fetch(loss)))


def _cnn_f64(vals, X, onehot):
    """Loss and the eight gradients of the config-4 network in float64 (torch on the CPU)."""
    import torch
    import torch.nn.functional as F
    ps = [torch.tensor(v, dtype=torch.float64, requires_grad=True) for v in vals]
    x, t = torch.tensor(X, dtype=torch.float64), torch.tensor(onehot, dtype=torch.float64)
    n = x.shape[0]
    h = F.max_pool2d(F.relu(F.conv2d(x, ps[0], ps[1])), 2)
    h = F.max_pool2d(F.relu(F.conv2d(h, ps[2], ps[3])), 2)
    h = F.linear(F.relu(F.linear(h.reshape(n, 1600), ps[4], ps[5])), ps[6], ps[7])
    loss = -(F.log_softmax(h, 1) * t).sum() / n
    loss.backward()
    return float(loss.detach()), [p.grad.numpy() for p in ps]


def test_cfg4_step_at_the_8_gpu_shard_size(dev, registry):
    """Loss and all eight gradients at 512 images (what one of 8 GPUs holds of the global
    batch 4096): this backend's one-kernel forms on the GPU against the reference's
    spelling of the same graph on the OpenMP oracle, with float64 as the arbiter.  The
    reference adds the 346 112 terms of a first-layer weight gradient one after the other
    in f32, so ITS distance to the exact result is the larger one; the bounds say so."""
    def run(fused, ex, fuse):
        loss, ps, grads, (x, onehot) = W.cnn_graph(512, fused_conv=fused)
        p = Program([loss] + grads, ex, fuse=fuse)
        p.run()
        return [np.array(p.fetch(t), np.float64) for t in [loss] + grads], ([q.node.data for q in ps], x.node.data, onehot.node.data)
    g, data = run(True, B200Executor(dev, registry), "chains")
    o, _ = run(False, OracleExecutor(openmp=True), "reference")
    loss64, grads64 = _cnn_f64(*data)
    assert abs(g[0] - o[0]) <= 1e-5 * abs(o[0]) and abs(g[0] - loss64) <= 1e-5 * abs(loss64)
    for j, (a, b, e) in enumerate(zip(g[1:], o[1:], grads64)):
        scale = np.abs(e).max() + 1e-12
        # The gradients of the convolutions pass backwards through a max-pool: of the 819 200 pooling
        # windows of this batch a handful hold two candidates that differ by about one f32 rounding, and
        # the 3xTF32 forward and the f32 / f64 forwards then pick different winners, which moves single
        # (large) gradient entries to a neighbouring pixel.  Measured here: 3 windows, up to 4e-3 of the
        # largest entry of a convolution's weight gradient.  Every kernel of this step on its own matches
        # the oracle to 1e-5 on identical inputs (test_cfg4_every_kernel_at_batch_4096[512]); the layers
        # after the last pool see no such discontinuity and get the tight bound.
        tol = 2e-2 if j < 4 else 2e-4
        assert np.abs(a.reshape(e.shape) - e).max() <= tol * scale, ("gpu", j, np.abs(a.reshape(e.shape) - e).max(), scale)
        assert np.abs(b.reshape(e.shape) - e).max() <= tol * scale, ("oracle", j, np.abs(b.reshape(e.shape) - e).max(), scale)
        assert np.abs(a - b).max() <= tol * scale, ("gpu vs oracle", j, np.abs(a - b).max(), scale)


def test_models_as_the_reference_tensor_api_builds_them(dev, registry):
    """Reference-faithful graphs (labelled as such): full-size `ones` / `zeros` operands as
    real buffers, tanh = sigmoid - 1, sum losses, exp's gradient = 2^x.  The kernel list is
    the one eclat would hand the backend (fusion level "reference": one kernel per
    arithmetic node, only the last elementwise node folded into a reduce) on the GPU,
    against the same list on the oracle."""
    for build, sizes in ((W.mlp_graph_reference, (512, 64)), (W.cnn_graph_reference, (8,))):
        outs = []
        for ex in (B200Executor(dev, registry), OracleExecutor()):
            loss, ps, grads, _ = build(*sizes)
            p = Program([loss] + grads, ex, fuse="reference")
            p.run()
            outs.append([np.array(p.fetch(t), np.float64) for t in [loss] + grads])
            if isinstance(ex, B200Executor):
                descs = p.kernel_descs()
                # binary elementwise kernels whose second operand is a full-size constant buffer exist and ran
                assert any(d.kclass == D.K_ELEMENTWISE and len(d.inputs) == 2 and all(o_.numel == d.iter_numel() and d.iter_numel() > 1
                           for o_ in d.inputs) for d in descs)
        g, o = outs
        assert abs(g[0] - o[0]) <= 1e-5 * abs(o[0]), (g[0], o[0])
        for a, b in zip(g[1:], o[1:]):
            scale = np.abs(b).max() + 1e-12
            assert np.abs(a - b).max() <= 2e-4 * scale, (build.__name__, np.abs(a - b).max(), scale)
