"""Kernel descriptors and seeded inputs of the benchmark configurations.

Each function returns what eclat's lowerer would hand the backend for that
configuration (with this backend's elementwise-chain fusion applied), plus the
synthetic inputs: numpy ``default_rng(seed)`` tensors with the shapes and value
distributions the configuration names.
"""
from __future__ import annotations

import numpy as np

from . import desc as D
from .desc import Ast

w = Ast.w


# ---- config 2: fused elementwise + reduce, column max, transposing copy --------

def cfg2_input(rows: int = 8192, cols: int = 8192, seed: int = 2) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((rows, cols), dtype=np.float32)


def cfg2_y(rows: int = 8192, cols: int = 8192) -> D.KernelDesc:
    """y = sum(exp(c0*x + c1) * x, axis=1).  The constants are D0 tensors
    broadcast with stride 0 (the Tensor API has no scalar literal:
    src/tensor/ops.rs:699-707).  The reference would run mul, add, exp as three
    E_ kernels and fuse only the last mul into the R_ kernel
    (src/lowerer/fusion.rs:28-56); here the whole chain is one map."""
    scalar = D.Operand([0, 0], 0, D.F32, 1)
    expr = ((w(0) * w(1)) + w(2)).exp() * w(1)
    return D.reduce([rows, cols], [scalar, D.contiguous([rows, cols]), scalar], expr, D.R_SUM, 1)


def cfg2_z(rows: int = 8192, cols: int = 8192) -> D.KernelDesc:
    """z = max(x, axis=0): kept axis outside, reduce axis innermost in the
    reference's loop nest (src/lowerer/loop_gen.rs:87-151)."""
    return D.reduce([rows, cols], [D.contiguous([rows, cols])], w(0), D.R_MAX, 0)


def cfg2_t(rows: int = 8192, cols: int = 8192) -> D.KernelDesc:
    """t = x.permute(1,0).contiguous(): identity-map E_ kernel over the permuted
    view (src/graph/node.rs:431-445); out[c][r] = x[r][c]."""
    src = D.Operand([1, cols], 0, D.F32, rows * cols)
    return D.elementwise([cols, rows], [src], w(0))


FLAG_SIBLINGS = 16384


def cfg2_siblings(rows: int = 8192, cols: int = 8192) -> D.KernelDesc:
    """y, z and t of config 2 from ONE pass over x (sibling fusion, descriptor flag bit 14): the
    row-sum descriptor of `cfg2_y` whose output buffer also receives z = max(x, axis 0) and
    t = x transposed: [y (rows) | z (cols) | t (cols * rows)], y and z padded to multiples of 64."""
    k = cfg2_y(rows, cols)
    pad = lambda v: (v + 63) // 64 * 64
    k.output = D.Operand([1, 0], 0, D.F32, pad(rows) + pad(cols) + rows * cols)
    k.flags = FLAG_SIBLINGS
    return k


def cfg2_consts():
    return np.array([0.5], np.float32), np.array([1.0], np.float32)


# ---- configs 1 and 5: dense contraction spelled as broadcast-mul + sum ----------

def matmul_desc(m: int, k: int, n: int, batch: int = 0, mode: int = D.GEMM_DEFAULT) -> D.KernelDesc:
    """C = A.B as examples/matmul_demo.rs:43-60 builds it: A [M,K] -> [M,K,1],
    B [K,N] -> [1,K,N], expand to [M,K,N], multiply, sum over axis 1."""
    if batch:
        a = D.Operand([m * k, k, 1, 0], 0, D.F32, batch * m * k)
        b = D.Operand([k * n, 0, n, 1], 0, D.F32, batch * k * n)
        return D.reduce([batch, m, k, n], [a, b], w(0) * w(1), D.R_SUM, 2, gemm_mode=mode)
    a = D.Operand([k, 1, 0], 0, D.F32, m * k)
    b = D.Operand([0, n, 1], 0, D.F32, k * n)
    return D.reduce([m, k, n], [a, b], w(0) * w(1), D.R_SUM, 1, gemm_mode=mode)


def linear_desc(batch: int, in_f: int, out_f: int, mode: int = D.GEMM_DEFAULT) -> D.KernelDesc:
    """x [B,I] . W[O,I]^T as functional::linear builds it
    (crates/nn/src/functional/linear.rs:27-56): [B,1,I] * [1,O,I] summed over axis 2."""
    x = D.Operand([in_f, 0, 1], 0, D.F32, batch * in_f)
    wt = D.Operand([0, in_f, 1], 0, D.F32, out_f * in_f)
    return D.reduce([batch, out_f, in_f], [x, wt], w(0) * w(1), D.R_SUM, 2, gemm_mode=mode)


def uniform_pm1(shape, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).uniform(-1.0, 1.0, shape).astype(np.float32)


# ---- configs 3 and 4: training steps built through the graph front end ---------------

def mlp_graph(batch: int = 65536, hidden: int = 256, seed: int = 3, weight_seed: int = 30):
    """Config 3: 1 -> hidden -> hidden -> 1 with tanh, inputs uniform[-pi, pi],
    target sin(x), Xavier-uniform weights, zero biases, MSE loss.  Returns
    (loss, parameters, gradients, inputs) as lazy tensors."""
    from .frontend import Tensor
    rng = np.random.default_rng(seed)
    X = rng.uniform(-np.pi, np.pi, (batch, 1)).astype(np.float32)
    T = np.sin(X.astype(np.float64)).astype(np.float32)
    prng = np.random.default_rng(weight_seed)

    def xavier(o, i):
        b = np.sqrt(6.0 / (i + o))
        return prng.uniform(-b, b, (o, i)).astype(np.float32)
    vals = [xavier(hidden, 1), np.zeros(hidden, np.float32), xavier(hidden, hidden), np.zeros(hidden, np.float32),
            xavier(1, hidden), np.zeros(1, np.float32)]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    x, t = Tensor.input(X), Tensor.input(T)
    h = x.linear(ps[0], ps[1]).tanh().linear(ps[2], ps[3]).tanh().linear(ps[4], ps[5])
    d = h - t
    loss = (d * d).sum() * (1.0 / batch)
    return loss, ps, loss.backward(ps), (x, t)


def cnn_graph(n: int = 4096, seed: int = 4, label_seed: int = 40, weight_seed: int = 41, fused_conv: bool = False,
              fused_pool=None):
    """Config 4: MNIST-shaped CNN (conv 1->32 3x3, ReLU, maxpool 2, conv 32->64 3x3,
    ReLU, maxpool 2, flatten 1600, linear 128, ReLU, linear 10, softmax
    cross-entropy) on synthetic images uniform[0,1] and uniform labels; `fused_conv`
    selects this backend's forms of the same functions (one implicit-GEMM kernel per
    convolution and per input gradient; ReLU + max-pool as one kernel each way, or with
    ``fused_pool=False`` as elementwise kernels over strided views) instead of the
    reference's spelling; Kaiming
    normal weights from `weight_seed` (the reference's deterministic sin() init is
    not used), zero biases."""
    from .frontend import Tensor
    X = np.random.default_rng(seed).uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    lab = np.random.default_rng(label_seed).integers(0, 10, n)
    prng = np.random.default_rng(weight_seed)

    def kaiming(*shape):
        fan_in = int(np.prod(shape[1:]))
        return (prng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    vals = [kaiming(32, 1, 3, 3), np.zeros(32, np.float32), kaiming(64, 32, 3, 3), np.zeros(64, np.float32),
            kaiming(128, 1600), np.zeros(128, np.float32), kaiming(10, 128), np.zeros(10, np.float32)]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    x = Tensor.input(X)
    onehot = Tensor.input(np.eye(10, dtype=np.float32)[lab])       # built on the host, as loss.rs:43-51 does
    if fused_pool is None:
        fused_pool = fused_conv
    if fused_conv and fused_pool:   # each convolution (and its input gradient) as one implicit-GEMM kernel, ReLU + pool as one
        h = x.conv2d_fused(ps[0], ps[1]).max_pool2d_fused(2, relu=True)
        h = h.conv2d_fused(ps[2], ps[3]).max_pool2d_fused(2, relu=True)
    elif fused_conv:
        h = x.conv2d_fused(ps[0], ps[1]).relu().max_pool2d(2)
        h = h.conv2d_fused(ps[2], ps[3]).relu().max_pool2d(2)
    else:               # the reference's spelling: pad, unfold, permute, contiguous, GEMM, bias; pools through unfold/fold
        h = x.conv2d(ps[0], ps[1]).relu().max_pool2d_unfold(2)
        h = h.conv2d(ps[2], ps[3]).relu().max_pool2d_unfold(2)
    h = h.reshape(n, 1600).linear(ps[4], ps[5]).relu().linear(ps[6], ps[7])
    if fused_conv:      # log-softmax + cross-entropy, loss and logits gradient, as one kernel
        loss = h.softmax_cross_entropy(onehot, -1.0 / n)
    else:
        loss = -(h.log_softmax(1) * onehot).sum() * (1.0 / n)
    return loss, ps, loss.backward(ps), (x, onehot)


# ---- the same models as eclat's own Tensor API would build them --------------------------

def mlp_graph_reference(batch: int = 512, hidden: int = 64, seed: int = 3, weight_seed: int = 30):
    """Config 3 with the reference's graph-level behaviours kept: `tanh` evaluates
    sigmoid(x) - 1 because Tensor::scale ignores its factor
    (crates/nn/src/functional/activation.rs:70-76, src/tensor/ops.rs:699-707), the
    constants are full-size `ones` input buffers (src/tensor/realize.rs:391-502),
    exp's gradient is 2^x (src/grad/rules.rs:254-259), and the loss is the SUM of
    squared errors (`mean` returns the sum, src/tensor/ops.rs:230-245)."""
    from .frontend import Tensor
    rng = np.random.default_rng(seed)
    X = rng.uniform(-np.pi, np.pi, (batch, 1)).astype(np.float32)
    T = np.sin(X.astype(np.float64)).astype(np.float32)
    prng = np.random.default_rng(weight_seed)

    def xavier(o, i):
        b = np.sqrt(6.0 / (i + o))
        return prng.uniform(-b, b, (o, i)).astype(np.float32)
    vals = [xavier(hidden, 1), np.zeros(hidden, np.float32), xavier(hidden, hidden), np.zeros(hidden, np.float32),
            xavier(1, hidden), np.zeros(1, np.float32)]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    x, t = Tensor.input(X), Tensor.input(T)
    h = x.linear(ps[0], ps[1]).tanh_ref().linear(ps[2], ps[3]).tanh_ref().linear(ps[4], ps[5])
    d = h - t
    loss = (d * d).sum()
    return loss, ps, loss.backward(ps), (x, t)


def cnn_graph_reference(n: int = 8, seed: int = 4, label_seed: int = 40, weight_seed: int = 41):
    """Config 4 as eclat spells it, graph-level behaviours kept: ReLU against a
    full-size `zeros` input buffer (crates/nn/src/functional/activation.rs:18-21),
    convolutions and pools through unfold / fold, and cross_entropy_loss returning
    +sum(one_hot * log_softmax) because its final scale(-1/N) multiplies by ones
    (crates/nn/src/functional/loss.rs:32-65)."""
    from .frontend import Tensor
    X = np.random.default_rng(seed).uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    lab = np.random.default_rng(label_seed).integers(0, 10, n)
    prng = np.random.default_rng(weight_seed)

    def kaiming(*shape):
        fan_in = int(np.prod(shape[1:]))
        return (prng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    vals = [kaiming(32, 1, 3, 3), np.zeros(32, np.float32), kaiming(64, 32, 3, 3), np.zeros(64, np.float32),
            kaiming(128, 1600), np.zeros(128, np.float32), kaiming(10, 128), np.zeros(10, np.float32)]
    ps = [Tensor.input(v, requires_grad=True) for v in vals]
    x = Tensor.input(X)
    onehot = Tensor.input(np.eye(10, dtype=np.float32)[lab])
    h = x.conv2d(ps[0], ps[1]).relu_ref().max_pool2d_unfold(2)
    h = h.conv2d(ps[2], ps[3]).relu_ref().max_pool2d_unfold(2)
    h = h.reshape(n, 1600).linear(ps[4], ps[5]).relu_ref().linear(ps[6], ps[7])
    loss = (h.log_softmax(1) * onehot).sum().scale_ref(-1.0 / n)
    return loss, ps, loss.backward(ps), (x, onehot)
