"""Map expressions that get an ahead-of-time compiled functor.

The reference emits one kernel per arithmetic graph node
(src/lowerer/fusion.rs:28-56); this backend first composes consecutive
elementwise nodes into one map (``harp_b200.frontend`` fusion) and then runs the
composed map either as one of the functors listed here or, for any other
expression, through the device-side bytecode interpreter.  Listing a chain is
purely a speed matter: results are the same either way.

Entries are matched by structure; constant values are launch parameters.
"""
from harp_b200.desc import Ast

w = Ast.w
c = Ast.const


def _sigmoid(x):
    # crates/nn/src/functional/activation.rs:50-58: 1 / (1 + exp(-x))
    return ((-x).exp() + c(1.0)).recip()


CHAINS = [
    # primitives, as single graph nodes produce them (src/graph/ops.rs)
    ("identity", w(0)),
    ("add", w(0) + w(1)),
    ("mul", w(0) * w(1)),
    ("sub", w(0) - w(1)),
    ("div", w(0) / w(1)),
    ("max", w(0).maximum(w(1))),
    ("neg", -w(0)),
    ("recip", w(0).recip()),
    ("sqrt", w(0).sqrt()),
    ("exp2", w(0).exp2()),
    ("log2", w(0).log2()),
    ("sin", w(0).sin()),
    ("exp", w(0).exp()),
    ("ln", w(0).ln()),
    ("cos", w(0).cos()),
    ("square", w(0) * w(0)),
    ("lt", w(0).lt(w(1))),
    ("select", Ast.select(w(0), w(1), w(2))),
    # scalar-constant forms (a constant folded into the map)
    ("mul_const", w(0) * c(2.0)),
    ("add_const", w(0) + c(1.0)),
    ("max_const", w(0).maximum(c(0.0))),
    ("axpb", w(0) * c(0.5) + c(1.0)),
    # config 2: sum(exp(c0*x + c1) * x), constants as tensors or folded
    ("cfg2_tensor_consts", ((w(0) * w(1)) + w(2)).exp() * w(1)),
    ("cfg2_folded", ((w(0) * c(0.5)) + c(1.0)).exp() * w(0)),
    # dense contraction body (GEMM-as-reduce) and squared error
    ("sq_diff", (w(0) - w(1)) * (w(0) - w(1))),
    # activations
    ("sigmoid", _sigmoid(w(0))),
    ("tanh_ref", _sigmoid(w(0) * w(1)) * w(2) - w(3)),
    ("relu_zeros", w(0).maximum(w(1))),
    ("bias_relu", (w(0) + w(1)).maximum(c(0.0))),
    ("bias_relu_zeros", (w(0) + w(1)).maximum(w(2))),
    ("fma3", w(0) * w(1) + w(2)),
    # softmax / cross-entropy pieces
    ("sub_exp", (w(0) - w(1)).exp()),
    ("sub_sub_ln", (w(0) - w(1)) - w(2).ln()),
    ("mul_neg", -(w(0) * w(1))),
]


def _model_chains():
    """Every elementwise / reduce map the fused training steps of configs 3 and 4
    lower to, so those steps never fall back to the bytecode interpreter."""
    from . import desc as D
    from . import workloads as W
    from .frontend import Program

    class _Null:           # lowers without a device
        def alloc(self, n): return None
        def free(self, b): pass
        def upload(self, b, d): pass
        def compile(self, d): return None

    out = []
    for tag, (loss, ps, grads, _) in (("mlp", W.mlp_graph(8, 8)), ("cnn", W.cnn_graph(2)), ("cnnf", W.cnn_graph(2, fused_conv=True, fused_pool=False)), ("cnnp", W.cnn_graph(2, fused_conv=True))):
        prog = Program([loss], _Null(), fuse="chains", sgd=list(zip(ps, grads)), lr=0.1)
        for i, d in enumerate(prog.kernel_descs()):
            if d.map is None or d.kclass not in (D.K_ELEMENTWISE, D.K_REDUCE):
                continue
            # one-element operands reach the kernels as launch-time constants
            sub = {}
            for j, op in enumerate(d.inputs):
                if not op.bounds and all(st == 0 or ext == 1 for st, ext in zip(op.strides, d.shape)):
                    sub[j] = Ast.const(1000003.0 + j)     # a distinct stand-in per operand (equal constants share a slot)
            out.append((f"{tag}_{i}", d.map.substitute(sub)))
    return out


CHAINS = CHAINS + _model_chains()
