"""A small graph front end: eclat's Tensor API for the ops the benchmark configs use.

eclat itself is Rust and cannot run here, so this module reproduces, for exactly
the operations configurations 1-5 need, what sits above the backend boundary:

* lazy tensors over a node DAG with view algebra (``View``; reference
  src/graph/shape/view.rs, src/tensor/ops.rs, src/graph/ops.rs);
* the derived forms the reference spells with primitives (``a-b = a+b*(-1)``,
  ``exp = exp2(x*log2e)``, matmul = unsqueeze/expand/mul/sum:
  crates/nn/src/functional/linear.rs:27-56, conv2d = pad/unfold/permute/
  contiguous/GEMM: crates/nn/src/functional/conv.rs:113-184, max_pool2d =
  unfold + max: crates/nn/src/functional/pool.rs:117-160);
* reverse-mode autograd (the role of src/grad/backward.rs:41-87), written as a
  tape of tensor ops so that gradients are graphs of the same kind;
* lowering of every surviving node to one ``KernelDesc`` -- the information of
  one ``AstNode::Kernel`` (src/lowerer/lower.rs:335-388) -- at three fusion
  levels: ``"none"`` (one kernel per op), ``"reference"`` (what eclat fuses:
  views inlined and the last elementwise node folded into a reduce,
  src/lowerer/fusion.rs:28-128) and ``"chains"`` (this backend's addition:
  whole elementwise chains composed by Wildcard substitution);
* a program runner (the role of execute_graph, src/backend/executor.rs:149-374)
  with liveness-based buffer release, multi-root realize and in-place
  parameter updates, running on any executor that exposes ``alloc / upload /
  compile / download``.

Nothing here computes: kernels run through ``harp_b200.backend`` (the CUDA
library).  The parity tests plug the CPU oracle into the same runner.
"""
from __future__ import annotations

import itertools
import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import desc as D
from .desc import Ast, Bound


# ---------------------------------------------------------------------------------------
# views
# ---------------------------------------------------------------------------------------
class View:
    """Affine view of a flat buffer: index = offset + sum strides[d]*idx[d], valid
    where every bound holds (else ``pad_value``).  Mirrors View::Linear and the
    padded IndexExpr views of the reference for the affine cases."""

    __slots__ = ("shape", "strides", "offset", "bounds", "pad_value")

    def __init__(self, shape, strides, offset=0, bounds=(), pad_value=0.0):
        self.shape = tuple(int(s) for s in shape)
        self.strides = tuple(int(s) for s in strides)
        self.offset = int(offset)
        self.bounds = tuple(bounds)
        self.pad_value = float(pad_value)

    @staticmethod
    def contiguous(shape) -> "View":
        return View(shape, D.contiguous_strides(shape))

    @property
    def ndim(self):
        return len(self.shape)

    def numel(self):
        return math.prod(self.shape) if self.shape else 1

    def is_contiguous(self) -> bool:
        return (not self.bounds and self.offset == 0 and
                all(s == 1 or st == c for s, st, c in zip(self.shape, self.strides, D.contiguous_strides(self.shape))))

    def _remap_bounds(self, fn):
        return tuple(Bound(fn(list(b.coef)), b.c, b.lo, b.hi) for b in self.bounds)

    def permute(self, axes) -> "View":
        axes = list(axes)
        return View([self.shape[a] for a in axes], [self.strides[a] for a in axes], self.offset,
                    self._remap_bounds(lambda c: [c[a] for a in axes]), self.pad_value)

    def unsqueeze(self, dim) -> "View":
        # a new size-1 axis gets stride 0 (src/graph/shape/view.rs:1556-1674)
        sh, st = list(self.shape), list(self.strides)
        sh.insert(dim, 1); st.insert(dim, 0)
        return View(sh, st, self.offset, self._remap_bounds(lambda c: c[:dim] + [0] + c[dim:]), self.pad_value)

    def squeeze(self, dim) -> "View":
        assert self.shape[dim] == 1
        sh, st = list(self.shape), list(self.strides)
        del sh[dim]; del st[dim]
        return View(sh, st, self.offset, self._remap_bounds(lambda c: c[:dim] + c[dim + 1:]), self.pad_value)

    def expand(self, shape) -> "View":
        assert len(shape) == self.ndim, f"expand keeps the rank: {self.shape} -> {tuple(shape)}"
        st = list(self.strides)
        for d, (old, new) in enumerate(zip(self.shape, shape)):
            if old != new:
                assert old == 1, f"cannot expand {self.shape} to {tuple(shape)}"
                st[d] = 0     # this front end always broadcasts with stride 0
        return View(shape, st, self.offset, self.bounds, self.pad_value)

    def reshape(self, shape) -> Optional["View"]:
        """Reshape without a copy: only for contiguous, unmasked views."""
        if self.bounds or math.prod(shape) != self.numel():
            return None
        if all(s == 1 or st == c for s, st, c in zip(self.shape, self.strides, D.contiguous_strides(self.shape))):
            return View(shape, D.contiguous_strides(shape), self.offset)
        return None

    def pad(self, pads: Sequence[Tuple[int, int]], value=0.0) -> "View":
        """View::padded (src/graph/shape/view.rs:980-1054): shape grows, index
        shifts by -before, one bound pair per axis (kept even when before=after=0,
        as the reference does)."""
        shape, offset, bounds = [], self.offset, list(self.bounds)
        shifted = []
        for b in bounds:   # existing bounds see idx - before
            shifted.append(Bound(list(b.coef), b.c - sum(k * p[0] for k, p in zip(b.coef, pads)), b.lo, b.hi))
        for d, ((before, after), s, st) in enumerate(zip(pads, self.shape, self.strides)):
            shape.append(s + before + after)
            offset -= before * st
            coef = [0] * self.ndim
            coef[d] = 1
            shifted.append(Bound(coef, 0, before, before + s))
        return View(shape, self.strides, offset, shifted, value)

    def unfold(self, axes, sizes, strides, dilations) -> "View":
        """Sliding windows (src/graph/shape/view.rs:1162-1381): output dims are
        [preserved..., window positions..., window offsets...]."""
        axes = list(axes)
        keep = [d for d in range(self.ndim) if d not in axes]
        n_pos = [(self.shape[a] - d * (k - 1) - 1) // s + 1 for a, k, s, d in zip(axes, sizes, strides, dilations)]
        shape = [self.shape[d] for d in keep] + n_pos + list(sizes)
        st = [self.strides[d] for d in keep] + [self.strides[a] * s for a, s in zip(axes, strides)] + \
             [self.strides[a] * d for a, d in zip(axes, dilations)]
        nk, nu = len(keep), len(axes)

        def remap(c):
            out = [c[d] for d in keep]
            out += [c[a] * s for a, s in zip(axes, strides)]
            out += [c[a] * d for a, d in zip(axes, dilations)]
            return out
        return View(shape, st, self.offset, self._remap_bounds(remap), self.pad_value)

    def operand(self, numel: int, dtype: int) -> D.Operand:
        return D.Operand(list(self.strides), self.offset, dtype, numel, list(self.bounds), self.pad_value)


# ---------------------------------------------------------------------------------------
# nodes (each produces one flat, contiguous buffer)
# ---------------------------------------------------------------------------------------
_ids = itertools.count()


class Node:
    """input: host data.  map: out = expr(operands) over `shape`.  reduce: the same
    folded over `axis` (output keeps the axis with extent 1).  fold: scatter-add
    of operand 0 through `out_view` into a zeroed buffer of `out_numel`."""

    def __init__(self, kind, shape, operands=(), expr=None, dtype=D.F32, reduce_op=D.R_NONE, axis=0,
                 data=None, out_view: Optional[View] = None, name=""):
        self.id = next(_ids)
        self.kind = kind
        self.shape = tuple(int(s) for s in shape)      # iteration shape
        self.operands: List[Tuple["Node", View]] = list(operands)
        self.expr = expr
        self.dtype = dtype
        self.reduce_op = reduce_op
        self.axis = axis
        self.data = data
        self.out_view = out_view
        self.name = name

    @property
    def out_shape(self):
        if self.kind == "reduce":
            return tuple(1 if d == self.axis else s for d, s in enumerate(self.shape))
        if self.kind == "fold":
            return (self.out_numel,)
        return self.shape

    @property
    def out_numel(self):
        if self.kind == "fold":
            return self._fold_numel
        return math.prod(self.out_shape) if self.out_shape else 1


# ---------------------------------------------------------------------------------------
# tensors
# ---------------------------------------------------------------------------------------
w = Ast.w


def _broadcast_shapes(a, b):
    n = max(len(a), len(b))
    a = (1,) * (n - len(a)) + tuple(a)
    b = (1,) * (n - len(b)) + tuple(b)
    out = []
    for x, y in zip(a, b):
        assert x == y or x == 1 or y == 1, f"shapes {a} and {b} do not broadcast"
        out.append(max(x, y))
    return tuple(out)


class Tensor:
    """Lazy tensor = (node, view).  Ops build graph nodes; ``realize`` runs them."""

    def __init__(self, node: Node, view: Optional[View] = None, requires_grad=False):
        self.node = node
        self.view = view if view is not None else View.contiguous(node.out_shape)
        self.requires_grad = requires_grad
        self.grad: Optional["Tensor"] = None
        self._parents: List[Tuple["Tensor", Callable[["Tensor"], "Tensor"]]] = []

    # ---- construction ----
    @staticmethod
    def input(data, requires_grad=False, name="") -> "Tensor":
        data = np.array(data, dtype=np.float32, order="C")      # keeps rank 0 for D0 tensors
        return Tensor(Node("input", data.shape if data.ndim else (1,), data=data, name=name),
                      View.contiguous(data.shape), requires_grad)

    @staticmethod
    def full(shape, value: float) -> "Tensor":
        """A constant: one stored element broadcast with stride 0 (the reference
        uploads full-size ones/zeros tensors, src/tensor/realize.rs:391-502)."""
        node = Node("input", (1,), data=np.array([value], np.float32), name="scalar")
        return Tensor(node, View(tuple(shape), (0,) * len(shape)))

    @property
    def shape(self):
        return self.view.shape

    @property
    def ndim(self):
        return self.view.ndim

    def _track(self, out: "Tensor", *parents):
        """Record (parent, grad_fn) pairs on `out` for parents that need gradients."""
        for p, fn in parents:
            if p.requires_grad:
                out.requires_grad = True
                out._parents.append((p, fn))
        return out

    # ---- views ----
    def _view_op(self, view: View, back) -> "Tensor":
        return self._track(Tensor(self.node, view), (self, back))

    def permute(self, *axes) -> "Tensor":
        axes = list(axes[0]) if len(axes) == 1 and isinstance(axes[0], (list, tuple)) else list(axes)
        inv = [axes.index(i) for i in range(len(axes))]
        return self._view_op(self.view.permute(axes), lambda g: g.permute(inv))

    def unsqueeze(self, dim) -> "Tensor":
        return self._view_op(self.view.unsqueeze(dim), lambda g: g.sum(dim))

    def squeeze(self, dim) -> "Tensor":
        return self._view_op(self.view.squeeze(dim), lambda g: g.unsqueeze(dim))

    def expand(self, *shape) -> "Tensor":
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (list, tuple)) else tuple(shape)
        dims = [d for d, (o, n) in enumerate(zip(self.shape, shape)) if o != n]

        def back(g):
            for d in dims:
                g = g.sum(d, keepdim=True)
            return g
        return self._view_op(self.view.expand(shape), back)

    def reshape(self, *shape) -> "Tensor":
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (list, tuple)) else tuple(shape)
        src = self
        v = self.view.reshape(shape)
        if v is None:
            src = self.contiguous()
            v = src.view.reshape(shape)
        old = self.shape
        return src._track(Tensor(src.node, v), (src, lambda g: g.reshape(old)))

    def pad(self, pads, value=0.0) -> "Tensor":
        sl = [(b, b + s) for (b, _), s in zip(pads, self.shape)]
        return self._view_op(self.view.pad(pads, value), lambda g: g._slice(sl))

    def _slice(self, ranges) -> "Tensor":
        v = self.view
        off = v.offset + sum(lo * st for (lo, _), st in zip(ranges, v.strides))
        bounds = tuple(Bound(list(b.coef), b.c + sum(k * lo for k, (lo, _) in zip(b.coef, ranges)), b.lo, b.hi) for b in v.bounds)
        nv = View([hi - lo for lo, hi in ranges], v.strides, off, bounds, v.pad_value)
        pads = [(lo, s - hi) for (lo, hi), s in zip(ranges, self.shape)]
        return self._view_op(nv, lambda g: g.pad(pads))

    def unfold(self, axes, sizes, strides, dilations) -> "Tensor":
        """Materialised like the reference (every Unfold lowers to a C_ kernel,
        src/lowerer/lower.rs:355-359); its gradient is fold, a scatter-add."""
        uv = self.view.unfold(axes, sizes, strides, dilations)
        node = Node("map", uv.shape, [(self.node, uv)], w(0), name="unfold")
        in_shape = self.shape
        out = Tensor(node)
        return self._track(out, (self, lambda g: g.fold(in_shape, axes, sizes, strides, dilations)))

    def fold(self, out_shape, axes, sizes, strides, dilations) -> "Tensor":
        """Scatter-add windows back (S_ kernel, src/lowerer/lower.rs:580-683)."""
        src = self          # the scatter kernel reads its input through any affine view
        dst = View.contiguous(out_shape).unfold(axes, sizes, strides, dilations)
        node = Node("fold", src.shape, [(src.node, src.view)], None, out_view=dst, name="fold")
        node._fold_numel = math.prod(out_shape)
        out = Tensor(node, View.contiguous(out_shape))
        return src._track(out, (src, lambda g: g.unfold(axes, sizes, strides, dilations)))

    def contiguous(self) -> "Tensor":
        if self.view.is_contiguous() and self.view.numel() == self.node.out_numel:
            return self
        node = Node("map", self.shape, [(self.node, self.view)], w(0), name="contiguous")
        return self._track(Tensor(node), (self, lambda g: g))

    # ---- elementwise ----
    @staticmethod
    def _map(expr_fn, *ts: "Tensor", grads=None, name="") -> "Tensor":
        shape = ()
        for t in ts:
            shape = _broadcast_shapes(shape, t.shape)
        ops = []
        for t in ts:
            v = t.view
            for _ in range(len(shape) - v.ndim):
                v = v.unsqueeze(0)
            ops.append((t.node, v.expand(shape)))
        node = Node("map", shape, ops, expr_fn(*[w(i) for i in range(len(ts))]), name=name)
        out = Tensor(node)
        if grads:
            for t, gfn in zip(ts, grads):
                if t.requires_grad and gfn is not None:
                    out.requires_grad = True
                    out._parents.append((t, (lambda gfn, t: lambda g: _unbroadcast(gfn(g), t.shape))(gfn, t)))
        return out

    def __add__(self, o):
        if not isinstance(o, Tensor):      # scalar literal: folded into the map
            c = float(o)
            return Tensor._map(lambda a: a + c, self, grads=[lambda g: g], name="add")
        return Tensor._map(lambda a, b: a + b, self, o, grads=[lambda g: g, lambda g: g], name="add")

    def __mul__(self, o):
        if not isinstance(o, Tensor):
            c = float(o)
            return Tensor._map(lambda a: a * c, self, grads=[lambda g: g * c], name="mul")
        return Tensor._map(lambda a, b: a * b, self, o, grads=[lambda g: g * o, lambda g: g * self], name="mul")

    def __sub__(self, o):
        if not isinstance(o, Tensor):
            c = float(o)
            return Tensor._map(lambda a: a - c, self, grads=[lambda g: g], name="sub")
        return Tensor._map(lambda a, b: a - b, self, o, grads=[lambda g: g, lambda g: -g], name="sub")

    def __truediv__(self, o):
        if not isinstance(o, Tensor):
            return self * (1.0 / float(o))
        return Tensor._map(lambda a, b: a / b, self, o,
                           grads=[lambda g: g / o, lambda g: -(g * self / (o * o))], name="div")

    __radd__ = __add__
    __rmul__ = __mul__

    def __neg__(self):
        return Tensor._map(lambda a: -a, self, grads=[lambda g: -g], name="neg")

    def exp(self):
        out = Tensor._map(lambda a: a.exp(), self, grads=[None], name="exp")
        return self._track(out, (self, lambda g: g * out))

    def ln(self):
        return Tensor._map(lambda a: a.ln(), self, grads=[lambda g: g / self], name="ln")

    def sqrt(self):
        out = Tensor._map(lambda a: a.sqrt(), self, grads=[None], name="sqrt")
        return self._track(out, (self, lambda g: g / (out * 2.0)))

    def recip(self):
        out = Tensor._map(lambda a: a.recip(), self, grads=[None], name="recip")
        return self._track(out, (self, lambda g: -(g * out * out)))

    def sin(self):
        return Tensor._map(lambda a: a.sin(), self, grads=[lambda g: g * self.cos()], name="sin")

    def cos(self):
        return Tensor._map(lambda a: a.cos(), self, grads=[lambda g: -(g * self.sin())], name="cos")

    def maximum(self, o):
        if not isinstance(o, Tensor):
            c = float(o)
            return Tensor._map(lambda a: a.maximum(c), self,
                               grads=[lambda g: Tensor._map(lambda g_, a: Ast.select(a.lt(c), 0.0, g_), g, self)], name="max")
        # gradient goes to the larger operand (ties to the first), as a select on a < b
        return Tensor._map(lambda a, b: a.maximum(b), self, o,
                           grads=[lambda g: Tensor._map(lambda g_, a, b: Ast.select(a.lt(b), 0.0, g_), g, self, o),
                                  lambda g: Tensor._map(lambda g_, a, b: Ast.select(a.lt(b), g_, 0.0), g, self, o)],
                           name="max")

    def relu(self):
        # relu(x) = max(x, zeros) (crates/nn/src/functional/activation.rs:18-21)
        # (the zeros tensor of the reference is a literal here)
        return self.maximum(0.0)

    def sigmoid(self):
        # 1 / (1 + exp(-x))  (crates/nn/src/functional/activation.rs:50-58)
        return ((-self).exp() + 1.0).recip()

    def tanh(self):
        # 2*sigmoid(2x) - 1, the mathematically intended form of
        # crates/nn/src/functional/activation.rs:70-76 (whose scale() is a no-op).
        # Gradient from the OUTPUT, d tanh = 1 - tanh^2 (as recip and exp above use theirs): differentiating
        # through the composite would recompute exp and the reciprocal in every backward kernel, which are
        # bound by those special functions, not by memory; the output is materialised anyway (the next
        # layer's contraction reads it).
        x = Tensor(self.node, self.view)                       # detached: one gradient rule for the whole function
        out = (x * 2.0).sigmoid() * 2.0 - 1.0
        o = Tensor(out.node, out.view)
        return self._track(out, (self, lambda g: g * ((o * o) * -1.0 + 1.0)))

    # ---- the reference's own spellings, quirks included ----
    # What eclat's Tensor API really builds for these functions (graph-level
    # behaviours that change numerics; kernel-level parity is unaffected because
    # both sides run the same lowered kernels).  Used by the *_reference graphs.
    def ones_like(self) -> "Tensor":
        """A full-size tensor of ones as a REAL input buffer: the reference builds
        constants named ones / zeros on the host and uploads them at every realize
        (src/tensor/realize.rs:391-502)."""
        return Tensor.input(np.ones(self.shape, np.float32), name="ones")

    def zeros_like(self) -> "Tensor":
        return Tensor.input(np.zeros(self.shape, np.float32), name="zeros")

    def scale_ref(self, _factor: float) -> "Tensor":
        """Tensor::scale ignores its factor and multiplies by ones (src/tensor/ops.rs:699-707)."""
        return self * self.ones_like()

    def exp_ref(self) -> "Tensor":
        """exp whose VJP is categorised as Exp2: the gradient is g * 2^x * ones
        (src/grad/rules.rs:254-259,752,854-860)."""
        out = Tensor._map(lambda a: a.exp(), self, grads=[None], name="exp")
        src = self
        return self._track(out, (self, lambda g: g * Tensor._map(lambda a: a.exp2(), Tensor(src.node, src.view)) * src.ones_like()))

    def sigmoid_ref(self) -> "Tensor":
        """crates/nn/src/functional/activation.rs:50-58 with ones as a tensor."""
        return (self.ones_like() + (-self).exp_ref()).recip()

    def tanh_ref(self) -> "Tensor":
        """crates/nn/src/functional/activation.rs:70-76: with scale() a no-op this
        evaluates sigmoid(x) - 1."""
        return self.scale_ref(2.0).sigmoid_ref().scale_ref(2.0) - self.ones_like()

    def relu_ref(self) -> "Tensor":
        """max(x, zeros) with zeros a full-size input buffer (activation.rs:18-21)."""
        return self.maximum(self.zeros_like())

    # ---- reductions ----
    def _reduce(self, op, axis, keepdim) -> "Tensor":
        axis = axis % self.ndim
        if self.shape[axis] == 1 and op in (D.R_SUM, D.R_MAX, D.R_MIN, D.R_PROD):
            return self if keepdim else self.squeeze(axis)     # nothing to fold
        node = Node("reduce", self.shape, [(self.node, self.view)], w(0), reduce_op=op, axis=axis,
                    name={D.R_SUM: "sum", D.R_MAX: "max"}.get(op, "reduce"))
        out = Tensor(node)
        if self.requires_grad:
            full = self.shape
            if op == D.R_SUM:
                back = lambda g: g.expand(full)    # g has the kept-dim shape here
            elif op == D.R_MAX:
                kept = out
                # mask of the positions equal to the maximum (all ties, unnormalised:
                # src/grad/rules.rs:379-399)
                back = lambda g: Tensor._map(lambda g_, x, m: Ast.select(x.lt(m), 0.0, g_),
                                             g.expand(full), self, kept.expand(full))
            else:
                raise NotImplementedError("gradient of this reduce op")
            out.requires_grad = True
            out._parents.append((self, back))
        if not keepdim:
            res = Tensor(out.node, out.view.squeeze(axis), out.requires_grad)
            if out.requires_grad:
                res._parents.append((out, lambda g: g.unsqueeze(axis)))
            return res
        return out

    def sum(self, axis=None, keepdim=False) -> "Tensor":
        if axis is None:
            t = self
            for _ in range(self.ndim):
                t = t.sum(0)
            return t
        return self._reduce(D.R_SUM, axis, keepdim)

    def max(self, axis, keepdim=False) -> "Tensor":
        return self._reduce(D.R_MAX, axis, keepdim)

    # ---- compositions ----
    def matmul(self, other: "Tensor") -> "Tensor":
        """[.., M, K] @ [.., K, N] spelled as the reference spells it
        (examples/matmul_demo.rs:43-60): unsqueeze, expand, multiply, sum over K."""
        a = self.unsqueeze(self.ndim)                 # [.., M, K, 1]
        b = other.unsqueeze(other.ndim - 2)           # [.., 1, K, N]
        shape = _broadcast_shapes(a.shape, b.shape)
        return (a.expand(shape) * b.expand(shape)).sum(len(shape) - 2)

    def linear(self, weight: "Tensor", bias: Optional["Tensor"] = None) -> "Tensor":
        """x [B, I], W [O, I] -> [B, O] (crates/nn/src/functional/linear.rs:27-56)."""
        b_, i_ = self.shape
        o_ = weight.shape[0]
        y = (self.unsqueeze(1).expand(b_, o_, i_) * weight.unsqueeze(0).expand(b_, o_, i_)).sum(2)
        if bias is not None:
            y = y + bias.unsqueeze(0).expand(b_, o_)
        return y

    def conv2d(self, weight: "Tensor", bias: Optional["Tensor"] = None, stride=1, padding=0) -> "Tensor":
        """crates/nn/src/functional/conv.rs:113-184: pad (always), unfold,
        permute to [N,Ho,Wo,C,kh,kw], contiguous, GEMM over C*kh*kw, bias, permute back."""
        n, c, h, wd = self.shape
        co, _, kh, kw = weight.shape
        x = self.pad([(0, 0), (0, 0), (padding, padding), (padding, padding)])
        u = x.unfold([2, 3], [kh, kw], [stride, stride], [1, 1])       # [N, C, Ho, Wo, kh, kw]
        ho, wo = u.shape[2], u.shape[3]
        cols = u.permute(0, 2, 3, 1, 4, 5).contiguous().reshape(n * ho * wo, c * kh * kw)
        y = cols.linear(weight.reshape(co, c * kh * kw))                  # [N*Ho*Wo, Co]
        if bias is not None:
            y = y + bias.unsqueeze(0).expand(n * ho * wo, co)
        return y.reshape(n, ho, wo, co).permute(0, 3, 1, 2)

    def conv2d_fused(self, weight: "Tensor", bias: Optional["Tensor"] = None, padding=0, relu=False,
                     mode: int = D.GEMM_DEFAULT, _flip=False) -> "Tensor":
        """The same function as ``conv2d`` (stride 1) as ONE kernel: the window
        tensor the reference materialises twice (conv.rs:150-166) is gathered on
        the fly inside an implicit GEMM, bias and ReLU run in its epilogue.

        Gradients: the input gradient is the same kernel over the transposed,
        flipped weights (what the reference reaches through unfold's VJP, a
        scatter-add: src/grad/rules.rs:40-53); the weight gradient contracts the
        output gradient with the unfolded input exactly as the composed spelling
        does; the bias gradient is a column sum."""
        n, c, h, wd = self.shape
        if _flip:
            c2, co, kh, kw = weight.shape
        else:
            co, c2, kh, kw = weight.shape
        assert c2 == c
        ho, wo = h + 2 * padding - kh + 1, wd + 2 * padding - kw + 1
        ops = [t.contiguous() for t in ([self, weight] + ([bias] if bias is not None else []))]
        # the kernel writes [N, Co, Ho, Wo] directly (a warp's 32 output positions are consecutive
        # in every channel plane), so consumers see the function's own layout, unit stride innermost
        node = Node("conv", (n, co, ho, wo), [(t.node, t.view) for t in ops], name="conv2d")
        node.conv = (n, c, h, wd, co, kh, kw, padding, bool(relu), mode, bool(_flip), False, False)
        out = Tensor(node)                                    # [N, Co, Ho, Wo]
        if any(t.requires_grad for t in ops):
            assert not relu and not _flip, "the fused ReLU and the gradient form are forward only"
            assert kh == kw and kh - 1 - padding >= 0, "input gradient as a convolution needs a square window and pad <= k-1"
            xc, wc = (Tensor(t.node, t.view) for t in ops[:2])     # detached: the backward graph is not differentiated again
            m, kk = n * ho * wo, c * kh * kw
            flat = {}

            def g2(g):                                        # [M, Co] rows, materialised once for both users
                if id(g) not in flat:
                    flat[id(g)] = g.permute(0, 2, 3, 1).reshape(m, co)
                return flat[id(g)]

            def back_x(g):
                return g.contiguous().conv2d_fused(wc, None, padding=kh - 1 - padding, mode=mode, _flip=True)

            def back_w(g):
                plane, pos = c * h * wd, ho * wo
                if kk <= 12:
                    # tiny reduction: streaming f32 kernel, reads the gradient in its own [N, Co, Ho, Wo] layout
                    gc = g.contiguous()
                    wnode = Node("conv", (co, c, kh, kw), [(xc.node, xc.view), (gc.node, gc.view)], name="conv2d_wgrad")
                    wnode.conv = (n, c, h, wd, co, kh, kw, padding, False, mode, False, True, True)
                    return Tensor(wnode)
                if kh * kw <= 32 and plane % 4 == 0 and plane * 4 <= 64 * 1024 and (pos + 31) // 32 * 32 <= 2048 \
                        and co % 4 == 0 and co <= 128:
                    # positions contracted on the tensor cores, the unfolded input never materialised
                    wnode = Node("conv", (co, c, kh, kw), [(xc.node, xc.view), (g2(g).node, g2(g).view)], name="conv2d_wgrad")
                    wnode.conv = (n, c, h, wd, co, kh, kw, padding, False, mode, False, True, False)
                    return Tensor(wnode)
                xp = xc.pad([(0, 0), (0, 0), (padding, padding), (padding, padding)])
                cols = xp.unfold([2, 3], [kh, kw], [1, 1], [1, 1]).permute(0, 2, 3, 1, 4, 5).contiguous().reshape(m, kk)
                gw = (g2(g).unsqueeze(2).expand(m, co, kk) * cols.unsqueeze(1).expand(m, co, kk)).sum(0)
                return gw.reshape(co, c, kh, kw)

            parents = [(ops[0], back_x), (ops[1], back_w)]
            if bias is not None:
                if kk <= 12:      # nobody else needs the [M, Co] rows: reduce the planes where they lie
                    parents.append((ops[2], lambda g: g.contiguous().reshape(n, co, ho * wo).sum(2).sum(0)))
                else:
                    parents.append((ops[2], lambda g: g2(g).sum(0)))
            self._track(out, *parents)
        return out

    def max_pool2d_unfold(self, k: int) -> "Tensor":
        """crates/nn/src/functional/pool.rs:117-160 as written: unfold windows
        (materialised), max over them; the gradient goes back through fold."""
        n, c, h, wd = self.shape
        u = self.unfold([2, 3], [k, k], [k, k], [1, 1])                 # [N, C, Ho, Wo, k, k]
        return u.reshape(n, c, u.shape[2], u.shape[3], k * k).max(4)

    def max_pool2d(self, k: int) -> "Tensor":
        """The same function without the window tensor: windows do not overlap
        (stride = k), so the k*k taps are k*k strided VIEWS of the input and the
        pool is one elementwise max over them; the gradient is one elementwise
        kernel over the input's own layout (every input element sits in exactly one
        window: the reference's mask-times-gradient followed by fold, pool.rs:117-160
        with src/grad/rules.rs:40-53,379-399, is a permutation here).  Values and
        gradients equal the unfold spelling bit for bit, ties included."""
        n, c, h, wd = self.shape
        if k * k > D.MAX_INPUTS or self.view.bounds:
            return self.max_pool2d_unfold(k)
        ho, wo = h // k, wd // k
        uv = self.view.unfold([2, 3], [k, k], [k, k], [1, 1])           # [N, C, Ho, Wo, k, k] over the input, no copy
        taps = [Tensor(self.node, View(uv.shape[:4], uv.strides[:4], uv.offset + i * uv.strides[4] + j * uv.strides[5]))
                for i in range(k) for j in range(k)]

        def fold_max(*a):
            e = a[0]
            for t in a[1:]:
                e = e.maximum(t)
            return e
        y = Tensor._map(fold_max, *taps, name="maxpool")
        if self.requires_grad:
            x6 = Tensor(self.node, uv.permute((0, 1, 2, 4, 3, 5)))      # [N, C, Ho, k, Wo, k]: the input's own order
            y_ = Tensor(y.node, y.view)

            def back(g):
                full = (n, c, ho, k, wo, k)
                g6 = g.unsqueeze(3).unsqueeze(5).expand(*full)
                y6 = y_.unsqueeze(3).unsqueeze(5).expand(*full)
                gx = Tensor._map(lambda g_, x, m: Ast.select(x.lt(m), 0.0, g_), g6, x6, y6, name="maxpool_grad")
                gx = gx.reshape(n, c, k * ho, k * wo)
                if (k * ho, k * wo) != (h, wd):                         # rows / columns no window covers get no gradient
                    gx = gx.pad([(0, 0), (0, 0), (0, h - k * ho), (0, wd - k * wo)])
                return gx
            y.requires_grad = True
            y._parents.append((self, back))
        return y

    def max_pool2d_fused(self, k: int, relu: bool = False) -> "Tensor":
        """``max_pool2d`` (of ``relu(self)`` when `relu`) as ONE kernel, and its gradient --
        through the ReLU as well -- as ONE kernel (EB200_K_MAXPOOL2D).  Values and gradients
        equal ``self.relu().max_pool2d(k)`` and its autograd bit for bit (only comparisons and
        selections are involved); what changes is the traffic: the strided-view spelling reads
        its taps through four operands and needs a second full-size pass for the activation's
        mask (and a third to zero-pad odd planes)."""
        n, c, h, wd = self.shape
        if k > 4 or h < k or wd < k:
            return (self.relu() if relu else self).max_pool2d(k)
        ho, wo = h // k, wd // k
        xc = self.contiguous()
        node = Node("pool", (n, c, ho, wo), [(xc.node, xc.view)], name="maxpool2d")
        node.pool = (n * c, h, wd, k, bool(relu), False)
        y = Tensor(node)
        if self.requires_grad:
            x_, y_ = Tensor(xc.node, xc.view), Tensor(node)

            def back(g):
                gc = g.contiguous()
                gnode = Node("pool", (n, c, h, wd), [(gc.node, gc.view), (x_.node, x_.view), (y_.node, y_.view)], name="maxpool2d_grad")
                gnode.pool = (n * c, h, wd, k, bool(relu), True)
                return Tensor(gnode)
            y.requires_grad = True
            y._parents.append((self, back))
        return y

    def log_softmax(self, axis=-1) -> "Tensor":
        """crates/nn/src/functional/activation.rs:174-187."""
        axis = axis % self.ndim
        m = self.max(axis, keepdim=True).expand(self.shape)
        z = self - m
        return z - z.exp().sum(axis, keepdim=True).expand(self.shape).ln()

    def softmax_cross_entropy(self, onehot: "Tensor", scale: float) -> "Tensor":
        """scale * sum(onehot * log_softmax(self, axis 1)) for [N, C] logits as ONE kernel that
        also produces the gradient with respect to the logits (the reference composes both
        directions from two dozen tiny kernels: crates/nn/src/functional/activation.rs:174-187,
        loss.rs:32-65, and their VJPs).  Same arithmetic, classes summed in index order."""
        n, c = self.shape
        ops = [self.contiguous(), onehot.contiguous()]
        node = Node("xent", (D.XENT_GRAD_OFFSET + n * c,), [(t.node, t.view) for t in ops], name="softmax_xent")
        node.xent = (n, c, float(scale))
        loss = Tensor(node, View((), (), 0))
        if ops[0].requires_grad:
            dlogits = Tensor(node, View((n, c), (c, 1), D.XENT_GRAD_OFFSET))

            def back(g):
                # the loss is normally the root: its upstream gradient is the constant 1
                if g.node.kind == "input" and g.node.name == "scalar" and float(g.node.data.reshape(-1)[0]) == 1.0:
                    return dlogits
                return dlogits * g.reshape(1, 1).expand(n, c)
            loss.requires_grad = True
            loss._parents.append((ops[0], back))
        return loss

    # ---- autograd ----
    def backward(self, params: Sequence["Tensor"]) -> List["Tensor"]:
        """Reverse-mode sweep from this scalar (the role of grad::backward,
        src/grad/backward.rs:41-87).  Returns one gradient tensor per parameter."""
        order, seen = [], set()

        def topo(t):
            if id(t) in seen:
                return
            seen.add(id(t))
            for p, _ in t._parents:
                topo(p)
            order.append(t)
        topo(self)
        grads: Dict[int, Tensor] = {id(self): Tensor.full(self.shape, 1.0)}
        for t in reversed(order):
            g = grads.get(id(t))
            if g is None:
                continue
            for p, fn in t._parents:
                gp = fn(g)
                assert gp.shape == p.shape, (t.node.name, gp.shape, p.shape)
                grads[id(p)] = gp if id(p) not in grads else grads[id(p)] + gp
        out = []
        for p in params:
            g = grads.get(id(p))
            p.grad = g if g is not None else Tensor.full(p.shape, 0.0)
            out.append(p.grad)
        return out


def _as_tensor(x, like: Tensor) -> Tensor:
    return x if isinstance(x, Tensor) else Tensor.full(like.shape, float(x))


def _unbroadcast(g: Tensor, shape) -> Tensor:
    """Sum a gradient over the dims an operand was broadcast along."""
    while g.ndim > len(shape):
        g = g.sum(0)
    for d, (gs, s) in enumerate(zip(g.shape, shape)):
        if gs != s:
            g = g.sum(d, keepdim=True)
    return g


# ---------------------------------------------------------------------------------------
# fusion + lowering
# ---------------------------------------------------------------------------------------
class _K:
    """A kernel-to-be: mutable copy of a Node used by the fusion passes."""

    def __init__(self, n: Node):
        self.id, self.kind, self.shape, self.expr = n.id, n.kind, n.shape, n.expr
        self.operands = [(src.id, v) for src, v in n.operands]
        self.reduce_op, self.axis, self.dtype, self.name = n.reduce_op, n.axis, n.dtype, n.name
        self.out_view, self.out_numel, self.out_shape = n.out_view, n.out_numel, n.out_shape
        self.data = n.data
        self.conv = getattr(n, "conv", None)
        self.xent = getattr(n, "xent", None)
        self.pool = getattr(n, "pool", None)


def _dim_map(view: View, prod_shape):
    """How a consumer's view walks a producer's contiguous output, as an affine map onto the
    producer's own multi-index: for every consumer dim (producer dim, multiplier) or None for a
    broadcast, plus a base index per producer dim -- producer index[pd] = base[pd] + sum over
    the consumer dims mapped to pd of multiplier * consumer index.  Permutes, broadcasts,
    slices, strided taps (the 2 x 2 taps of a pooling window) and sliding windows all have this
    form.  None when the view is masked or does not decompose without carries between dims."""
    if view.bounds or view.offset < 0:
        return None
    nd = len(prod_shape)
    cstr = D.contiguous_strides(prod_shape)
    base, rest = [0] * nd, view.offset
    for d in range(nd):
        base[d], rest = divmod(rest, cstr[d]) if prod_shape[d] > 1 else (0, rest)
        if base[d] >= max(prod_shape[d], 1):
            return None
    if rest != 0:
        return None
    top = list(base)                       # largest index reached per producer dim so far
    out = []
    for s_, st in zip(view.shape, view.strides):
        if s_ == 1 or st == 0:
            out.append(None)
            continue
        if st < 0:
            return None
        choice = None
        for pd in range(nd):               # outermost first: the largest producer stride that divides st and fits
            if prod_shape[pd] > 1 and st % cstr[pd] == 0:
                mult = st // cstr[pd]
                if top[pd] + mult * (s_ - 1) < prod_shape[pd]:
                    choice = (pd, mult)
                    break
        if choice is None:
            return None
        top[choice[0]] += choice[1] * (s_ - 1)
        out.append(choice)
    return out, base


def _through(view: View, dmap, shape) -> View:
    """A producer operand's view re-expressed over the consumer's dims (composition of the two
    affine maps)."""
    dims, base = dmap
    strides = [view.strides[pd] * mult if pd is not None else 0 for pd, mult in ((d if d is not None else (None, 0)) for d in dims)]
    offset = view.offset + sum(st * b for st, b in zip(view.strides, base))
    bounds = tuple(Bound([b.coef[d[0]] * d[1] if d is not None else 0 for d in dims],
                         b.c + sum(k * o for k, o in zip(b.coef, base)), b.lo, b.hi) for b in view.bounds)
    return View(shape, strides, offset, bounds, view.pad_value)


def _view_key(v: View):
    return (v.shape, v.strides, v.offset, tuple((tuple(b.coef), b.c, b.lo, b.hi) for b in v.bounds), v.pad_value)


def _absorb(c_ops, c_expr, c_shape, j, p: _K):
    """Consumer (operands, expr, shape) with its operand `j` -- the output of the elementwise
    producer `p` -- replaced by p's own expression over p's operands (Wildcard substitution,
    src/ast/mod.rs:1196-1207).  Returns the new (operands, expr) or None when the view is not
    a pure permute / broadcast of the producer or the result would not fit a descriptor."""
    dmap = _dim_map(c_ops[j][1], p.shape)
    if dmap is None:
        return None
    # merged operand list (deduplicated), wildcard renumbering
    new_ops = [o for i, o in enumerate(c_ops) if i != j]
    remap_c = {}
    for i in range(len(c_ops)):
        if i != j:
            remap_c[i] = w(i if i < j else i - 1)
    sub = {}
    for i, (ps, pv) in enumerate(p.operands):
        nv = _through(pv, dmap, c_shape)
        key = (ps, _view_key(nv))
        idx = next((t for t, (s2, v2) in enumerate(new_ops) if (s2, _view_key(v2)) == key), None)
        if idx is None:
            new_ops.append((ps, nv))
            idx = len(new_ops) - 1
        sub[i] = w(idx)
    if len(new_ops) > D.MAX_INPUTS:
        return None
    remap_c[j] = p.expr.substitute(sub)
    new_expr = c_expr.substitute(remap_c)
    prog = new_expr.postfix()
    if len(prog) > D.MAX_INSNS or sum(1 for o in prog if o[0] == D.OP_CONST) > 24 or _stack_depth(prog) > 14:
        return None
    return new_ops, new_expr


def _stack_depth(prog) -> int:
    pops = {D.OP_LOAD: 0, D.OP_CONST: 0, D.OP_SELECT: 3, D.OP_FMA: 3, D.OP_RECIP: 1, D.OP_SQRT: 1, D.OP_LOG2: 1, D.OP_EXP2: 1,
            D.OP_SIN: 1, D.OP_FLOOR: 1, D.OP_NOT: 1, D.OP_CAST: 1}
    depth = best = 0
    for op, _, _ in prog:
        depth += 1 - pops.get(op, 2)
        best = max(best, depth)
    return best


def _fold_constants(e: Ast) -> Ast:
    """Products and sums with several literal operands keep ONE: x*2*(-1)*log2(e) -> x*(-2 log2 e)
    (eclat's AST optimiser folds constants the same way, src/opt/ast/rules.rs; under the reference's
    `-ffast-math` the C compiler may reassociate them too).  Chains of `mul` / `add` are flattened,
    their literals combined in f32, the other operands kept in order."""
    if not e.args:
        return e
    if e.op not in ("mul", "add"):
        return Ast(e.op, tuple(_fold_constants(a) for a in e.args), e.value)
    terms, stack = [], [e]
    while stack:
        t = stack.pop()
        if t.op == e.op:
            stack.extend(reversed(t.args))
        else:
            terms.append(t)
    ident = np.float32(1.0 if e.op == "mul" else 0.0)
    c, rest = ident, []
    for t in terms:
        if t.op == "const":
            c = np.float32(c * np.float32(t.value)) if e.op == "mul" else np.float32(c + np.float32(t.value))
        else:
            rest.append(_fold_constants(t))
    if not rest:
        return Ast.const(float(c))
    out = rest[0]
    for t in rest[1:]:
        out = Ast(e.op, (out, t))
    if c != ident or not np.isfinite(c):
        out = Ast(e.op, (out, Ast.const(float(c))))
    return out


def _is_contraction(k: _K) -> bool:
    """sum over a product of two loads: what the planner serves as a GEMM.  Nothing is inlined
    into its operands (the pattern must survive)."""
    return (k.kind == "reduce" and k.reduce_op == D.R_SUM and k.expr is not None and k.expr.op == "mul"
            and all(a.op == "w" for a in k.expr.args))


def _fuse(ks: Dict[int, _K], order: List[int], roots: set, level: str):
    """Graph-level fusion.  "reference": what eclat does (the last elementwise node folded
    into the reduce that consumes it, src/lowerer/fusion.rs:28-128).  "chains": (1) an
    elementwise node with ONE consumer is composed into it; (2) an elementwise node with
    several elementwise / reduce consumers is RECOMPUTED inside each of them when that moves
    fewer bytes than writing it once and reading it back k times (k consumers, m full-size
    operands: k * m <= m + k) -- e.g. the exp and the reciprocal inside tanh, which the backward
    pass needs again, or a ReLU read by the pool and by two gradient masks."""
    if level == "none":
        return
    changed = True
    while changed:
        changed = False
        uses: Dict[int, List[Tuple[int, int]]] = {}
        for kid in order:
            if kid in ks:
                for j, (src, _) in enumerate(ks[kid].operands):
                    uses.setdefault(src, []).append((kid, j))
        # (1) single consumer
        for kid in order:
            c = ks.get(kid)
            if c is None or c.kind not in ("map", "reduce"):
                continue
            if level == "reference" and c.kind != "reduce":
                continue       # eclat only folds an elementwise node into the reduce that consumes it
            for j, (src, v) in enumerate(c.operands):
                p = ks.get(src)
                if p is None or p.kind != "map" or src in roots or len(uses.get(src, [])) != 1:
                    continue
                if level == "reference" and getattr(c, "_absorbed", False):
                    continue
                res = _absorb(c.operands, c.expr, c.shape, j, p)
                if res is None:
                    continue
                c.operands, c.expr = res
                c._absorbed = True
                del ks[src]
                changed = True
                break
            if changed:
                break
        if changed or level != "chains":
            continue
        # (2) several consumers: recompute instead of store + reload, all consumers or none
        for pid in order:
            p = ks.get(pid)
            cons = uses.get(pid, [])
            if p is None or p.kind != "map" or pid in roots or len(cons) < 2:
                continue
            if p.expr.op == "w" and len(p.operands) == 1:
                continue               # a materialising copy (contiguous / unfold) exists to be read many times
            # operands that are as large as the node itself (broadcast rows / scalars cost next to nothing to re-read)
            p_numel = math.prod(p.shape) if p.shape else 1
            m = sum(1 for _, v in p.operands
                    if 2 * math.prod(ext for st, ext in zip(v.strides, v.shape) if st != 0) > p_numel)
            k = len(cons)
            if k * m > m + k:
                continue
            staged: Dict[int, Tuple[list, Ast]] = {}
            ok = True
            for cid in sorted({cid for cid, _ in cons}):
                c = ks[cid]
                if c.kind not in ("map", "reduce") or _is_contraction(c):
                    ok = False
                    break
                ops_, expr_ = list(c.operands), c.expr
                while ok:                       # a consumer may read the producer through more than one operand
                    j = next((t for t, (s_, _) in enumerate(ops_) if s_ == pid), None)
                    if j is None:
                        break
                    res = _absorb(ops_, expr_, c.shape, j, p)
                    if res is None:
                        ok = False
                        break
                    ops_, expr_ = res
                if not ok:
                    break
                staged[cid] = (ops_, expr_)
            if not ok:
                continue
            for cid, (ops_, expr_) in staged.items():
                ks[cid].operands, ks[cid].expr = ops_, expr_
                ks[cid]._absorbed = True
            del ks[pid]
            changed = True
            break
    if level == "chains":
        for k in ks.values():
            if k.kind in ("map", "reduce") and k.expr is not None and not _is_contraction(k):
                k.expr = _fold_constants(k.expr)


def _lower(k: _K, loc) -> D.KernelDesc:
    """`loc(node id) -> (offset, numel)` of the buffer that holds a node's value
    (its own buffer, or a slice of a flat parameter / gradient buffer)."""
    ins = []
    for src, v in k.operands:
        off, numel = loc(src)
        op = v.operand(numel, D.F32)
        op.offset += off
        ins.append(op)
    out_off, out_numel = loc(k.id)
    if k.kind == "map":
        out = D.Operand(D.contiguous_strides(k.shape), out_off, D.F32, out_numel)
        identity = k.expr.op == "w" and len(k.operands) == 1
        if identity:
            return D.KernelDesc(D.K_COPY, k.shape, ins, out, None, name=k.name)
        return D.KernelDesc(D.K_ELEMENTWISE, k.shape, ins, out, k.expr, name=k.name)
    if k.kind == "reduce":
        kept = [1 if d == k.axis else e for d, e in enumerate(k.shape)]
        st = D.contiguous_strides(kept)
        st[k.axis] = 0
        return D.reduce(list(k.shape), ins, k.expr, k.reduce_op, k.axis, out=D.Operand(st, out_off, D.F32, out_numel))
    if k.kind == "conv":
        n, c, h, wd, co, kh, kw, pad, relu, mode, flip, wgrad, g_nchw = k.conv
        z8 = [0] * 8
        for op in ins:
            op.strides = z8
        return D.KernelDesc(D.K_CONV2D, [n, c, h, wd, co, kh, kw, pad], ins, D.Operand(z8, out_off, D.F32, out_numel),
                            None, gemm_mode=mode, flags=(D.FLAG_RELU if relu else 0) | (D.FLAG_WFLIP if flip else 0) | (D.FLAG_WGRAD if wgrad else D.FLAG_NCHW) | (D.FLAG_G_NCHW if g_nchw else 0), name=k.name)
    if k.kind == "pool":
        planes, h, wd, win, relu, grad = k.pool
        d = D.maxpool2d(planes, h, wd, win, relu, grad)
        for op, src in zip(d.inputs, ins):
            op.offset, op.numel = src.offset, src.numel
        d.output.offset, d.output.numel = out_off, out_numel
        d.name = k.name
        return d
    if k.kind == "xent":
        n, c, scale = k.xent
        d = D.softmax_xent(n, c, scale)
        for op, src in zip(d.inputs, ins):
            op.offset, op.numel = src.offset, src.numel
        d.output.offset, d.output.numel = out_off, out_numel
        d.name = k.name
        return d
    if k.kind == "fold":
        assert out_off == 0, "a scatter output owns its buffer (it is zero-filled as a whole)"
        return D.KernelDesc(D.K_SCATTER, k.shape, ins, k.out_view.operand(k.out_numel, D.F32), None, name=k.name)
    raise ValueError(k.kind)


_FLAT_P, _FLAT_G = -1, -2       # container ids of the flat parameter / gradient buffers


class Program:
    """Compiled multi-root realize: every root (and every gradient) comes out of
    one kernel list, parameters live in persistent buffers and are updated in
    place.  (The reference re-runs the whole graph once per gradient and updates
    on the host: crates/nn/src/optim/optimizer.rs:100-131, sgd.rs:73-103.)"""

    def __init__(self, roots: Sequence[Tensor], executor, fuse: str = "chains",
                 sgd: Sequence[Tuple[Tensor, Tensor]] = (), lr: float = 0.0, persistent: bool = False,
                 flat: bool = False, optimizer: str = "sgd", momentum: float = 0.0,
                 betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, comm=None, overlap: bool = True):
        """`flat=True` lays all parameters out in one buffer and all gradients in
        another (same offsets): one all-reduce and one update kernel per step.

        `optimizer`: "sgd" (crates/nn/src/optim/sgd.rs:91-95), "momentum"
        (sgd.rs:84-89) or "adam" (adam.rs:104-147); the stateful ones keep their
        velocity / moments / step counter in device buffers laid out like the flat
        parameters.

        `comm` (a ``B200Comm`` or the CPU stand-in ``HostComm``) makes the step
        data parallel: the gradients are summed over the ranks before the update
        (pass lr / world size for the gradient mean).  With plain SGD the
        all-reduce and the update are one kernel, and with `overlap` the part of the
        flat buffer whose gradients are complete early in the backward pass is
        reduced and updated on the communicator's side stream while the rest of the
        backward pass runs."""
        assert optimizer in ("sgd", "momentum", "adam")
        assert optimizer == "sgd" or flat, "stateful optimizers run over the flat parameter buffer"
        assert comm is None or flat, "a data-parallel step all-reduces the flat gradient buffer"
        self.optimizer, self.lr, self.comm, self.overlap = optimizer, lr, comm, overlap
        self.ex = executor
        self.persistent = persistent      # keep every intermediate buffer between runs (no per-step allocation)
        self.graph = None
        self.graph_has_update = False
        self.roots = list(roots)
        self.sgd = [(p_, g_.contiguous()) for p_, g_ in sgd]     # gradient buffers share the parameter layout
        all_roots = self.roots + [g for _, g in self.sgd] + [p for p, _ in self.sgd]
        nodes: Dict[int, Node] = {}
        order: List[int] = []

        def visit(n: Node):
            if n.id in nodes:
                return
            nodes[n.id] = n
            for src, _ in n.operands:
                visit(src)
            order.append(n.id)
        import sys
        sys.setrecursionlimit(max(10000, sys.getrecursionlimit()))
        for t in all_roots:
            visit(t.node)
        ks = {i: _K(nodes[i]) for i in order}
        root_ids = {t.node.id for t in all_roots}
        _fuse(ks, order, root_ids, fuse)
        self.order = [i for i in order if i in ks]
        # As-soon-as-possible order: a kernel runs right after the level of its last producer (ties keep
        # the depth-first order).  The depth-first walk alone leaves, e.g., the weight gradients of the
        # last layers at the very end of the backward pass although their inputs exist early; with them
        # early, their share of a data-parallel step's gradient all-reduce overlaps the rest of the pass.
        level: Dict[int, int] = {}
        for i in self.order:
            srcs = [s_ for s_, _ in ks[i].operands]
            level[i] = 0 if ks[i].kind == "input" else 1 + max([level[s_] for s_ in srcs], default=0)
        rank_of = {i: r for r, i in enumerate(self.order)}
        self.order.sort(key=lambda i: (level[i], rank_of[i]))
        self.ks = ks
        self.numel = {i: ks[i].out_numel for i in self.order}
        self.inputs = {i: ks[i] for i in self.order if ks[i].kind == "input"}
        # where each node's value lives: (container id, offset); containers own the buffers
        self.where: Dict[int, Tuple[int, int]] = {i: (i, 0) for i in self.order}
        self.cnumel: Dict[int, int] = dict(self.numel)
        pids, gids = [p_.node.id for p_, _ in self.sgd], [g_.node.id for _, g_ in self.sgd]
        self.flat = bool(flat and self.sgd and len(set(pids)) == len(pids) and len(set(gids)) == len(gids)
                         and all(ks[i].kind == "input" for i in pids)
                         and all(ks[i].kind in ("map", "reduce", "conv") for i in gids))
        assert comm is None or self.flat, "a data-parallel step needs every gradient to be a kernel output that can live in the flat buffer"
        if self.flat:
            off = 0
            for pid, gid in zip(pids, gids):
                self.where[pid], self.where[gid] = (_FLAT_P, off), (_FLAT_G, off)
                off += (self.numel[pid] + 63) // 64 * 64        # 256-byte aligned slices
            self.cnumel[_FLAT_P] = self.cnumel[_FLAT_G] = off

        def loc(i):
            c, off = self.where[i]
            return off, self.cnumel[c]
        self.kernels = []          # (node id, desc, compiled kernel, [src ids])
        for i in self.order:
            k = ks[i]
            if k.kind == "input":
                continue
            d = _lower(k, loc)
            self.kernels.append((i, d, self.ex.compile(d), [s for s, _ in k.operands]))
        # liveness: a buffer may go once its last consumer has run
        last = {}
        for pos, (i, _, _, srcs) in enumerate(self.kernels):
            for s in srcs:
                last[s] = pos
        keep = set(root_ids) | set(self.inputs)
        self.release_after = [[] for _ in self.kernels]
        for s, pos in last.items():
            if s not in keep and self.where[s][0] == s:
                self.release_after[pos].append(s)
        self.sgd_kernels = []
        self.state: List[object] = []        # optimizer state buffers (velocity | moments and step counter)
        self.buckets: List[Tuple[int, int, int]] = []     # (offset, count, kernel position after which it may go) of the async part
        if self.flat:
            n = self.cnumel[_FLAT_P]
            if optimizer == "momentum":
                d = D.sgd_momentum(n, lr, momentum)
            elif optimizer == "adam":
                d = D.adam(n, lr, betas[0], betas[1], eps)
            else:
                d = D.KernelDesc(D.K_SGD, [n], [D.contiguous([n]), D.contiguous([n])], D.contiguous([n]), scalar=lr)
            self.sgd_kernels.append((_FLAT_P, _FLAT_G, self.ex.compile(d)))
            if comm is not None and optimizer == "sgd" and overlap and comm.info()["nranks"] > 1:
                self.buckets = self._plan_buckets(pids, gids)
        else:
            for p, g in self.sgd:
                n = p.node.out_numel
                d = D.KernelDesc(D.K_SGD, [n], [D.contiguous([n]), D.contiguous([n])], D.contiguous([n]), scalar=lr)
                self.sgd_kernels.append((p.node.id, g.node.id, self.ex.compile(d)))
        self.buf: Dict[int, object] = {}
        if self.flat:
            host = np.zeros(self.cnumel[_FLAT_P], np.float32)
            for pid in pids:
                o = self.where[pid][1]
                host[o:o + self.numel[pid]] = ks[pid].data.reshape(-1)
            self.buf[_FLAT_P] = self.ex.alloc(host.size)
            self.ex.upload(self.buf[_FLAT_P], host)
            self.buf[_FLAT_G] = self.ex.alloc(host.size)
            self.ex.upload(self.buf[_FLAT_G], np.zeros_like(host))
            if optimizer in ("momentum", "adam"):
                for _ in range(1 if optimizer == "momentum" else 2):
                    b = self.ex.alloc(host.size)
                    self.ex.upload(b, np.zeros_like(host))
                    self.state.append(b)
                if optimizer == "adam":
                    self.state.append(self.ex.alloc_counter())
        for i, k in self.inputs.items():
            if self.where[i][0] != i:
                continue
            self.buf[i] = self.ex.alloc(self.numel[i])
            self.ex.upload(self.buf[i], k.data.reshape(-1))

    def set_input(self, t: Tensor, data: np.ndarray):
        assert self.where[t.node.id][0] == t.node.id, "parameters of a flat program are not re-uploaded one by one"
        self.ex.upload(self.buf[t.node.id], np.ascontiguousarray(data, np.float32).reshape(-1))

    def _b(self, i):
        return self.buf[self.where[i][0]]

    def kernel_descs(self) -> List[D.KernelDesc]:
        return [d for _, d, _, _ in self.kernels]

    def _plan_buckets(self, pids, gids):
        """Which contiguous part of the flat buffers can be reduced and updated
        before the backward pass has finished: the part whose gradients are
        written, and whose parameters are last read, earliest.  Scored by size
        times the number of kernels still to run behind it."""
        pos_of = {i: pos for pos, (i, _, _, _) in enumerate(self.kernels)}
        last_read: Dict[int, int] = {}
        for pos, (_, _, _, srcs) in enumerate(self.kernels):
            for s_ in srcs:
                last_read[s_] = pos
        items = []
        total = self.cnumel[_FLAT_P]
        for j, (pid, gid) in enumerate(zip(pids, gids)):
            off = self.where[pid][1]
            end = self.where[pids[j + 1]][1] if j + 1 < len(pids) else total
            items.append((off, end - off, max(pos_of.get(gid, -1), last_read.get(pid, -1), last_read.get(gid, -1))))
        n = len(self.kernels)
        best = None
        for k in range(1, len(items)):
            for early in (items[k:], items[:k]):
                ready = max(it[2] for it in early)
                count = sum(it[1] for it in early)
                score = count * (n - 1 - ready)
                if ready < n - 1 and (best is None or score > best[0]):
                    best = (score, early[0][0], count, ready)
        return [best[1:]] if best else []

    def _rest_of_flat(self):
        """The (offset, count) ranges of the flat buffers no early bucket covers."""
        total = self.cnumel[_FLAT_P]
        if not self.buckets:
            return [(0, total)]
        off, cnt, _ = self.buckets[0]
        return [r for r in ((0, off), (off + cnt, total - off - cnt)) if r[1] > 0]

    def run_forward(self):
        """All kernels up to and including the gradients.  In a data-parallel step
        with overlap, the early bucket's all-reduce + update is issued on the
        communicator's side stream as soon as its gradients are complete."""
        for pos, (i, d, kern, srcs) in enumerate(self.kernels):
            c = self.where[i][0]
            if c not in self.buf:
                self.buf[c] = self.ex.alloc(self.cnumel[c])
            kern.execute([self._b(s) for s in srcs], [self.buf[c]])
            if not self.persistent:
                for s in self.release_after[pos]:
                    self.ex.free(self.buf.pop(s))
            for off, cnt, ready in self.buckets:
                if ready == pos:
                    self.comm.allreduce_sgd(self.buf[_FLAT_P], self.buf[_FLAT_G], self.lr, off, cnt, side_stream=True)

    def run_update(self):
        if self.comm is not None and self.optimizer == "sgd":
            # gradient all-reduce and p -= lr * sum as one kernel per range
            for off, cnt in self._rest_of_flat():
                self.comm.allreduce_sgd(self.buf[_FLAT_P], self.buf[_FLAT_G], self.lr, off, cnt)
            self.comm.join()
            return
        if self.comm is not None:
            self.comm.allreduce(self.buf[_FLAT_G], D.R_SUM)
        for pid, gid, kern in self.sgd_kernels:
            kern.execute([self.buf[pid], self.buf[gid]] + self.state, [self.buf[pid]])

    def run(self, between=None):
        """One step.  `between` (optional callable) runs after the gradients are
        complete and before the parameter update."""
        if self.graph is not None:
            self.graph.launch()
        else:
            self.run_forward()
        if between is not None:
            between()
        if self.graph is None or not self.graph_has_update:
            self.run_update()

    def capture(self, include_update: bool = True):
        """Record one step as a CUDA graph; later ``run`` calls replay it.  With
        ``include_update=False`` only forward+backward are recorded and the
        parameter update stays a separate launch sequence (so a collective can sit
        between them).  Needs ``persistent=True`` and the CUDA executor."""
        assert self.persistent, "capture needs persistent buffers"
        assert include_update or not self.buckets, "an overlapped data-parallel step is recorded as a whole"
        self.run_forward()                              # allocates every buffer, warms every kernel
        if self.buckets:
            self.run_update()                           # (a whole step: the early bucket's update has been issued)
        self.ex.synchronize()
        self.ex.dev.graph_begin()
        try:
            self.run_forward()
            if include_update:
                self.run_update()
        finally:
            self.graph = self.ex.dev.graph_end()
        self.graph_has_update = include_update

    def grad_buffers(self):
        """The buffers a data-parallel job all-reduces (one when flat)."""
        if self.flat:
            return [self.buf[_FLAT_G]]
        return [self.buf[g.node.id] for _, g in self.sgd]

    def buffer_of(self, t: Tensor):
        return self._b(t.node.id)

    def fetch(self, t: Tensor) -> np.ndarray:
        """Root value as a numpy array of the tensor's logical shape."""
        c, off = self.where[t.node.id]
        flat = self.ex.download(self.buf[c], self.cnumel[c])[off:off + self.numel[t.node.id]]
        v = t.view
        if v.is_contiguous() or not v.shape:
            return flat[v.offset:v.offset + max(1, v.numel())].reshape(v.shape)
        return np.lib.stride_tricks.as_strided(flat[v.offset:], v.shape, [s * 4 for s in v.strides]).copy()


class B200Executor:
    """Runs programs on the CUDA library."""

    def __init__(self, device=None, registry=None):
        from .backend import B200BackendRegistry
        self.reg = registry or B200BackendRegistry()
        self.dev = device or self.reg.create_device(0)

    def alloc(self, numel):
        from .backend import B200Buffer
        return B200Buffer.allocate(self.dev, [numel], D.F32, zero=False)

    def free(self, buf):
        buf.release()

    def upload(self, buf, data):
        buf.write_vec(data)

    def download(self, buf, numel):
        return buf.read_vec()

    def alloc_counter(self):
        """One zeroed I32 element (Adam's step counter)."""
        from .backend import B200Buffer
        return B200Buffer.allocate(self.dev, [1], D.I32, zero=True)

    def compile(self, d):
        return self.reg.compile_ast(self.dev, d)

    def synchronize(self):
        self.dev.synchronize()
