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
