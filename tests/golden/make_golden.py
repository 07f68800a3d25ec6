"""Writes tests/golden/kernels.json: pairs {lowered-kernel descriptor <-> the C the
reference's C backend is expected to emit for that kernel}.

Purpose: eclat is Rust and cannot be built where this backend is developed, so the
shape of the C its renderer emits (and therefore of the kernels the lowerer hands
a backend) is restated by oracle/c_emit.py from the renderer's source.  Whoever
has a Rust toolchain can lower the same graphs with eclat (ECLAT_OPT_LEVEL=0),
dump the kernels and diff them against this file: `c` is the text to compare,
`desc` the descriptor the eclat-side lowering walk should produce for it.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from harp_b200 import desc as D                     # noqa: E402
from harp_b200 import workloads as W                # noqa: E402
from harp_b200.frontend import Program, Tensor      # noqa: E402
from oracle import c_emit as O                      # noqa: E402

w = D.Ast.w


class _Null:
    def alloc(self, n): return None
    def alloc_counter(self): return None
    def free(self, b): pass
    def upload(self, b, d): pass
    def compile(self, d): return None


def cases():
    """(name, reference source the kernel comes from, descriptor)"""
    out = []
    c4 = D.contiguous([4])
    out.append(("add_1d", "crates/backend-c/src/lib.rs:181-215", D.elementwise([4], [c4, c4], w(0) + w(1))))
    out.append(("mul_1d", "crates/backend-c/src/lib.rs:217-251", D.elementwise([4], [c4, c4], w(0) * w(1))))
    c23 = D.contiguous([2, 3])
    out.append(("add_2d", "crates/backend-c/src/lib.rs:253-295", D.elementwise([2, 3], [c23, c23], w(0) + w(1))))
    out.append(("exp", "src/graph/ops.rs:151-367 (exp = exp2(x * log2e))", D.elementwise([8], [D.contiguous([8])], w(0).exp())))
    out.append(("sub", "src/graph/ops.rs:151-367 (a - b = a + b * -1)", D.elementwise([8], [D.contiguous([8])] * 2, w(0) - w(1))))
    out.append(("relu_zeros", "crates/nn/src/functional/activation.rs:18-21", D.elementwise([8], [D.contiguous([8])] * 2, w(0).maximum(w(1)))))
    out.append(("sum_axis1", "src/lowerer/loop_gen.rs:87-151", D.reduce([8, 16], [D.contiguous([8, 16])], w(0), D.R_SUM, 1)))
    out.append(("max_axis0", "src/lowerer/loop_gen.rs:87-151", D.reduce([8, 16], [D.contiguous([8, 16])], w(0), D.R_MAX, 0)))
    out.append(("min_axis1", "src/graph/node.rs:67-74", D.reduce([8, 16], [D.contiguous([8, 16])], w(0), D.R_MIN, 1)))
    out.append(("matmul_demo_16", "examples/matmul_demo.rs:43-60", W.matmul_desc(16, 16, 16)))
    out.append(("linear_8x4x6", "crates/nn/src/functional/linear.rs:27-56", W.linear_desc(8, 4, 6)))
    out.append(("permute_contiguous", "src/graph/node.rs:431-445", W.cfg2_t(8, 16)))
    out.append(("cumsum_axis1", "src/lowerer/loop_gen.rs:237-327", D.scan([4, 8], [D.contiguous([4, 8])], w(0), D.R_SUM, 1)))
    out.append(("cumsum_axis0_of_3d", "src/lowerer/loop_gen.rs:237-327", D.scan([3, 4, 5], [D.contiguous([3, 4, 5])], w(0), D.R_SUM, 0)))
    # kernels of a padded convolution as functional::conv2d composes it (crates/nn/src/functional/conv.rs:113-184)
    x = Tensor.input([[[[float(i + j) for j in range(5)] for i in range(5)]]], requires_grad=True)
    wt = Tensor.input([[[[1.0, 0.0, -1.0]] * 3]] * 2, requires_grad=True)
    b = Tensor.input([0.5, -0.5], requires_grad=True)
    y = x.conv2d(wt, b, padding=1)
    loss = (y * y).sum()
    prog = Program([loss] + loss.backward([x, wt, b]), _Null(), fuse="reference")
    for i, d in enumerate(prog.kernel_descs()):
        out.append((f"conv2d_pad1_step_{i:02d}_{d.name}", "crates/nn/src/functional/conv.rs:113-184 + src/grad/rules.rs", d))
    # 16-bit storage types as the C backend declares them (crates/backend-c/src/renderer.rs:129-130)
    h8, b8 = D.contiguous([8], D.F16), D.contiguous([8], D.BF16)
    out.append(("add_f16", "crates/backend-c/src/renderer.rs:129 (_Float16)", D.KernelDesc(D.K_ELEMENTWISE, [8], [h8, h8], D.contiguous([8], D.F16), w(0) + w(1))))
    out.append(("sum_bf16_into_f32", "crates/backend-c/src/renderer.rs:130 (__bf16), src/lowerer/loop_gen.rs:87-151",
                D.reduce([4, 8], [D.contiguous([4, 8], D.BF16)], w(0), D.R_SUM, 1)))
    # max_pool2d as functional::max_pool2d composes it (crates/nn/src/functional/pool.rs:117-160) and its gradient
    xp = Tensor.input([[[[float((i * 7 + j * 3) % 5) for j in range(4)] for i in range(4)]]], requires_grad=True)
    yp = xp.max_pool2d_unfold(2)
    lp = (yp * yp).sum()
    prog = Program([lp] + lp.backward([xp]), _Null(), fuse="reference")
    for i, d in enumerate(prog.kernel_descs()):
        out.append((f"max_pool2d_step_{i:02d}_{d.name}", "crates/nn/src/functional/pool.rs:117-160 + src/grad/rules.rs", d))
    # config 2 as three realizes at the reference's fusion level
    rows, cols = 8, 16
    xt = Tensor.input([[float(i * cols + j) * 0.01 for j in range(cols)] for i in range(rows)])
    c0, c1 = Tensor.input(0.5), Tensor.input(1.0)
    bc = lambda c: c.unsqueeze(0).unsqueeze(1).expand(rows, cols)
    prog = Program([((bc(c0) * xt + bc(c1)).exp() * xt).sum(1), xt.max(0), xt.permute(1, 0).contiguous()], _Null(), fuse="reference")
    for i, d in enumerate(prog.kernel_descs()):
        out.append((f"cfg2_small_{i:02d}_{d.name}", "configs[1] through src/tensor/ops.rs", d))
    return out


def build():
    items = []
    for name, source, d in cases():
        items.append({"name": name, "reference": source, "desc": d.to_json(),
                      "c": O.emit_kernel_c(d, "kernel"), "c_fma": O.emit_kernel_c(d, "kernel", fma=True),
                      "c_openmp": O.emit_kernel_c(d, "kernel", openmp=True)})
    return items


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels.json")
    with open(path, "w") as f:
        json.dump(build(), f, indent=1)
    print(f"wrote {path}")
