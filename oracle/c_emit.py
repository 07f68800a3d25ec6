"""CPU oracle: the C the reference's C backend would emit for a lowered kernel.

TEST INFRASTRUCTURE ONLY.  Nothing on the product path may import this module;
it is the checker for the parity tests, for ``__graft_entry__.smoke()`` and for
the CPU-baseline legs of ``bench.py``.

The reference (eclat, 100 % Rust) has no native sources and cannot be built
without a Rust toolchain, but the arithmetic of its CPU backend is C text that
it generates at run time and hands to the system ``gcc``.  This module restates
that generator for the kernel classes on the hot path, so the oracle is real
compiled C built with the reference's own flags:

* loop nests: ``for (long long ridxN = 0; ridxN < S; ridxN += 1)`` in axis order,
  reduce axis innermost (src/lowerer/loop_gen.rs:51-151, range rendering
  src/backend/renderer.rs:638-648);
* addressing: ``offset + sum ridx_d * stride_d`` (src/lowerer/index_gen.rs:45-63),
  reduce output index with the reduce axis forced to 0 (index_gen.rs:107-112);
* padded loads ``(cond ? buf[idx] : pad)`` (src/lowerer/lower.rs:1145-1157) with
  ``cond`` built from ``<``, ``&&``, ``!`` (src/graph/shape/view.rs:997-1011);
* expressions: every binary op parenthesised, ``fmaxf/sqrtf/log2f/exp2f/sinf/
  floorf``, ``(1.0f / x)`` (src/backend/renderer.rs:268-441,
  crates/backend-c/src/renderer.rs:181-206), f32 literal formatting
  (src/backend/renderer.rs:196-215);
* reduce: block-scope ``float acc;``, identity store, sequential combine
  (src/lowerer/lower.rs:525-571, src/graph/node.rs:29-77);
* scatter: zero-fill nest then ``out[dst] += in[src]`` nest
  (src/lowerer/lower.rs:580-683, crates/backend-c/src/renderer.rs:208-214);
* header and signature (crates/backend-c/src/renderer.rs:153-174): pointers
  without ``const``, inputs first then the output;
* flags ``gcc -O3 -ffast-math -shared -fPIC -o lib.so kernel.c -lm``
  (crates/backend-c/src/compiler.rs:153-165); the OpenMP variant adds
  ``#include <omp.h>``, ``#pragma omp parallel for`` on the outermost loop
  (crates/backend-openmp/src/renderer.rs:217-259) and ``-fopenmp``
  (crates/backend-openmp/src/compiler.rs:161).

Parity pinning: the known-answer vectors of the reference's backend tests
(crates/backend-c/src/lib.rs:164-339, crates/backend-openmp/src/lib.rs:167-231)
are replayed against this oracle in tests/test_oracle.py.  Transcendentals come
from glibc libm under ``-ffast-math``; no reference test pins their values:
PARITY UNPINNED at that boundary (the 1e-5 relative tolerance is the contract).
"""
from __future__ import annotations

import ctypes
import hashlib
import math
import os
import subprocess
from typing import List, Sequence

import numpy as np

from harp_b200 import desc as D

_CACHE_DIR = os.environ.get(
    "EB200_ORACLE_CACHE", os.path.join(os.path.dirname(os.path.abspath(__file__)), "_build"))

C_TYPE = {D.F32: "float", D.BOOL: "unsigned char", D.I32: "int", D.I64: "long long",
          D.F16: "_Float16", D.BF16: "__bf16"}      # crates/backend-c/src/renderer.rs:129-130

HEADER = """/* Generated C code by Harp */
/* This code is pure C99 without parallelization */

#include <math.h>
#include <stdlib.h>
#include <stdint.h>

"""


def f32_literal(v: float) -> str:
    """Literal::F32 rendering (src/backend/renderer.rs:196-215): Rust's shortest
    round-trip ``{}`` formatting, ``.0`` appended when no point/exponent."""
    f = np.float32(v)
    if np.isnan(f):
        return "NAN"
    if np.isinf(f):
        return "INFINITY" if f > 0 else "(-INFINITY)"
    s = np.format_float_positional(f, unique=True, trim="-")  # Rust prints no exponent for f32 Display
    if "." not in s:
        s += ".0"
    return s + "f"


def _affine(offset: int, strides: Sequence[int], skip_axis: int = -1) -> str:
    """Index expression after Expr::simplify: zero terms dropped, ``*1`` folded."""
    terms: List[str] = []
    if offset:
        terms.append(str(int(offset)))
    for d, s in enumerate(strides):
        if s == 0 or d == skip_axis:
            continue
        terms.append(f"ridx{d}" if s == 1 else f"(ridx{d} * {int(s)})")
    if not terms:
        return "0"
    out = terms[0]
    for t in terms[1:]:
        out = f"({out} + {t})"
    return out


def _cond(b: D.Bound) -> str:
    e = _affine(b.c, b.coef)
    return f"((!({e} < {int(b.lo)})) && ({e} < {int(b.hi)}))"


def _load(name: str, op: D.Operand) -> str:
    ld = f"{name}[{_affine(op.offset, op.strides)}]"
    if op.bounds:
        cond = _cond(op.bounds[0])
        for b in op.bounds[1:]:
            cond = f"({cond} && {_cond(b)})"
        return f"({cond} ? {ld} : {f32_literal(op.pad_value)})"
    return ld


def render_expr(n: D.Ast, loads: List[str], fma: bool = False) -> str:
    r = lambda a: render_expr(a, loads, fma)
    a = n.args
    if n.op == "w":
        return loads[n.value]
    if n.op == "const":
        return f32_literal(n.value)
    if n.op == "add":
        if fma and a[0].op == "mul":
            return f"fma({r(a[0].args[0])}, {r(a[0].args[1])}, {r(a[1])})"
        return f"({r(a[0])} + {r(a[1])})"
    if n.op == "mul":
        return f"({r(a[0])} * {r(a[1])})"
    if n.op == "max":
        return f"fmaxf({r(a[0])}, {r(a[1])})"
    if n.op == "recip":
        return f"(1.0f / {r(a[0])})"
    if n.op in ("sqrt", "log2", "exp2", "sin", "floor"):
        return f"{n.op}f({r(a[0])})"
    if n.op == "lt":
        return f"({r(a[0])} < {r(a[1])})"
    if n.op == "and":
        return f"({r(a[0])} && {r(a[1])})"
    if n.op == "not":
        return f"(!{r(a[0])})"
    if n.op == "select":
        return f"({r(a[0])} ? {r(a[1])} : {r(a[2])})"
    if n.op == "rem":
        return f"({r(a[0])} % {r(a[1])})"
    if n.op == "idiv":
        return f"({r(a[0])} / {r(a[1])})"
    if n.op == "cast":
        return f"({C_TYPE[n.value]})({r(a[0])})"
    if n.op == "fma":
        return f"fma({r(a[0])}, {r(a[1])}, {r(a[2])})"
    raise ValueError(n.op)


_IDENTITY = {D.R_SUM: 0.0, D.R_MAX: -math.inf, D.R_MIN: math.inf, D.R_PROD: 1.0}


def _combine(op: int, acc: str, val: str, fma: bool, val_ast) -> str:
    if op == D.R_SUM:
        if fma and val_ast is not None and val_ast.op == "mul":
            return None  # handled by caller
        return f"({acc} + {val})"
    if op == D.R_MAX:
        return f"fmaxf({acc}, {val})"
    if op == D.R_MIN:
        # ReduceOp::Min combines with Select(Lt) (src/graph/node.rs:67-74)
        return f"(({acc} < {val}) ? {acc} : {val})"
    if op == D.R_PROD:
        return f"({acc} * {val})"
    raise ValueError(op)


def emit_kernel_c(k: D.KernelDesc, fn_name: str = "kernel", openmp: bool = False,
                  fma: bool = False) -> str:
    """C source for one kernel.  ``fma=True`` gives the form the backend-side
    AST rule ``a*b+c -> fma(a,b,c)`` produces (src/opt/ast/rules/mod.rs:115-143),
    rendered as the double-precision ``fma()`` (src/backend/renderer.rs:107-109)."""
    nd = k.ndim
    names = [f"buf{i}" for i in range(len(k.inputs))]
    params = [f"{C_TYPE[o.dtype]}* {n}" for o, n in zip(k.inputs, names)]
    params.append(f"{C_TYPE[k.output.dtype]}* out")
    src = HEADER
    if openmp:
        src = src.replace("#include <math.h>", "#include <omp.h>\n#include <math.h>")
    src += "// === Kernel Functions ===\n"
    src += f"void {fn_name}({', '.join(params)}) {{\n"
    ind = 1
    pragma_done = [not openmp]

    def open_loop(d: int, extent: int):
        nonlocal src, ind
        if not pragma_done[0]:
            src += " " * (4 * ind) + "#pragma omp parallel for\n"
            pragma_done[0] = True
        src += " " * (4 * ind) + f"for (long long ridx{d} = 0; ridx{d} < {extent}; ridx{d} += 1) {{\n"
        ind += 1

    def close_loop():
        nonlocal src, ind
        ind -= 1
        src += " " * (4 * ind) + "}\n"

    def line(s: str):
        nonlocal src
        src += " " * (4 * ind) + s + "\n"

    loads = [_load(n, o) for n, o in zip(names, k.inputs)]

    if k.kclass in (D.K_ELEMENTWISE, D.K_COPY):
        value = render_expr(k.map, loads, fma) if k.map is not None else loads[0]
        for d in range(nd):
            open_loop(d, k.shape[d])
        line(f"out[{_affine(k.output.offset, k.output.strides)}] = {value};")
        for _ in range(nd):
            close_loop()
    elif k.kclass == D.K_REDUCE:
        ax = k.reduce_axis
        order = [d for d in range(nd) if d != ax]
        for d in order:
            open_loop(d, k.shape[d])
        line("float acc;")
        line(f"acc = {f32_literal(_IDENTITY[k.reduce_op])};")
        pragma_done[0] = True  # never parallelise the sequential reduce loop
        open_loop(ax, k.shape[ax])
        if fma and k.reduce_op == D.R_SUM and k.map is not None and k.map.op == "mul":
            a, b = k.map.args
            line(f"acc = fma({render_expr(a, loads, fma)}, {render_expr(b, loads, fma)}, acc);")
        else:
            val = render_expr(k.map, loads, fma) if k.map is not None else loads[0]
            line(f"acc = {_combine(k.reduce_op, 'acc', val, False, None)};")
        close_loop()
        line(f"out[{_affine(k.output.offset, k.output.strides, skip_axis=ax)}] = acc;")
        for _ in order:
            close_loop()
    elif k.kclass == D.K_SCATTER:
        # zero-fill over the (contiguous) output, then accumulate in loop order
        line(f"for (long long ridx0 = 0; ridx0 < {int(k.output.numel)}; ridx0 += 1) {{")
        line("    out[ridx0] = 0.0f;")
        line("}")
        pragma_done[0] = True  # `+=` is not atomic in the C backend: keep sequential
        for d in range(nd):
            open_loop(d, k.shape[d])
        line(f"/* atomic_add (sequential) */ (out[{_affine(k.output.offset, k.output.strides)}] += {loads[0]});")
        for _ in range(nd):
            close_loop()
    elif k.kclass == D.K_CONV2D:
        # What the reference's composition computes (crates/nn/src/functional/conv.rs:113-184):
        # the R_ kernel over the unfolded-and-permuted windows adds, for every output
        # position and channel, the products in (c, kh, kw) order; padding reads 0.0f.
        n, c, h, w_, co, kh, kw, pad = k.shape
        ho, wo = h + 2 * pad - kh + 1, w_ + 2 * pad - kw + 1
        relu = bool(k.flags & D.FLAG_RELU)
        if k.flags & D.FLAG_WGRAD:
            # dW[co][c][kh][kw] = sum over (n, oh, ow) of g[(n,oh,ow)][co] * x[n][c][oh+kh-pad][ow+kw-pad]:
            # the R_ kernel of the reference's gradient, reduce loop innermost in (n, oh, ow) order
            o = [op.offset for op in k.inputs]
            for d, e in enumerate((co, c, kh, kw)):
                open_loop(d, e)
            line("float acc;")
            line("acc = 0.0f;")
            pragma_done[0] = True
            for d, e in ((4, n), (5, ho), (6, wo)):
                open_loop(d, e)
            ih, iw = f"((ridx5 + ridx2) + {-pad})", f"((ridx6 + ridx3) + {-pad})"
            xv = f"buf0[{o[0]} + ((((ridx4 * {c}) + ridx1) * {h} + {ih}) * {w_} + {iw})]"
            if pad:
                xv = f"((((!({ih} < 0)) && ({ih} < {h})) && ((!({iw} < 0)) && ({iw} < {w_}))) ? {xv} : 0.0f)"
            if k.flags & D.FLAG_G_NCHW:
                gv = f"buf1[{o[1]} + ((((ridx4 * {co}) + ridx0) * {ho} + ridx5) * {wo} + ridx6)]"
            else:
                gv = f"buf1[{o[1]} + ((((ridx4 * {ho}) + ridx5) * {wo} + ridx6) * {co} + ridx0)]"
            line(f"acc = (acc + ({xv} * {gv}));")
            for _ in range(3):
                close_loop()
            line(f"out[{k.output.offset} + ((((ridx0 * {c}) + ridx1) * {kh} + ridx2) * {kw} + ridx3)] = acc;")
            for _ in range(4):
                close_loop()
            src += "}\n"
            return src
        for d, e in enumerate((n, ho, wo, co)):
            open_loop(d, e)
        line("float acc;")
        line("acc = 0.0f;")
        pragma_done[0] = True
        for d, e in ((4, c), (5, kh), (6, kw)):
            open_loop(d, e)
        ih, iw = f"((ridx1 + ridx5) + {-pad})", f"((ridx2 + ridx6) + {-pad})"
        o = [op.offset for op in k.inputs] + [0]
        xv = f"buf0[{o[0]} + ((((ridx0 * {c}) + ridx4) * {h} + {ih}) * {w_} + {iw})]"
        if pad:
            xv = f"((((!({ih} < 0)) && ({ih} < {h})) && ((!({iw} < 0)) && ({iw} < {w_}))) ? {xv} : 0.0f)"
        if k.flags & D.FLAG_WFLIP:      # forward weights [C, Co, KH, KW] read transposed and flipped
            wv = f"buf1[{o[1]} + ((((ridx4 * {co}) + ridx3) * {kh} + ({kh - 1} + (-1 * ridx5))) * {kw} + ({kw - 1} + (-1 * ridx6)))]"
        else:
            wv = f"buf1[{o[1]} + ((((ridx3 * {c}) + ridx4) * {kh} + ridx5) * {kw} + ridx6)]"
        line(f"acc = (acc + ({xv} * {wv}));")
        for _ in range(3):
            close_loop()
        val = f"(acc + buf2[{o[2]} + ridx3])" if len(k.inputs) == 3 else "acc"
        if relu:
            val = f"fmaxf({val}, 0.0f)"
        if k.flags & D.FLAG_NCHW:
            line(f"out[{k.output.offset} + ((((ridx0 * {co}) + ridx3) * {ho} + ridx1) * {wo} + ridx2)] = {val};")
        else:
            line(f"out[{k.output.offset} + ((((ridx0 * {ho}) + ridx1) * {wo} + ridx2) * {co} + ridx3)] = {val};")
        for _ in range(4):
            close_loop()
    elif k.kclass == D.K_MAXPOOL2D:
        # max_pool2d with stride = window (crates/nn/src/functional/pool.rs:117-160): the window tensor
        # unfold would materialise is read in place; the reduce over it is the R_ loop nest (acc = -inf,
        # acc = fmaxf(acc, tap) in row-major window order, src/lowerer/loop_gen.rs:87-151).  Gradient:
        # mask-times-gradient of the max reduce (src/grad/rules.rs:379-399) written where unfold's VJP
        # (src/grad/rules.rs:40-53) would scatter it -- every element lies in at most one window --
        # zero where no window covers the element, then the ReLU's mask when the taps were max(x, 0)
        planes, h, w_, win = k.shape
        ho, wo = h // win, w_ // win
        relu = bool(k.flags & D.FLAG_RELU)
        o = [op.offset for op in k.inputs]
        if not (k.flags & D.FLAG_POOL_GRAD):
            for d, e in enumerate((planes, ho, wo)):
                open_loop(d, e)
            line("float acc;")
            line("acc = (-INFINITY);")
            pragma_done[0] = True
            open_loop(3, win); open_loop(4, win)
            tap = f"buf0[{o[0]} + (((ridx0 * {h}) + ((ridx1 * {win}) + ridx3)) * {w_} + ((ridx2 * {win}) + ridx4))]"
            if relu:
                tap = f"fmaxf({tap}, 0.0f)"
            line(f"acc = fmaxf(acc, {tap});")
            close_loop(); close_loop()
            line(f"out[{k.output.offset} + (((ridx0 * {ho}) + ridx1) * {wo} + ridx2)] = acc;")
            for _ in range(3):
                close_loop()
        else:
            for d, e in enumerate((planes, h, w_)):
                open_loop(d, e)
            xv = f"buf1[{o[1]} + (((ridx0 * {h}) + ridx1) * {w_} + ridx2)]"
            win_i = f"(((ridx0 * {ho}) + (ridx1 / {win})) * {wo} + (ridx2 / {win}))"
            tap = f"fmaxf({xv}, 0.0f)" if relu else xv
            val = f"((({tap} < buf2[{o[2]} + {win_i}]) ? 0.0f : buf0[{o[0]} + {win_i}]))"
            val = f"(((ridx1 < {ho * win}) && (ridx2 < {wo * win})) ? {val} : 0.0f)"
            if relu:
                val = f"(({xv} < 0.0f) ? 0.0f : {val})"
            line(f"out[{k.output.offset} + (((ridx0 * {h}) + ridx1) * {w_} + ridx2)] = {val};")
            for _ in range(3):
                close_loop()
    elif k.kclass == D.K_SCAN:
        # generate_scan (src/lowerer/loop_gen.rs:237-327): loops before the axis outside, then
        # `acc = identity`, then the scan loop with the loops of the later dims INSIDE it; the body
        # updates the one accumulator and stores it at every position
        ax = k.reduce_axis
        for d in range(ax):
            open_loop(d, k.shape[d])
        line("float acc;")
        line(f"acc = {f32_literal(_IDENTITY[k.reduce_op])};")
        pragma_done[0] = True
        for d in range(ax, nd):
            open_loop(d, k.shape[d])
        val = render_expr(k.map, loads, fma) if k.map is not None else loads[0]
        line(f"acc = {_combine(k.reduce_op, 'acc', val, False, None)};")
        line(f"out[{_affine(k.output.offset, k.output.strides)}] = acc;")
        for _ in range(nd):
            close_loop()
    elif k.kclass == D.K_SOFTMAX_XENT:
        # log_softmax (crates/nn/src/functional/activation.rs:174-187: x - max, exp, sum, ln, subtract)
        # followed by cross_entropy_loss (loss.rs:32-65: multiply by the one-hot targets, sum over classes,
        # sum over the batch, scale), each step a loop nest of its own with f32 temporaries as the
        # reference's separate kernels have; then the gradient with respect to the logits
        n, c = k.shape
        sc = f32_literal(k.scalar)
        L2E, IL2E = f32_literal(D.LOG2_E), f"(1.0f / {f32_literal(D.LOG2_E)})"
        line("float total;")
        line("total = 0.0f;")
        pragma_done[0] = True           # one accumulator across the rows: sequential
        open_loop(0, n)
        line("float m;"); line("m = (-INFINITY);")
        open_loop(1, c); line(f"m = fmaxf(m, buf0[((ridx0 * {c}) + ridx1)]);"); close_loop()
        line("float s;"); line("s = 0.0f;")
        line("float ts;"); line("ts = 0.0f;")
        open_loop(1, c)
        line(f"s = (s + exp2f(((buf0[((ridx0 * {c}) + ridx1)] + (m * -1.0f)) * {L2E})));")
        line(f"ts = (ts + buf1[((ridx0 * {c}) + ridx1)]);")
        close_loop()
        line(f"float lse = (log2f(s) * {IL2E});")
        line("float acc;"); line("acc = 0.0f;")
        open_loop(1, c)
        line(f"float z = (buf0[((ridx0 * {c}) + ridx1)] + (m * -1.0f));")
        line(f"acc = (acc + (buf1[((ridx0 * {c}) + ridx1)] * (z + (lse * -1.0f))));")
        line(f"out[{D.XENT_GRAD_OFFSET} + ((ridx0 * {c}) + ridx1)] = ({sc} * (buf1[((ridx0 * {c}) + ridx1)] + (((exp2f((z * {L2E})) * (1.0f / s)) * ts) * -1.0f)));")
        close_loop()
        line("total = (total + acc);")
        close_loop()
        line(f"out[0] = ({sc} * total);")
    elif k.kclass == D.K_SGD:
        # host loop of SGD::step (crates/nn/src/optim/sgd.rs:91-95): p - lr*g
        open_loop(0, k.shape[0])
        line(f"out[ridx0] = (buf0[ridx0] - ({f32_literal(k.scalar)} * buf1[ridx0]));")
        close_loop()
    elif k.kclass == D.K_SGD_MOMENTUM:
        # crates/nn/src/optim/sgd.rs:84-89: v = momentum*v - lr*g; p = p + v (v kept between steps)
        open_loop(0, k.shape[0])
        line(f"buf2[ridx0] = (({f32_literal(k.hyper[0])} * buf2[ridx0]) - ({f32_literal(k.scalar)} * buf1[ridx0]));")
        line("out[ridx0] = (buf0[ridx0] + buf2[ridx0]);")
        close_loop()
    elif k.kclass == D.K_ADAM:
        # Adam::step (crates/nn/src/optim/adam.rs:104-147); f32::powi is the runtime's
        # repeated-squaring __powisf2
        b1, b2, eps = (f32_literal(h) for h in k.hyper[:3])
        src = src.replace("// === Kernel Functions ===\n", "// === Kernel Functions ===\n"
                          "static float powi_f32(float a, int b) {\n"
                          "    float r = 1.0f;\n"
                          "    while (1) { if (b & 1) r *= a; b /= 2; if (b == 0) break; a *= a; }\n"
                          "    return r;\n}\n")
        line("buf4[0] = (buf4[0] + 1);")
        line(f"float bias_correction1 = (1.0f - powi_f32({b1}, buf4[0]));")
        line(f"float bias_correction2 = (1.0f - powi_f32({b2}, buf4[0]));")
        open_loop(0, k.shape[0])
        line("float g = buf1[ridx0];")
        line(f"buf2[ridx0] = (({b1} * buf2[ridx0]) + ((1.0f - {b1}) * g));")
        line(f"buf3[ridx0] = (({b2} * buf3[ridx0]) + (((1.0f - {b2}) * g) * g));")
        line("float m_hat = (buf2[ridx0] / bias_correction1);")
        line("float v_hat = (buf3[ridx0] / bias_correction2);")
        line(f"out[ridx0] = (buf0[ridx0] - (({f32_literal(k.scalar)} * m_hat) / (sqrtf(v_hat) + {eps})));")
        close_loop()
    else:
        raise ValueError(f"kernel class {k.kclass}")
    src += "}\n"
    return src


def gcc_flags(openmp: bool, strict: bool = False) -> List[str]:
    if strict:
        # the optimizer steps are Rust host loops, not emitted C: IEEE f32, no contraction, no reassociation
        return ["-O2", "-ffp-contract=off", "-shared", "-fPIC"]
    flags = ["-O3", "-ffast-math", "-shared", "-fPIC"]
    if openmp:
        flags.insert(2, "-fopenmp")
    return flags


def compile_c(source: str, openmp: bool = False, strict: bool = False) -> str:
    """Compile with the reference's flags; returns the path of the .so (cached)."""
    os.makedirs(_CACHE_DIR, exist_ok=True)
    h = hashlib.sha256((source + str(openmp) + ("strict" if strict else "")).encode()).hexdigest()[:24]
    so = os.path.join(_CACHE_DIR, f"lib{h}.so")
    if not os.path.exists(so):
        cfile = os.path.join(_CACHE_DIR, f"k{h}.c")
        with open(cfile, "w") as f:
            f.write(source)
        tmp = so + f".{os.getpid()}.tmp"
        cmd = ["gcc"] + gcc_flags(openmp, strict) + ["-o", tmp, cfile, "-lm"]
        subprocess.run(cmd, check=True, capture_output=True)
        os.replace(tmp, so)
    return so


class OracleKernel:
    """A compiled oracle kernel; call with numpy inputs in parameter order."""

    def __init__(self, k: D.KernelDesc, openmp: bool = False, fma: bool = False):
        self.desc = k
        self.source = emit_kernel_c(k, "kernel", openmp, fma)
        strict = k.kclass in (D.K_SGD, D.K_SGD_MOMENTUM, D.K_ADAM)
        self.lib = ctypes.CDLL(compile_c(self.source, openmp and not strict, strict))
        self.fn = self.lib.kernel
        self.fn.restype = None

    def __call__(self, inputs: Sequence[np.ndarray], out: np.ndarray = None) -> np.ndarray:
        k = self.desc
        assert len(inputs) == len(k.inputs)
        args = []
        keep = []
        for a, o in zip(inputs, k.inputs):
            # optimizer state is updated in place: a conforming array is passed as it is
            a = np.ascontiguousarray(a, dtype=D.DTYPE_NP[o.dtype])
            keep.append(a)
            args.append(a.ctypes.data_as(ctypes.c_void_p))
        if out is None:
            # zero-initialised like CBuffer (crates/backend-c/src/buffer.rs:84-93)
            out = np.zeros(int(k.output.numel), dtype=D.DTYPE_NP[k.output.dtype])
        args.append(out.ctypes.data_as(ctypes.c_void_p))
        self.fn(*args)
        return out


def run(k: D.KernelDesc, inputs: Sequence[np.ndarray], openmp: bool = False,
        fma: bool = False) -> np.ndarray:
    return OracleKernel(k, openmp, fma)(inputs)


# ---- float64 evaluation (cross-check for cancellation-prone sums) ----------

def eval_f64(k: D.KernelDesc, inputs: Sequence[np.ndarray]) -> np.ndarray:
    """Evaluate an ELEMENTWISE / REDUCE / COPY descriptor in float64 with numpy.
    Used to show that CPU and GPU both sit within rounding of the exact result
    where sums cancel."""
    shape = tuple(k.shape)

    def affine(c, coef):
        idx = np.full(shape, c, dtype=np.int64)
        for d, s in enumerate(coef):
            if s:
                sh = [1] * len(shape)
                sh[d] = shape[d]
                idx = idx + (np.arange(shape[d], dtype=np.int64) * s).reshape(sh)
        return idx

    def view(a, op):
        a = np.asarray(a).reshape(-1)
        idx = affine(op.offset, op.strides)
        if not op.bounds:
            return a[idx].astype(np.float64)
        ok = np.ones(shape, dtype=bool)
        for b in op.bounds:           # a masked load reads the pad value where a bound fails
            e = affine(b.c, b.coef)
            ok &= (e >= b.lo) & (e < b.hi)
        return np.where(ok, a[np.where(ok, idx, 0)].astype(np.float64), np.float64(np.float32(op.pad_value)))

    loads = [view(a, o) for a, o in zip(inputs, k.inputs)]

    def ev(n):
        a = n.args
        if n.op == "w": return loads[n.value]
        if n.op == "const": return np.float64(np.float32(n.value))
        if n.op == "add": return ev(a[0]) + ev(a[1])
        if n.op == "mul": return ev(a[0]) * ev(a[1])
        if n.op == "max": return np.maximum(ev(a[0]), ev(a[1]))
        if n.op == "recip": return 1.0 / ev(a[0])
        if n.op == "sqrt": return np.sqrt(ev(a[0]))
        if n.op == "log2": return np.log2(ev(a[0]))
        if n.op == "exp2": return np.exp2(ev(a[0]))
        if n.op == "sin": return np.sin(ev(a[0]))
        if n.op == "floor": return np.floor(ev(a[0]))
        if n.op == "lt": return (ev(a[0]) < ev(a[1])).astype(np.float64)
        if n.op == "and": return ((ev(a[0]) != 0) & (ev(a[1]) != 0)).astype(np.float64)
        if n.op == "not": return (ev(a[0]) == 0).astype(np.float64)
        if n.op == "select": return np.where(ev(a[0]) != 0, ev(a[1]), ev(a[2]))
        if n.op == "fma": return ev(a[0]) * ev(a[1]) + ev(a[2])
        raise ValueError(n.op)

    val = ev(k.map) if k.map is not None else loads[0]
    val = np.broadcast_to(val, shape)
    if k.kclass == D.K_REDUCE:
        f = {D.R_SUM: np.sum, D.R_MAX: np.max, D.R_MIN: np.min, D.R_PROD: np.prod}[k.reduce_op]
        return f(val, axis=k.reduce_axis).reshape(-1)
    return np.ascontiguousarray(val).reshape(-1)
