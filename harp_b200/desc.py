"""Kernel descriptors: the language-neutral form of one lowered ``AstNode::Kernel``.

The reference lowers every surviving graph node to one loop-nest kernel
(src/lowerer/lower.rs:335-388).  A backend receives that kernel as an AST and,
in the reference, renders it to source text.  This backend instead receives the
same information as plain data:

* the iteration shape (loop bounds ``ridx0 .. ridxN``, src/lowerer/loop_gen.rs:51-68),
* per parameter an affine element index ``offset + sum_d stride_d * ridx_d``
  (src/lowerer/index_gen.rs:45-63) with optional bound conditions for padded
  views (src/lowerer/lower.rs:1145-1157),
* the ``map`` expression over ``Wildcard`` inputs (src/graph/ops.rs:69-95),
* an optional reduce op and axis (src/graph/node.rs:29-77).

``KernelDesc.to_c()`` packs it into the ``eb200_kernel_desc`` struct of
``include/eb200.h``.  The same Python object drives the CPU oracle, so both
sides always see identical kernels.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

MAX_DIMS = 8
MAX_INPUTS = 8
MAX_BOUNDS = 4
MAX_INSNS = 96

# eb200_dtype
F32, BOOL, I32, I64, F16, BF16 = 0, 1, 2, 3, 4, 5
DTYPE_SIZE = {F32: 4, BOOL: 1, I32: 4, I64: 8, F16: 2, BF16: 2}
DTYPE_NP = {F32: "float32", BOOL: "uint8", I32: "int32", I64: "int64", F16: "float16", BF16: "uint16"}   # bf16 travels as its bits


def bf16_bits(a) -> "np.ndarray":
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even (finite values)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_value(bits) -> "np.ndarray":
    """bfloat16 bit patterns (uint16) -> float32."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)

# eb200_kclass
K_ELEMENTWISE, K_REDUCE, K_COPY, K_SCATTER, K_SGD, K_CONV2D, K_SCAN, K_SGD_MOMENTUM, K_ADAM, K_SOFTMAX_XENT = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9
K_MAXPOOL2D = 10
KCLASS_PREFIX = {K_ELEMENTWISE: "E", K_REDUCE: "R", K_COPY: "C", K_SCATTER: "S", K_SGD: "U", K_CONV2D: "CONV",
                 K_SCAN: "P", K_SGD_MOMENTUM: "UM", K_ADAM: "UA", K_SOFTMAX_XENT: "XENT", K_MAXPOOL2D: "POOL"}
FLAG_RELU = 64
FLAG_WFLIP = 128
FLAG_POOL_GRAD = 128       # K_MAXPOOL2D: the gradient kernel
FLAG_WGRAD = 256
FLAG_NCHW = 512
FLAG_G_NCHW = 1024
FLAG_TENSOR_CORE = 2048

# eb200_reduce_op
R_NONE, R_SUM, R_MAX, R_MIN, R_PROD = 0, 1, 2, 3, 4

# eb200_gemm_mode
GEMM_DEFAULT, GEMM_TF32, GEMM_3XTF32 = 0, 1, 2

# eb200_opcode
(OP_LOAD, OP_CONST, OP_ADD, OP_MUL, OP_MAX, OP_RECIP, OP_SQRT, OP_LOG2, OP_EXP2,
 OP_SIN, OP_FLOOR, OP_LT, OP_AND, OP_NOT, OP_SELECT, OP_REM, OP_IDIV, OP_CAST,
 OP_FMA) = range(19)

_ARITY = {
    "add": 2, "mul": 2, "max": 2, "recip": 1, "sqrt": 1, "log2": 1, "exp2": 1,
    "sin": 1, "floor": 1, "lt": 2, "and": 2, "not": 1, "select": 3, "rem": 2,
    "idiv": 2, "cast": 1, "fma": 3,
}
_OPCODE = {
    "add": OP_ADD, "mul": OP_MUL, "max": OP_MAX, "recip": OP_RECIP, "sqrt": OP_SQRT,
    "log2": OP_LOG2, "exp2": OP_EXP2, "sin": OP_SIN, "floor": OP_FLOOR, "lt": OP_LT,
    "and": OP_AND, "not": OP_NOT, "select": OP_SELECT, "rem": OP_REM,
    "idiv": OP_IDIV, "cast": OP_CAST, "fma": OP_FMA,
}
_OPNAME = {v: k for k, v in _OPCODE.items()}

LOG2_E = float.fromhex("0x1.715476p+0")     # std::f32::consts::LOG2_E
FRAC_PI_2 = float.fromhex("0x1.921fb6p+0")  # std::f32::consts::FRAC_PI_2


class Ast:
    """A ``map`` expression tree over the reference's AST primitive set
    (src/ast/mod.rs:107-385).  ``Ast.w(i)`` is ``Wildcard("i")``."""

    __slots__ = ("op", "args", "value")

    def __init__(self, op: str, args: Tuple["Ast", ...] = (), value=None):
        self.op = op
        self.args = tuple(args)
        self.value = value

    # constructors ---------------------------------------------------------
    @staticmethod
    def w(i: int) -> "Ast":
        return Ast("w", (), int(i))

    @staticmethod
    def const(v: float) -> "Ast":
        return Ast("const", (), float(v))

    @staticmethod
    def of(x) -> "Ast":
        return x if isinstance(x, Ast) else Ast.const(x)

    def _bin(self, op, other):
        return Ast(op, (self, Ast.of(other)))

    # primitives -----------------------------------------------------------
    def __add__(self, o): return self._bin("add", o)
    def __mul__(self, o): return self._bin("mul", o)
    def maximum(self, o): return self._bin("max", o)
    def lt(self, o): return self._bin("lt", o)
    def logical_and(self, o): return self._bin("and", o)
    def logical_not(self): return Ast("not", (self,))
    def recip(self): return Ast("recip", (self,))
    def sqrt(self): return Ast("sqrt", (self,))
    def log2(self): return Ast("log2", (self,))
    def exp2(self): return Ast("exp2", (self,))
    def sin(self): return Ast("sin", (self,))
    def floor(self): return Ast("floor", (self,))
    def cast(self, dtype): return Ast("cast", (self,), int(dtype))

    @staticmethod
    def select(c, t, e): return Ast("select", (Ast.of(c), Ast.of(t), Ast.of(e)))

    @staticmethod
    def fma(a, b, c): return Ast("fma", (Ast.of(a), Ast.of(b), Ast.of(c)))

    # derived forms, spelled exactly as the reference spells them
    # (src/graph/ops.rs:151-367)
    def __sub__(self, o): return self + (Ast.of(o) * Ast.const(-1.0))
    def __truediv__(self, o): return self * Ast.of(o).recip()
    def __neg__(self): return self * Ast.const(-1.0)
    def exp(self): return (self * Ast.const(LOG2_E)).exp2()
    def ln(self): return self.log2() * Ast.const(LOG2_E).recip()
    def cos(self): return (self + Ast.const(FRAC_PI_2)).sin()

    # utilities ------------------------------------------------------------
    def substitute(self, mapping) -> "Ast":
        """Replace ``Wildcard(i)`` by ``mapping[i]`` (an ``Ast``): the
        substitution primitive of src/ast/mod.rs:1196-1207."""
        if self.op == "w":
            return mapping.get(self.value, self)
        if not self.args:
            return self
        return Ast(self.op, tuple(a.substitute(mapping) for a in self.args), self.value)

    def wildcards(self) -> List[int]:
        out: List[int] = []

        def rec(n):
            if n.op == "w":
                if n.value not in out:
                    out.append(n.value)
            for a in n.args:
                rec(a)
        rec(self)
        return out

    def postfix(self) -> List[Tuple[int, int, float]]:
        out: List[Tuple[int, int, float]] = []

        def rec(n):
            if n.op == "w":
                out.append((OP_LOAD, n.value, 0.0))
            elif n.op == "const":
                out.append((OP_CONST, 0, n.value))
            else:
                for a in n.args:
                    rec(a)
                out.append((_OPCODE[n.op], n.value if n.op == "cast" else 0, 0.0))
        rec(self)
        return out

    def key(self) -> str:
        """Canonical text of the expression (used to select compiled functors)."""
        if self.op == "w":
            return f"w{self.value}"
        if self.op == "const":
            return f"c({float32_hex(self.value)})"
        inner = ",".join(a.key() for a in self.args)
        if self.op == "cast":
            return f"cast{self.value}({inner})"
        return f"{self.op}({inner})"

    def __repr__(self):
        return self.key()


def float32_hex(v: float) -> str:
    import struct
    return "0x%08x" % struct.unpack("<I", struct.pack("<f", v))[0]


@dataclass
class Bound:
    """``lo <= c + sum_d coef[d]*idx[d] < hi``"""
    coef: Sequence[int]
    c: int
    lo: int
    hi: int


@dataclass
class Operand:
    """A kernel parameter as the loop nest addresses it."""
    strides: Sequence[int]
    offset: int = 0
    dtype: int = F32
    numel: int = 0
    bounds: List[Bound] = field(default_factory=list)
    pad_value: float = 0.0


@dataclass
class KernelDesc:
    kclass: int
    shape: Sequence[int]
    inputs: List[Operand]
    output: Operand
    map: Optional[Ast] = None
    reduce_op: int = R_NONE
    reduce_axis: int = 0
    gemm_mode: int = GEMM_DEFAULT
    scalar: float = 0.0
    name: str = ""
    flags: int = 0
    hyper: Sequence[float] = ()

    def __post_init__(self):
        self.shape = [int(s) for s in self.shape]
        nd = len(self.shape)
        if nd > MAX_DIMS:
            raise ValueError(f"rank {nd} exceeds {MAX_DIMS}")
        if len(self.inputs) > MAX_INPUTS:
            raise ValueError(f"{len(self.inputs)} inputs exceed {MAX_INPUTS}")
        for op in list(self.inputs) + [self.output]:
            if len(op.strides) != nd:
                raise ValueError("operand stride rank differs from iteration rank")
            if len(op.bounds) > MAX_BOUNDS:
                raise ValueError("too many bound conditions")
        if not self.name:
            # kernel naming of the lowerer: <prefix>_<shape>_<...> (lower.rs:227-273)
            self.name = KCLASS_PREFIX[self.kclass] + "_" + "_".join(str(s) for s in self.shape)

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def iter_numel(self) -> int:
        return math.prod(self.shape) if self.shape else 1

    def program(self) -> List[Tuple[int, int, float]]:
        return self.map.postfix() if self.map is not None else []

    def to_c(self) -> "CKernelDesc":
        d = CKernelDesc()
        d.kclass = self.kclass
        d.ndim = self.ndim
        for i, s in enumerate(self.shape):
            d.shape[i] = s
        d.n_inputs = len(self.inputs)
        d.reduce_op = self.reduce_op
        d.reduce_axis = self.reduce_axis
        d.gemm_mode = self.gemm_mode
        d.scalar = self.scalar
        d.flags = self.flags
        for i, h in enumerate(self.hyper):
            d.hyper[i] = float(h)
        prog = self.program()
        if len(prog) > MAX_INSNS:
            raise ValueError(f"map program of {len(prog)} instructions exceeds {MAX_INSNS}")
        d.n_insns = len(prog)
        for i, (op, arg, imm) in enumerate(prog):
            d.prog[i].op, d.prog[i].arg, d.prog[i].imm = op, arg, imm
        for i, o in enumerate(self.inputs):
            _fill_operand(d.inputs[i], o)
        _fill_operand(d.output, self.output)
        return d


    # ---- serialised form (golden files, ahead-of-time descriptor programs) ----------------
    def to_json(self) -> dict:
        def op(o: Operand):
            return {"dtype": o.dtype, "offset": int(o.offset), "strides": [int(x) for x in o.strides], "numel": int(o.numel),
                    "pad_value": float(o.pad_value),
                    "bounds": [{"coef": [int(c) for c in b.coef], "c": int(b.c), "lo": int(b.lo), "hi": int(b.hi)} for b in o.bounds]}
        return {"name": self.name, "kclass": self.kclass, "shape": list(self.shape), "inputs": [op(o) for o in self.inputs],
                "output": op(self.output), "reduce_op": self.reduce_op, "reduce_axis": self.reduce_axis,
                "gemm_mode": self.gemm_mode, "flags": self.flags, "scalar": float(self.scalar), "hyper": [float(h) for h in self.hyper],
                "prog": [[o, a, float32_hex(i)] for o, a, i in self.program()]}

    @staticmethod
    def from_json(j: dict) -> "KernelDesc":
        import struct

        def op(o):
            return Operand(o["strides"], o["offset"], o["dtype"], o["numel"],
                           [Bound(b["coef"], b["c"], b["lo"], b["hi"]) for b in o["bounds"]], o["pad_value"])
        stack: List[Ast] = []
        for opc, arg, imm in j["prog"]:
            v = struct.unpack("<f", struct.pack("<I", int(imm, 16)))[0]
            if opc == OP_LOAD:
                stack.append(Ast.w(arg))
            elif opc == OP_CONST:
                stack.append(Ast.const(v))
            else:
                name = _OPNAME[opc]
                n = _ARITY[name]
                args = stack[len(stack) - n:]
                del stack[len(stack) - n:]
                stack.append(Ast(name, tuple(args), arg if name == "cast" else None))
        return KernelDesc(j["kclass"], j["shape"], [op(o) for o in j["inputs"]], op(j["output"]), stack[0] if stack else None,
                          j["reduce_op"], j["reduce_axis"], j["gemm_mode"], j["scalar"], j["name"], j["flags"], j["hyper"])


def _fill_operand(c, o: Operand):
    c.dtype = o.dtype
    c.n_bounds = len(o.bounds)
    c.offset = o.offset
    for i, s in enumerate(o.strides):
        c.strides[i] = int(s)
    c.numel = int(o.numel)
    c.pad_value = o.pad_value
    for j, b in enumerate(o.bounds):
        for i, k in enumerate(b.coef):
            c.bounds[j].coef[i] = int(k)
        c.bounds[j].c, c.bounds[j].lo, c.bounds[j].hi = int(b.c), int(b.lo), int(b.hi)


# ---- ctypes mirrors of include/eb200.h ------------------------------------

class CInsn(C.Structure):
    _fields_ = [("op", C.c_int32), ("arg", C.c_int32), ("imm", C.c_float), ("_pad", C.c_int32)]


class CBound(C.Structure):
    _fields_ = [("coef", C.c_int64 * MAX_DIMS), ("c", C.c_int64), ("lo", C.c_int64), ("hi", C.c_int64)]


class COperand(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("n_bounds", C.c_int32), ("offset", C.c_int64),
        ("strides", C.c_int64 * MAX_DIMS), ("numel", C.c_int64),
        ("pad_value", C.c_float), ("_pad", C.c_int32),
        ("bounds", CBound * MAX_BOUNDS),
    ]


class CKernelDesc(C.Structure):
    _fields_ = [
        ("kclass", C.c_int32), ("ndim", C.c_int32), ("shape", C.c_int64 * MAX_DIMS),
        ("n_inputs", C.c_int32), ("reduce_op", C.c_int32), ("reduce_axis", C.c_int32),
        ("n_insns", C.c_int32), ("gemm_mode", C.c_int32), ("flags", C.c_int32),
        ("scalar", C.c_float), ("hyper", C.c_float * 7),
        ("inputs", COperand * MAX_INPUTS), ("output", COperand),
        ("prog", CInsn * MAX_INSNS),
    ]


class CDeviceProps(C.Structure):
    _fields_ = [
        ("name", C.c_char * 128), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
        ("sm_count", C.c_int32), ("_pad", C.c_int32), ("total_mem_bytes", C.c_int64),
        ("l2_bytes", C.c_int64), ("smem_per_block_optin", C.c_int64),
    ]


class CKernelInfo(C.Structure):
    _fields_ = [
        ("impl", C.c_char * 64), ("launches", C.c_int32), ("specialised", C.c_int32),
        ("scratch_bytes", C.c_int64), ("algo_bytes", C.c_int64), ("algo_flops", C.c_int64),
    ]


# ---- convenience constructors ---------------------------------------------

def contiguous_strides(shape: Sequence[int]) -> List[int]:
    """Row-major strides, as View::contiguous (src/graph/shape/view.rs:1437-1470)."""
    st, acc = [], 1
    for s in reversed(list(shape)):
        st.append(acc)
        acc *= int(s)
    return list(reversed(st))


def contiguous(shape: Sequence[int], dtype: int = F32) -> Operand:
    return Operand(contiguous_strides(shape), 0, dtype, math.prod(shape) if len(shape) else 1)


def elementwise(shape, inputs: List[Operand], expr: Ast, out: Optional[Operand] = None,
                out_dtype: int = F32) -> KernelDesc:
    return KernelDesc(K_ELEMENTWISE, shape, inputs, out or contiguous(shape, out_dtype), expr)


def reduce(shape, inputs: List[Operand], expr: Ast, op: int, axis: int,
           out: Optional[Operand] = None, gemm_mode: int = GEMM_DEFAULT) -> KernelDesc:
    """Output addressed by the node view with the reduce index forced to 0
    (src/lowerer/index_gen.rs:107-112): contiguous over the kept-dim shape."""
    if out is None:
        kept = [1 if d == axis else s for d, s in enumerate(shape)]
        st = contiguous_strides(kept)
        st[axis] = 0
        out = Operand(st, 0, F32, math.prod(kept))
    return KernelDesc(K_REDUCE, shape, inputs, out, expr, op, axis, gemm_mode)


def scan(shape, inputs: List[Operand], expr: Ast, op: int, axis: int, out: Optional[Operand] = None) -> KernelDesc:
    """Cumulative op along `axis` (P_ kernel, src/lowerer/lower.rs:691-735); the
    output has the iteration shape."""
    return KernelDesc(K_SCAN, shape, inputs, out or contiguous(shape), expr, op, axis)


def sgd_momentum(n: int, lr: float, momentum: float) -> KernelDesc:
    """SGD with momentum over flat buffers (crates/nn/src/optim/sgd.rs:84-89):
    inputs p, g, v (v updated in place), output p."""
    return KernelDesc(K_SGD_MOMENTUM, [n], [contiguous([n])] * 3, contiguous([n]), scalar=lr, hyper=[momentum])


def adam(n: int, lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8) -> KernelDesc:
    """Adam over flat buffers (crates/nn/src/optim/adam.rs:104-147): inputs p, g, m, v
    and the one-element I32 step counter (m, v, t updated in place), output p."""
    ins = [contiguous([n])] * 4 + [Operand([0], 0, I32, 1)]
    return KernelDesc(K_ADAM, [n], ins, contiguous([n]), scalar=lr, hyper=[beta1, beta2, eps])


XENT_GRAD_OFFSET = 64     # where the gradient starts in a K_SOFTMAX_XENT output (element 0 is the loss)


def softmax_xent(n: int, c: int, scale: float) -> KernelDesc:
    """scale * sum(onehot * log_softmax(logits)) and its gradient with respect to the
    logits as one kernel (crates/nn/src/functional/activation.rs:174-187, loss.rs:32-65)."""
    z2 = [0, 0]
    return KernelDesc(K_SOFTMAX_XENT, [n, c], [Operand(z2, 0, F32, n * c), Operand(z2, 0, F32, n * c)],
                      Operand(z2, 0, F32, XENT_GRAD_OFFSET + n * c), None, scalar=scale)


def maxpool2d(p: int, h: int, w: int, k: int, relu: bool = False, grad: bool = False) -> KernelDesc:
    """functional::max_pool2d with stride = window (crates/nn/src/functional/pool.rs:117-160)
    over P = N*C planes as one kernel: x [P, H, W] -> y [P, H//k, W//k]; `relu`: the taps are
    max(x, 0); `grad`: inputs g, x, y -> gx [P, H, W] (with `relu` the activation's gradient
    mask is applied too)."""
    z4 = [0] * 4
    full, pooled = p * h * w, p * (h // k) * (w // k)
    ins = [Operand(z4, 0, F32, pooled), Operand(z4, 0, F32, full), Operand(z4, 0, F32, pooled)] if grad else [Operand(z4, 0, F32, full)]
    return KernelDesc(K_MAXPOOL2D, [p, h, w, k], ins, Operand(z4, 0, F32, full if grad else pooled), None,
                      flags=(FLAG_RELU if relu else 0) | (FLAG_POOL_GRAD if grad else 0))


def copy(shape, src: Operand, out: Optional[Operand] = None) -> KernelDesc:
    return KernelDesc(K_COPY, shape, [src], out or contiguous(shape, src.dtype), None)


def conv2d(n, c, h, w, co, kh, kw, pad=0, bias=True, relu=False, mode: int = GEMM_DEFAULT, flip=False, nchw=False) -> KernelDesc:
    """functional::conv2d (crates/nn/src/functional/conv.rs:113-184) as one kernel:
    x [N,C,H,W], weight [Co,C,KH,KW] (, bias [Co]) -> [N*Ho*Wo, Co] row-major, the
    buffer the reference's GEMM step produces (its result is a permuted view of it).
    `flip`: the weight buffer holds [C, Co, KH, KW] (the forward layer's weights) and is
    read transposed and flipped: the input-gradient convolution."""
    ho, wo = h + 2 * pad - kh + 1, w + 2 * pad - kw + 1
    z8 = [0] * 8
    ins = [Operand(z8, 0, F32, n * c * h * w), Operand(z8, 0, F32, co * c * kh * kw)]
    if bias:
        ins.append(Operand(z8, 0, F32, co))
    return KernelDesc(K_CONV2D, [n, c, h, w, co, kh, kw, pad], ins, Operand(z8, 0, F32, n * ho * wo * co),
                      None, gemm_mode=mode, flags=(FLAG_RELU if relu else 0) | (FLAG_WFLIP if flip else 0) | (FLAG_NCHW if nchw else 0))


def conv2d_wgrad(n, c, h, w, co, kh, kw, pad=0, mode: int = GEMM_DEFAULT, g_nchw=False) -> KernelDesc:
    """Weight gradient of ``conv2d``: x [N,C,H,W] and the output gradient [N*Ho*Wo, Co]
    -> dW [Co,C,KH,KW], the unfolded input never materialised.  `g_nchw`: the gradient is
    given as [N,Co,Ho,Wo] instead (layers with C*KH*KW <= 12 only)."""
    ho, wo = h + 2 * pad - kh + 1, w + 2 * pad - kw + 1
    z8 = [0] * 8
    ins = [Operand(z8, 0, F32, n * c * h * w), Operand(z8, 0, F32, n * ho * wo * co)]
    return KernelDesc(K_CONV2D, [n, c, h, w, co, kh, kw, pad], ins, Operand(z8, 0, F32, co * c * kh * kw),
                      None, gemm_mode=mode, flags=FLAG_WGRAD | (FLAG_G_NCHW if g_nchw else 0))
