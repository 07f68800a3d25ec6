//! `AstNode::Kernel` -> `eb200_kernel_desc`: a mechanical walk with no arithmetic in it.
//!
//! The lowerer (src/lowerer/lower.rs:335-388) hands a backend one loop-nest kernel at
//! a time.  Its shapes, as produced at ECLAT_OPT_LEVEL=0 (no AST rewrites):
//!
//! * `E_` / `C_` (lower.rs:448-522): nested `Range ridxN`, innermost body
//!   `Store { ptr: Var(out), offset: index, value: map }`;
//! * `R_` (lower.rs:525-571, loop_gen.rs:87-151): outer ranges, then a block
//!   `acc = identity; Range ridx<axis> { acc = combine(acc, map) }; Store(out, index, acc)`;
//! * `P_` (lower.rs:691-735, loop_gen.rs:237-327): ranges before the axis, then
//!   `acc = identity; Range ridx<axis> { Range inner.. { acc = combine(acc, map); Store(out, index, acc) } }`;
//! * `S_` (lower.rs:580-683): a zero-fill nest, then a nest whose body is
//!   `AtomicAdd { ptr: Var(out), offset: dst index, value: load }`.
//!
//! Loads are `Load { ptr: Var(buffer), offset: index }`, wrapped in
//! `Select { cond, load, Const(pad) }` for padded views (lower.rs:1145-1157), where `cond`
//! is an `And` chain of `Not(Lt(e, lo))` / `Lt(e, hi)` over affine `e`
//! (src/graph/shape/view.rs:997-1011).  Index expressions are sums of
//! `ridxN * stride` terms and constants (src/lowerer/index_gen.rs:45-63,
//! src/graph/shape/expr.rs:62-105).  Anything that does not have this shape is
//! reported as unsupported; nothing is guessed.
//!
//! Parameter order (lower.rs:1047-1105): input buffers (immutable pointers) in source
//! order, then the output (mutable pointer), then i64 shape symbols (not supported yet).
//!
//! Written without a Rust toolchain at hand: this file has not been compiled.
//! `tests/golden/kernels.json` in the backend's repository pairs descriptors with the C
//! the C backend is expected to render for the same kernels; diff it against the real
//! renderer's output first.

use eclat::ast::{AstNode, DType, Literal, Mutability};

use crate::ffi::*;

#[derive(Debug)]
pub struct Unsupported(pub String);

fn unsupported<T>(what: impl Into<String>) -> Result<T, Unsupported> {
    Err(Unsupported(what.into()))
}

/// offset + sum strides[d] * ridx_d
#[derive(Clone, Debug, Default, PartialEq)]
struct Affine {
    offset: i64,
    coef: [i64; MAX_DIMS],
}

fn loop_axis(var: &str) -> Option<usize> {
    var.strip_prefix("ridx").and_then(|n| n.parse::<usize>().ok()).filter(|&n| n < MAX_DIMS)
}

fn const_i64(n: &AstNode) -> Option<i64> {
    match n {
        AstNode::Const(Literal::I64(v)) => Some(*v),
        AstNode::Const(Literal::I32(v)) => Some(*v as i64),
        AstNode::Const(Literal::U64(v)) => Some(*v as i64),
        _ => None,
    }
}

fn affine(n: &AstNode) -> Result<Affine, Unsupported> {
    match n {
        AstNode::Var(v) => {
            let d = loop_axis(v).ok_or_else(|| Unsupported(format!("index variable {v}")))?;
            let mut a = Affine::default();
            a.coef[d] = 1;
            Ok(a)
        }
        AstNode::Add(x, y) => {
            let (a, b) = (affine(x)?, affine(y)?);
            let mut r = Affine { offset: a.offset + b.offset, ..Default::default() };
            for d in 0..MAX_DIMS { r.coef[d] = a.coef[d] + b.coef[d]; }
            Ok(r)
        }
        AstNode::Mul(x, y) => {
            let (a, b) = (affine(x)?, affine(y)?);
            let (k, v) = if a.coef.iter().all(|&c| c == 0) { (a.offset, b) }
                         else if b.coef.iter().all(|&c| c == 0) { (b.offset, a) }
                         else { return unsupported("product of two loop variables in an index") };
            let mut r = Affine { offset: k * v.offset, ..Default::default() };
            for d in 0..MAX_DIMS { r.coef[d] = k * v.coef[d]; }
            Ok(r)
        }
        other => const_i64(other).map(|v| Affine { offset: v, ..Default::default() })
            .ok_or_else(|| Unsupported(format!("index expression {other:?}"))),
    }
}

fn dtype_code(dt: &DType) -> Result<i32, Unsupported> {
    match dt {
        DType::F32 => Ok(F32),
        DType::Bool => Ok(BOOL),
        DType::I32 => Ok(I32),
        DType::I64 => Ok(I64),
        DType::F16 => Ok(F16),
        DType::BF16 => Ok(BF16),
        other => unsupported(format!("element type {other:?}")),
    }
}

struct Walk<'a> {
    inputs: Vec<&'a str>,          // immutable pointer params, in order
    in_dtypes: Vec<i32>,
    desc: eb200_kernel_desc,
    operands: Vec<eb200_operand>,  // deduplicated (buffer, view) pairs in first-use order
    operand_buf: Vec<usize>,       // which input buffer each operand reads
}

impl<'a> Walk<'a> {
    fn push(&mut self, op: i32, arg: i32, imm: f32) -> Result<(), Unsupported> {
        let n = self.desc.n_insns as usize;
        if n >= MAX_INSNS { return unsupported("map longer than the descriptor's program"); }
        self.desc.prog[n] = eb200_insn { op, arg, imm, _pad: 0 };
        self.desc.n_insns += 1;
        Ok(())
    }

    /// bounds of a padded load: And chain of Not(Lt(e, lo)) and Lt(e, hi)
    fn bounds(&self, cond: &AstNode, out: &mut Vec<(Affine, Option<i64>, Option<i64>)>) -> Result<(), Unsupported> {
        match cond {
            AstNode::And(a, b) => { self.bounds(a, out)?; self.bounds(b, out) }
            AstNode::Not(inner) => match inner.as_ref() {
                AstNode::Lt(e, lo) => { out.push((affine(e)?, const_i64(lo), None)); Ok(()) }
                other => unsupported(format!("bound condition {other:?}")),
            },
            AstNode::Lt(e, hi) => { out.push((affine(e)?, None, const_i64(hi))); Ok(()) }
            other => unsupported(format!("bound condition {other:?}")),
        }
    }

    fn load(&mut self, ptr: &AstNode, offset: &AstNode, cond: Option<&AstNode>, pad: f32) -> Result<(), Unsupported> {
        let name = match ptr { AstNode::Var(v) => v.as_str(), other => return unsupported(format!("load through {other:?}")) };
        let buf = self.inputs.iter().position(|b| *b == name).ok_or_else(|| Unsupported(format!("load from unknown buffer {name}")))?;
        let a = affine(offset)?;
        let mut op = eb200_operand::default();
        op.dtype = self.in_dtypes[buf];
        op.offset = a.offset;
        op.strides = a.coef;
        op.pad_value = pad;
        if let Some(c) = cond {
            let mut terms = Vec::new();
            self.bounds(c, &mut terms)?;
            // lower and upper halves over the same expression merge into one bound
            let mut merged: Vec<(Affine, i64, i64)> = Vec::new();
            for (e, lo, hi) in terms {
                if let Some(m) = merged.iter_mut().find(|m| m.0.coef == e.coef && m.0.offset == e.offset) {
                    if let Some(l) = lo { m.1 = m.1.max(l); }
                    if let Some(h) = hi { m.2 = m.2.min(h); }
                } else {
                    merged.push((e, lo.unwrap_or(i64::MIN / 2), hi.unwrap_or(i64::MAX / 2)));
                }
            }
            if merged.len() > MAX_BOUNDS { return unsupported("more bound conditions than the descriptor holds"); }
            for (j, (e, lo, hi)) in merged.into_iter().enumerate() {
                op.bounds[j] = eb200_bound { coef: e.coef, c: e.offset, lo, hi };
            }
            op.n_bounds = op.bounds.iter().filter(|b| b.lo != 0 || b.hi != 0 || b.c != 0 || b.coef.iter().any(|&c| c != 0)).count() as i32;
        }
        // the same buffer through the same view is one operand (lower.rs:1047-1105 deduplicates buffers; views may differ)
        let idx = match (0..self.operands.len()).find(|&i| self.operand_buf[i] == buf && same_view(&self.operands[i], &op)) {
            Some(i) => i,
            None => {
                if self.operands.len() >= MAX_INPUTS { return unsupported("more operands than the descriptor holds"); }
                self.operands.push(op);
                self.operand_buf.push(buf);
                self.operands.len() - 1
            }
        };
        self.push(OP_LOAD, idx as i32, 0.0)
    }

    /// post-order emission of the map expression
    fn expr(&mut self, n: &AstNode) -> Result<(), Unsupported> {
        match n {
            AstNode::Load { ptr, offset, count: 1, .. } => self.load(ptr, offset, None, 0.0),
            AstNode::Select { cond, then_val, else_val } => {
                // a padded load, or a genuine select
                if let (AstNode::Load { ptr, offset, count: 1, .. }, AstNode::Const(Literal::F32(pad))) = (then_val.as_ref(), else_val.as_ref()) {
                    if is_bound_condition(cond) { return self.load(ptr, offset, Some(cond), *pad); }
                }
                self.expr(cond)?; self.expr(then_val)?; self.expr(else_val)?;
                self.push(OP_SELECT, 0, 0.0)
            }
            AstNode::Const(Literal::F32(v)) => self.push(OP_CONST, 0, *v),
            AstNode::Const(Literal::Bool(b)) => self.push(OP_CONST, 0, if *b { 1.0 } else { 0.0 }),
            AstNode::Const(other) => const_i64(&AstNode::Const(other.clone())).map(|v| v as f32)
                .ok_or_else(|| Unsupported(format!("literal {other:?}"))).and_then(|v| self.push(OP_CONST, 0, v)),
            AstNode::Add(a, b) => { self.expr(a)?; self.expr(b)?; self.push(OP_ADD, 0, 0.0) }
            AstNode::Mul(a, b) => { self.expr(a)?; self.expr(b)?; self.push(OP_MUL, 0, 0.0) }
            AstNode::Max(a, b) => { self.expr(a)?; self.expr(b)?; self.push(OP_MAX, 0, 0.0) }
            AstNode::Rem(a, b) => { self.expr(a)?; self.expr(b)?; self.push(OP_REM, 0, 0.0) }
            AstNode::Idiv(a, b) => { self.expr(a)?; self.expr(b)?; self.push(OP_IDIV, 0, 0.0) }
            AstNode::Lt(a, b) => { self.expr(a)?; self.expr(b)?; self.push(OP_LT, 0, 0.0) }
            AstNode::And(a, b) => { self.expr(a)?; self.expr(b)?; self.push(OP_AND, 0, 0.0) }
            AstNode::Not(a) => { self.expr(a)?; self.push(OP_NOT, 0, 0.0) }
            AstNode::Recip(a) => { self.expr(a)?; self.push(OP_RECIP, 0, 0.0) }
            AstNode::Sqrt(a) => { self.expr(a)?; self.push(OP_SQRT, 0, 0.0) }
            AstNode::Log2(a) => { self.expr(a)?; self.push(OP_LOG2, 0, 0.0) }
            AstNode::Exp2(a) => { self.expr(a)?; self.push(OP_EXP2, 0, 0.0) }
            AstNode::Sin(a) => { self.expr(a)?; self.push(OP_SIN, 0, 0.0) }
            AstNode::Floor(a) => { self.expr(a)?; self.push(OP_FLOOR, 0, 0.0) }
            AstNode::Cast(a, dt) => { self.expr(a)?; let c = dtype_code(dt)?; self.push(OP_CAST, c, 0.0) }
            AstNode::Fma { a, b, c } => { self.expr(a)?; self.expr(b)?; self.expr(c)?; self.push(OP_FMA, 0, 0.0) }
            other => unsupported(format!("map node {other:?}")),
        }
    }
}

fn same_view(a: &eb200_operand, b: &eb200_operand) -> bool {
    a.offset == b.offset && a.strides == b.strides && a.n_bounds == b.n_bounds && a.pad_value == b.pad_value
        && (0..a.n_bounds as usize).all(|j| a.bounds[j].coef == b.bounds[j].coef && a.bounds[j].c == b.bounds[j].c
            && a.bounds[j].lo == b.bounds[j].lo && a.bounds[j].hi == b.bounds[j].hi)
}

fn is_bound_condition(c: &AstNode) -> bool {
    match c {
        AstNode::And(a, b) => is_bound_condition(a) && is_bound_condition(b),
        AstNode::Not(inner) => matches!(inner.as_ref(), AstNode::Lt(e, k) if affine(e).is_ok() && const_i64(k).is_some()),
        AstNode::Lt(e, k) => affine(e).is_ok() && const_i64(k).is_some(),
        _ => false,
    }
}

fn statements(n: &AstNode) -> Vec<&AstNode> {
    match n {
        AstNode::Block { statements, .. } => statements.iter().collect(),
        other => vec![other],
    }
}

/// `acc = combine(acc, map)`: which reduce op, and the map
fn split_combine<'a>(value: &'a AstNode, acc: &str) -> Result<(i32, &'a AstNode), Unsupported> {
    let is_acc = |n: &AstNode| matches!(n, AstNode::Var(v) if v == acc);
    match value {
        AstNode::Add(a, b) if is_acc(a) => Ok((R_SUM, b.as_ref())),
        AstNode::Max(a, b) if is_acc(a) => Ok((R_MAX, b.as_ref())),
        AstNode::Mul(a, b) if is_acc(a) => Ok((R_PROD, b.as_ref())),
        // ReduceOp::Min combines with Select(Lt(acc, v), acc, v) (src/graph/node.rs:67-74)
        AstNode::Select { cond, then_val, else_val } if is_acc(then_val) => match cond.as_ref() {
            AstNode::Lt(a, _) if is_acc(a) => Ok((R_MIN, else_val.as_ref())),
            _ => unsupported("select-shaped combine that is not min"),
        },
        // the backend-side a*b+c -> fma rule (src/opt/ast/rules/mod.rs:115-143) on a sum of products
        AstNode::Fma { c, .. } if is_acc(c) => unsupported("fma-rewritten combine: run with ECLAT_OPT_LEVEL=0"),
        other => unsupported(format!("reduce combine {other:?}")),
    }
}

/// The descriptor of one lowered kernel, the names of its input buffers in parameter order
/// and, for each descriptor operand, which of those buffers it reads (a buffer read through
/// two different views appears as two operands).
pub struct Lowered {
    pub desc: eb200_kernel_desc,
    pub operand_buffer: Vec<usize>,
}

pub fn lower_kernel_to_desc(kernel: &AstNode, numel_of: &dyn Fn(&str) -> Option<i64>) -> Result<Lowered, Unsupported> {
    let (name, params, body) = match kernel {
        AstNode::Kernel { name, params, body, .. } => (name.clone().unwrap_or_default(), params, body.as_ref()),
        _ => return unsupported("not a Kernel node"),
    };
    let mut w = Walk { inputs: vec![], in_dtypes: vec![], desc: eb200_kernel_desc::default(), operands: vec![], operand_buf: vec![] };
    let mut out_name: Option<&str> = None;
    let mut out_dtype = F32;
    for p in params {
        match (&p.dtype, &p.mutability) {
            (DType::Ptr(inner), Mutability::Immutable) => { w.inputs.push(p.name.as_str()); w.in_dtypes.push(dtype_code(inner)?); }
            (DType::Ptr(inner), Mutability::Mutable) => {
                if out_name.is_some() { return unsupported("kernel with more than one output"); }
                out_name = Some(p.name.as_str());
                out_dtype = dtype_code(inner)?;
            }
            _ => return unsupported(format!("non-pointer kernel parameter {} (dynamic shape symbols are not served yet)", p.name)),
        }
    }
    let out_name = out_name.ok_or_else(|| Unsupported("kernel without an output".into()))?;

    // walk down the loop nest
    let mut shape = [1i64; MAX_DIMS];
    let mut ndim = 0usize;
    let mut cur = body;
    let mut acc: Option<(String, i32)> = None;      // (accumulator name, reduce op) once an `acc = identity` is met
    let mut reduce_axis: Option<usize> = None;
    let mut is_scan = false;
    let mut scatter = false;
    loop {
        let stmts = statements(cur);
        match stmts.as_slice() {
            [AstNode::Range { var, stop, body, .. }] => {
                let d = loop_axis(var).ok_or_else(|| Unsupported(format!("loop variable {var}")))?;
                shape[d] = const_i64(stop).ok_or_else(|| Unsupported("symbolic loop bound".into()))?;
                ndim = ndim.max(d + 1);
                if acc.is_some() && reduce_axis.is_none() { reduce_axis = Some(d); }
                cur = body.as_ref();
            }
            // R_: acc = identity; Range { acc = combine }; Store(out, idx, acc)
            [AstNode::Assign { var, .. }, AstNode::Range { var: rvar, stop, body: rbody, .. }, AstNode::Store { offset, .. }] => {
                let d = loop_axis(rvar).ok_or_else(|| Unsupported(format!("loop variable {rvar}")))?;
                shape[d] = const_i64(stop).ok_or_else(|| Unsupported("symbolic loop bound".into()))?;
                ndim = ndim.max(d + 1);
                let inner = statements(rbody.as_ref());
                let value = match inner.as_slice() {
                    [AstNode::Assign { var: v2, value }] if v2 == var => value.as_ref(),
                    _ => return unsupported("reduce loop body"),
                };
                let (rop, map) = split_combine(value, var)?;
                w.expr(map)?;
                w.desc.kclass = K_REDUCE;
                w.desc.reduce_op = rop;
                w.desc.reduce_axis = d as i32;
                let a = affine(offset)?;
                w.desc.output.offset = a.offset;
                w.desc.output.strides = a.coef;
                break;
            }
            // P_: acc = identity; Range(axis) { [Range inner..] { acc = combine; Store } }
            [AstNode::Assign { var, .. }, AstNode::Range { .. }] => {
                acc = Some((var.clone(), R_NONE));
                is_scan = true;
                cur = stmts[1];
                // re-enter the loop on the Range itself
                if let AstNode::Range { var: rvar, stop, body, .. } = cur {
                    let d = loop_axis(rvar).ok_or_else(|| Unsupported(format!("loop variable {rvar}")))?;
                    shape[d] = const_i64(stop).ok_or_else(|| Unsupported("symbolic loop bound".into()))?;
                    ndim = ndim.max(d + 1);
                    reduce_axis = Some(d);
                    cur = body.as_ref();
                }
            }
            [AstNode::Assign { var, value }, AstNode::Store { offset, .. }] if is_scan => {
                let (rop, map) = split_combine(value, var)?;
                w.expr(map)?;
                w.desc.kclass = K_SCAN;
                w.desc.reduce_op = rop;
                w.desc.reduce_axis = reduce_axis.unwrap_or(0) as i32;
                let a = affine(offset)?;
                w.desc.output.offset = a.offset;
                w.desc.output.strides = a.coef;
                break;
            }
            // E_ / C_
            [AstNode::Store { ptr, offset, value }] => {
                if !matches!(ptr.as_ref(), AstNode::Var(v) if v == out_name) { return unsupported("store to a buffer that is not the output"); }
                w.expr(value)?;
                let identity = w.desc.n_insns == 1 && w.desc.prog[0].op == OP_LOAD;
                w.desc.kclass = if identity && name.starts_with("C_") { K_COPY } else { K_ELEMENTWISE };
                if w.desc.kclass == K_COPY { w.desc.n_insns = 0; }
                let a = affine(offset)?;
                w.desc.output.offset = a.offset;
                w.desc.output.strides = a.coef;
                break;
            }
            // S_: [zero-fill nest, accumulate nest]
            [AstNode::Range { .. }, second @ AstNode::Range { .. }] if !scatter => {
                scatter = true;
                cur = second;
            }
            [AstNode::AtomicAdd { ptr, offset, value, .. }] if scatter => {
                if !matches!(ptr.as_ref(), AstNode::Var(v) if v == out_name) { return unsupported("scatter into a buffer that is not the output"); }
                w.expr(value)?;
                if !(w.desc.n_insns == 1 && w.desc.prog[0].op == OP_LOAD) { return unsupported("scatter-add with a map"); }
                w.desc.n_insns = 0;
                w.desc.kclass = K_SCATTER;
                let a = affine(offset)?;
                w.desc.output.offset = a.offset;
                w.desc.output.strides = a.coef;
                break;
            }
            _ => return unsupported(format!("kernel body shape in {name}")),
        }
    }
    if scatter {
        // the nest that was walked is the accumulate nest; restart the shape from it
        // (the zero-fill nest runs over the output, which the library zero-fills itself)
    }
    w.desc.ndim = ndim as i32;
    w.desc.shape = shape;
    w.desc.n_inputs = w.operands.len() as i32;
    for (i, mut op) in w.operands.clone().into_iter().enumerate() {
        op.numel = numel_of(w.inputs[w.operand_buf[i]]).ok_or_else(|| Unsupported("input buffer of unknown size".into()))?;
        w.desc.inputs[i] = op;
    }
    w.desc.output.dtype = out_dtype;
    w.desc.output.numel = numel_of(out_name).ok_or_else(|| Unsupported("output buffer of unknown size".into()))?;
    Ok(Lowered { desc: w.desc, operand_buffer: w.operand_buf })
}
