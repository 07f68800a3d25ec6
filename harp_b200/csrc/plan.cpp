// Kernel-class dispatch: descriptor -> plan.
//
// The reference decides the kernel class in Lowerer::lower_node
// (src/lowerer/lower.rs:335-388) and then emits a loop nest for it.  Here the
// loop nest arrives as an eb200_kernel_desc and this file decides which
// hand-written kernel serves it:
//
//   E_ (elementwise)            -> ew (vectorised fused chain)
//   E_/C_ identity over a view  -> transpose (shared-memory tiles) or ew gather
//   R_ (reduce)                 -> gemm      if it is sum(mul(A,B)) over two broadcast views
//                                  reduce_inner if the reduce dim is innermost
//                                  reduce_outer otherwise (also the generic fallback)
//   S_ (scatter-add / fold)     -> scatter
//
// Pure host logic: no CUDA calls, so it is unit-testable without a GPU.
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "common.h"

namespace eb200 {

namespace {

struct Op {
    int dtype;
    long long offset;
    long long strides[KMAX_DIMS];
    long long numel;
    float pad;
    std::vector<eb200_bound> bounds;
};

int dtype_size(int dt) {
    switch (dt) {
        case EB200_F32: return 4;
        case EB200_BOOL: return 1;
        case EB200_I32: return 4;
        case EB200_F16: return 2;
        case EB200_BF16: return 2;
        case EB200_I64: return 8;
    }
    return 0;
}

// min / max of c + sum coef[d]*idx[d] over the box 0 <= idx[d] < shape[d]
template <class TC, class TS>
void affine_range(const TC* coef, long long c, const TS* shape, int nd, int skip,
                  long long* lo, long long* hi) {
    long long mn = c, mx = c;
    for (int d = 0; d < nd; ++d) {
        if (d == skip || shape[d] <= 0) continue;
        long long e = (long long)coef[d] * ((long long)shape[d] - 1);
        if (e < 0) mn += e; else mx += e;
    }
    *lo = mn;
    *hi = mx;
}

// Address range of a masked operand over the iterations where all of its bounds
// hold.  Bounds are affine conditions lo <= c + coef.idx < hi (what pad, slice and
// unfold produce, src/graph/shape/view.rs:980-1054,1162-1381).  Bounds with equal
// coefficient vectors form a group; when the groups touch disjoint dims and the
// operand's strides over a group's dims are a multiple alpha of its coefficients,
// the address is offset + sum alpha_g * t_g + (free dims), with t_g = coef_g.idx
// confined to an interval, so the range is exact.  Any other form is checked by
// enumeration when the iteration space is small.  Returns 1 with [*lo, *hi],
// 0 when no iteration satisfies the bounds, -1 when the form cannot be validated.
int masked_range(const eb200_operand& o, const int64_t* shape, int nd, long long total, long long* lo, long long* hi) {
    struct Group { int64_t coef[KMAX_DIMS]; long long tlo, thi; };
    std::vector<Group> groups;
    for (int b = 0; b < o.n_bounds; ++b) {
        const eb200_bound& bd = o.bounds[b];
        Group* g = nullptr;
        for (auto& q : groups) {
            bool same = true;
            for (int d = 0; d < nd; ++d) same = same && q.coef[d] == bd.coef[d];
            if (same) { g = &q; break; }
        }
        const long long tlo = bd.lo - bd.c, thi = bd.hi - 1 - bd.c;     // lo <= c + t <= hi - 1
        if (g) { g->tlo = std::max(g->tlo, tlo); g->thi = std::min(g->thi, thi); continue; }
        Group ng{};
        for (int d = 0; d < nd; ++d) ng.coef[d] = bd.coef[d];
        long long mn, mx;
        affine_range(bd.coef, 0, shape, nd, -1, &mn, &mx);
        ng.tlo = std::max(tlo, mn); ng.thi = std::min(thi, mx);
        groups.push_back(ng);
    }
    bool analytic = true;
    bool used[KMAX_DIMS] = {false};
    long long alpha[16] = {0};
    for (size_t gi = 0; gi < groups.size() && analytic; ++gi) {
        const Group& g = groups[gi];
        bool have = false;
        for (int d = 0; d < nd && analytic; ++d) {
            if (g.coef[d] == 0 || shape[d] <= 1) continue;
            if (used[d]) { analytic = false; break; }
            used[d] = true;
            if (o.strides[d] % g.coef[d] != 0) { analytic = false; break; }
            const long long a = o.strides[d] / g.coef[d];
            if (have && a != alpha[gi]) { analytic = false; break; }
            alpha[gi] = a; have = true;
        }
        if (gi >= 15) analytic = false;
    }
    if (analytic) {
        long long mn = o.offset, mx = o.offset;
        for (size_t gi = 0; gi < groups.size(); ++gi) {
            Group& g = groups[gi];
            // one active dim: t = k * idx only takes multiples of k, so round the interval inwards
            int active = -1, n_active = 0;
            for (int d = 0; d < nd; ++d) if (g.coef[d] != 0 && shape[d] > 1) { active = d; ++n_active; }
            if (n_active == 1 && g.tlo <= g.thi) {
                const long long k = g.coef[active];
                auto fdiv = [](long long a, long long b) { long long q = a / b; return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q; };
                auto cdiv = [&](long long a, long long b) { return -fdiv(-a, b); };
                long long i0 = k > 0 ? cdiv(g.tlo, k) : cdiv(g.thi, k), i1 = k > 0 ? fdiv(g.thi, k) : fdiv(g.tlo, k);
                i0 = std::max(i0, 0LL); i1 = std::min(i1, (long long)shape[active] - 1);
                if (i0 > i1) return 0;
                g.tlo = std::min(k * i0, k * i1); g.thi = std::max(k * i0, k * i1);
            }
            if (g.tlo > g.thi) return 0;
            const long long e0 = alpha[gi] * g.tlo, e1 = alpha[gi] * g.thi;
            mn += std::min(e0, e1); mx += std::max(e0, e1);
        }
        for (int d = 0; d < nd; ++d) {
            if (used[d] || shape[d] <= 1) continue;
            const long long e = (long long)o.strides[d] * (shape[d] - 1);
            if (e < 0) mn += e; else mx += e;
        }
        *lo = mn; *hi = mx;
        return 1;
    }
    if (total > (1LL << 22)) return -1;
    long long idx[KMAX_DIMS] = {0};
    bool any = false;
    long long mn = 0, mx = 0;
    for (long long e = 0; e < total; ++e) {
        bool ok = true;
        for (int b = 0; b < o.n_bounds && ok; ++b) {
            long long v = o.bounds[b].c;
            for (int d = 0; d < nd; ++d) v += o.bounds[b].coef[d] * idx[d];
            ok = v >= o.bounds[b].lo && v < o.bounds[b].hi;
        }
        if (ok) {
            long long a = o.offset;
            for (int d = 0; d < nd; ++d) a += o.strides[d] * idx[d];
            if (!any) { mn = mx = a; any = true; }
            else { mn = std::min(mn, a); mx = std::max(mx, a); }
        }
        for (int d = nd - 1; d >= 0; --d) { if (++idx[d] < shape[d]) break; idx[d] = 0; }
    }
    if (!any) return 0;
    *lo = mn; *hi = mx;
    return 1;
}

int check_program(const eb200_kernel_desc* d) {
    int depth = 0, maxdepth = 0;
    for (int i = 0; i < d->n_insns; ++i) {
        const eb200_insn& in = d->prog[i];
        int pop = 0;
        switch (in.op) {
            case EB200_OP_LOAD:
                EB_REQUIRE(in.arg >= 0 && in.arg < d->n_inputs, EB200_ERR_INVALID,
                           "map instruction %d loads input %d of %d", i, in.arg, d->n_inputs);
                pop = 0; break;
            case EB200_OP_CONST: pop = 0; break;
            case EB200_OP_ADD: case EB200_OP_MUL: case EB200_OP_MAX: case EB200_OP_LT:
            case EB200_OP_AND: case EB200_OP_REM: case EB200_OP_IDIV: pop = 2; break;
            case EB200_OP_RECIP: case EB200_OP_SQRT: case EB200_OP_LOG2: case EB200_OP_EXP2:
            case EB200_OP_SIN: case EB200_OP_FLOOR: case EB200_OP_NOT: pop = 1; break;
            case EB200_OP_CAST:
                EB_REQUIRE(dtype_size(in.arg) != 0, EB200_ERR_INVALID, "cast to unknown dtype %d", in.arg);
                pop = 1; break;
            case EB200_OP_SELECT: case EB200_OP_FMA: pop = 3; break;
            default:
                return set_error(EB200_ERR_INVALID, "unknown map opcode %d at %d", in.op, i);
        }
        EB_REQUIRE(depth >= pop, EB200_ERR_INVALID, "map program underflows its stack at %d", i);
        depth = depth - pop + 1;
        maxdepth = std::max(maxdepth, depth);
    }
    if (d->n_insns) {
        EB_REQUIRE(depth == 1, EB200_ERR_INVALID, "map program leaves %d values on the stack", depth);
        EB_REQUIRE(maxdepth <= KSTACK, EB200_ERR_UNSUPPORTED, "map program needs stack depth %d > %d", maxdepth, KSTACK);
    }
    return EB200_OK;
}

bool try_gemm(const KParams& p, Plan* plan, int mode) {
    if (p.rop != EB200_R_SUM || p.raxis < 0) return false;
    if (p.n_insns != 3) return false;
    if (p.prog[0].op != EB200_OP_LOAD || p.prog[1].op != EB200_OP_LOAD || p.prog[2].op != EB200_OP_MUL) return false;
    int ia = p.prog[0].arg, ib = p.prog[1].arg;
    if (ia == ib) return false;
    const KOperand* A = &p.in[ia];
    const KOperand* B = &p.in[ib];
    // f32 x f32 -> f32, or f16 x f16 / bf16 x bf16 -> f32 or the operands' own type (the reference's F16 MatMul node,
    // src/lowerer/lower.rs:745-1000, accumulating in f32)
    const bool half = A->dtype == EB200_F16 || A->dtype == EB200_BF16;
    if (A->dtype != B->dtype || (!half && A->dtype != EB200_F32)) return false;
    if (p.out.dtype != EB200_F32 && !(half && p.out.dtype == A->dtype)) return false;
    if (A->n_bounds || B->n_bounds) return false;
    if (A->strides[p.raxis] == 0 || B->strides[p.raxis] == 0) return false;
    int dm = -1, dn = -1, db = -1;
    for (int d = 0; d < p.ndim; ++d) {
        if (d == p.raxis) continue;
        bool a = A->strides[d] != 0, b = B->strides[d] != 0;
        if (a && !b) { if (dm >= 0) return false; dm = d; }
        else if (!a && b) { if (dn >= 0) return false; dn = d; }
        else if (a && b) { if (db >= 0) return false; db = d; }
        else return false;
    }
    if (dm < 0 || dn < 0) return false;
    GemmShape g;
    g.mode = mode == EB200_GEMM_DEFAULT ? EB200_GEMM_3XTF32 : mode;
    g.a_input = ia; g.b_input = ib;
    g.half = half ? A->dtype : 0;
    g.c_dtype = p.out.dtype;
    g.m = p.shape[dm]; g.n = p.shape[dn]; g.k = p.shape[p.raxis];
    g.batch = db >= 0 ? p.shape[db] : 1;
    g.a_sm = A->strides[dm]; g.a_sk = A->strides[p.raxis]; g.a_sb = db >= 0 ? A->strides[db] : 0; g.a_off = A->offset;
    g.b_sn = B->strides[dn]; g.b_sk = B->strides[p.raxis]; g.b_sb = db >= 0 ? B->strides[db] : 0; g.b_off = B->offset;
    g.c_sm = p.out.strides[dm]; g.c_sn = p.out.strides[dn]; g.c_sb = db >= 0 ? p.out.strides[db] : 0; g.c_off = p.out.offset;
    if (g.c_sm == 0 || g.c_sn == 0) return false;
    // Orient so that C is written along n (c_sn == 1) where possible:
    // C^T = B^T A^T swaps the roles of the operands.
    if (g.c_sn != 1 && g.c_sm == 1) {
        GemmShape t = g;
        t.a_input = g.b_input; t.b_input = g.a_input;
        t.m = g.n; t.n = g.m;
        t.a_sm = g.b_sn; t.a_sk = g.b_sk; t.a_sb = g.b_sb; t.a_off = g.b_off;
        t.b_sn = g.a_sm; t.b_sk = g.a_sk; t.b_sb = g.a_sb; t.b_off = g.a_off;
        t.c_sm = g.c_sn; t.c_sn = g.c_sm;
        g = t;
    }
    // 16-bit operands are served by the tensor-core kernel only, and only with both operands contiguous along k
    if (g.half && !gemm_tc_supported(g)) return false;
    plan->gemm = g;
    return true;
}

}  // namespace

int build_plan(const eb200_kernel_desc* d, int sm_count, Plan* plan) {
    EB_REQUIRE(d && plan, EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(d->kclass >= EB200_K_ELEMENTWISE && d->kclass <= EB200_K_MAXPOOL2D, EB200_ERR_INVALID, "unknown kernel class %d", d->kclass);
    if (d->kclass == EB200_K_CONV2D) {
        // structured descriptor: shape = {N, C, H, W, Co, KH, KW, pad}
        EB_REQUIRE(d->ndim == 8, EB200_ERR_INVALID, "conv2d descriptor wants 8 shape entries, got %d", d->ndim);
        EB_REQUIRE(d->n_inputs == 2 || d->n_inputs == 3, EB200_ERR_INVALID, "conv2d takes x, w and optionally bias");
        Plan& pl = *plan;
        pl = Plan();
        memset(&pl.p, 0, sizeof(pl.p));
        ConvShape& c = pl.conv;
        for (int i = 0; i < 8; ++i) EB_REQUIRE(d->shape[i] >= 0 && d->shape[i] < (1LL << 31), EB200_ERR_INVALID, "conv2d shape[%d] out of range", i);
        c.N = (int)d->shape[0]; c.C = (int)d->shape[1]; c.H = (int)d->shape[2]; c.W = (int)d->shape[3];
        c.Co = (int)d->shape[4]; c.KH = (int)d->shape[5]; c.KW = (int)d->shape[6]; c.pad = (int)d->shape[7];
        c.relu = (d->flags & 64) ? 1 : 0;
        c.flip = (d->flags & 128) ? 1 : 0;
        c.wgrad = (d->flags & 256) ? 1 : 0;
        c.nchw = (d->flags & 512) ? 1 : 0;
        c.g_nchw = (d->flags & 1024) ? 1 : 0;
        c.has_bias = !c.wgrad && d->n_inputs == 3;
        c.mode = d->gemm_mode == EB200_GEMM_TF32 ? EB200_GEMM_TF32 : EB200_GEMM_3XTF32;
        EB_REQUIRE(conv2d_supported(c), EB200_ERR_UNSUPPORTED, "conv2d shape is not served by the implicit-GEMM kernel (C*KH*KW <= 2048 unless C % 32 == 0, stride 1)");
        const long long Ho = c.H + 2 * c.pad - c.KH + 1, Wo = c.W + 2 * c.pad - c.KW + 1;
        const long long M = (long long)c.N * Ho * Wo, K = (long long)c.C * c.KH * c.KW;
        for (int i = 0; i <= d->n_inputs; ++i) {
            const eb200_operand& o = i < d->n_inputs ? d->inputs[i] : d->output;
            EB_REQUIRE(o.dtype == EB200_F32 && o.n_bounds == 0 && o.offset >= 0, EB200_ERR_UNSUPPORTED, "conv2d operands are plain contiguous f32 buffers");
        }
        EB_REQUIRE(d->inputs[0].numel - d->inputs[0].offset >= (long long)c.N * c.C * c.H * c.W, EB200_ERR_BOUNDS, "conv2d input buffer too small");
        // tiny reductions stream through FFMA code instead (flag 2048 keeps the tensor-core form)
        c.direct = !(d->flags & 2048) && conv2d_direct_supported(c);
        if (c.wgrad) {
            // inputs x and the output gradient [M, Co]; output dW [Co, C, KH, KW]
            EB_REQUIRE(d->n_inputs == 2 && !c.flip && !c.relu, EB200_ERR_INVALID, "conv2d weight gradient takes x and the output gradient");
            EB_REQUIRE(c.direct || !c.g_nchw, EB200_ERR_UNSUPPORTED, "the tensor-core weight gradient reads the output gradient as [N*Ho*Wo, Co] rows");
            EB_REQUIRE(c.direct || conv2d_wgrad_supported(c), EB200_ERR_UNSUPPORTED, "conv2d weight gradient: image planes must fit shared memory, Co % 4 == 0, Co <= 128");
            EB_REQUIRE(d->inputs[1].numel - d->inputs[1].offset >= M * c.Co, EB200_ERR_BOUNDS, "conv2d output-gradient buffer too small");
            EB_REQUIRE(d->output.numel - d->output.offset >= c.Co * K, EB200_ERR_BOUNDS, "conv2d weight-gradient buffer too small");
        } else {
            EB_REQUIRE(d->inputs[1].numel - d->inputs[1].offset >= (long long)c.Co * K, EB200_ERR_BOUNDS, "conv2d weight buffer too small");
            EB_REQUIRE(!c.has_bias || d->inputs[2].numel - d->inputs[2].offset >= c.Co, EB200_ERR_BOUNDS, "conv2d bias buffer too small");
            EB_REQUIRE(d->output.numel - d->output.offset >= M * c.Co, EB200_ERR_BOUNDS, "conv2d output buffer too small");
        }
        for (int i = 0; i < d->n_inputs; ++i) pl.p.in[i].offset = d->inputs[i].offset;
        pl.p.out.offset = d->output.offset;
        pl.impl = c.direct ? (c.wgrad ? IMPL_CONV2D_DIRECT_WGRAD : IMPL_CONV2D_DIRECT) : (c.wgrad ? IMPL_CONV2D_WGRAD : IMPL_CONV2D);
        pl.n_inputs = d->n_inputs;
        pl.p.n_in = d->n_inputs;
        for (int i = 0; i < d->n_inputs; ++i) { pl.in_dtype[i] = EB200_F32; pl.in_numel[i] = d->inputs[i].numel; pl.perm[i] = i; }
        for (int j = 0; j < KMAX_CONSTS; ++j) pl.dyn_input[j] = -1;
        pl.out_dtype = EB200_F32;
        pl.out_numel = d->output.numel;
        if (c.direct) pl.scratch_bytes = c.wgrad ? conv2d_direct_wgrad_scratch_floats(c, sm_count) * 4 : 0;
        else pl.scratch_bytes = (c.wgrad ? conv2d_wgrad_scratch_floats(c, sm_count) : conv2d_scratch_floats(c)) * 4;
        pl.launches = c.direct && !c.wgrad ? 1 : 2;
        pl.algo_flops = 2 * M * c.Co * K;
        pl.algo_bytes = 4 * ((long long)c.N * c.C * c.H * c.W + (long long)c.Co * K + M * c.Co + (c.has_bias ? c.Co : 0));
        if (c.direct) snprintf(pl.name, sizeof(pl.name), "conv2d_direct_f32%s", c.wgrad ? "_wgrad" : (c.flip ? "_dgrad" : ""));
        else snprintf(pl.name, sizeof(pl.name), "conv2d_igemm_%s%s", c.mode == EB200_GEMM_TF32 ? "tf32" : "3xtf32", c.wgrad ? "_wgrad" : (c.flip ? "_dgrad" : ""));
        return EB200_OK;
    }
    if (d->kclass == EB200_K_MAXPOOL2D) {
        // structured descriptor: shape = {P, H, W, k}; forward x -> y, gradient (g, x, y) -> gx
        const bool grad = (d->flags & 128) != 0;
        EB_REQUIRE(d->ndim == 4 && d->n_inputs == (grad ? 3 : 1), EB200_ERR_INVALID,
                   "max_pool2d takes shape {P, H, W, k} and %d input(s)", grad ? 3 : 1);
        const long long P = d->shape[0], H = d->shape[1], W = d->shape[2], K = d->shape[3];
        EB_REQUIRE(P >= 1 && K >= 1 && K <= 4 && H >= K && W >= K && H < 65536 && W < 65536 && P * H * W < (1LL << 40) &&
                   P * ((H + K - 1) / K) * ((W + K - 1) / K) < (1LL << 31), EB200_ERR_UNSUPPORTED,
                   "max_pool2d over [%lld, %lld, %lld] with window %lld", P, H, W, K);
        const long long full = P * H * W, pooled = P * (H / K) * (W / K);
        Plan& pl = *plan;
        pl = Plan();
        memset(&pl.p, 0, sizeof(pl.p));
        for (int i = 0; i <= d->n_inputs; ++i) {
            const eb200_operand& o = i < d->n_inputs ? d->inputs[i] : d->output;
            EB_REQUIRE(o.dtype == EB200_F32 && o.n_bounds == 0 && o.offset >= 0, EB200_ERR_UNSUPPORTED, "max_pool2d operands are plain contiguous f32 buffers");
            const bool is_full = grad ? (i == 1 || i == d->n_inputs) : (i == 0);
            EB_REQUIRE(o.numel - o.offset >= (is_full ? full : pooled), EB200_ERR_BOUNDS, "max_pool2d operand %d too small", i);
            (i < d->n_inputs ? pl.p.in[i] : pl.p.out).offset = o.offset;
        }
        pl.p.shape[0] = P; pl.p.shape[1] = H; pl.p.shape[2] = W; pl.p.ndim = 3; pl.p.total = full; pl.p.n_in = d->n_inputs;
        pl.impl = IMPL_MAXPOOL;
        pl.pool[0] = P; pl.pool[1] = H; pl.pool[2] = W; pl.pool[3] = K;
        pl.pool_flags = ((d->flags & 64) ? 1 : 0) | (grad ? 2 : 0);
        pl.n_inputs = d->n_inputs;
        for (int i = 0; i < d->n_inputs; ++i) { pl.in_dtype[i] = EB200_F32; pl.in_numel[i] = d->inputs[i].numel; pl.perm[i] = i; }
        for (int j = 0; j < KMAX_CONSTS; ++j) pl.dyn_input[j] = -1;
        pl.out_dtype = EB200_F32;
        pl.out_numel = d->output.numel;
        pl.launches = 1;
        // forward: the covered part of x once, y once; gradient: g, y, the covered part of x in, gx out
        const long long covered = P * (H / K) * K * (W / K) * K;
        pl.algo_bytes = 4 * (grad ? 2 * pooled + covered + full : covered + pooled);
        snprintf(pl.name, sizeof(pl.name), "maxpool2d_k%lld%s%s", K, (d->flags & 64) ? "_relu" : "", grad ? "_grad" : "");
        return EB200_OK;
    }
    if (d->kclass == EB200_K_SOFTMAX_XENT) {
        // structured descriptor: shape = {N, C}; logits and one-hot targets in, [64 + N*C] out
        EB_REQUIRE(d->ndim == 2 && d->n_inputs == 2, EB200_ERR_INVALID, "softmax cross-entropy takes shape {N, C} and two inputs");
        const long long N = d->shape[0], Cn = d->shape[1];
        EB_REQUIRE(N >= 1 && Cn >= 1 && N < (1LL << 31) && Cn <= 65536, EB200_ERR_UNSUPPORTED, "softmax cross-entropy over [%lld, %lld]", N, Cn);
        Plan& pl = *plan;
        pl = Plan();
        memset(&pl.p, 0, sizeof(pl.p));
        for (int i = 0; i <= 2; ++i) {
            const eb200_operand& o = i < 2 ? d->inputs[i] : d->output;
            EB_REQUIRE(o.dtype == EB200_F32 && o.n_bounds == 0 && o.offset >= 0, EB200_ERR_UNSUPPORTED, "softmax cross-entropy operands are plain contiguous f32 buffers");
            EB_REQUIRE(o.numel - o.offset >= N * Cn + (i == 2 ? 64 : 0), EB200_ERR_BOUNDS, "softmax cross-entropy operand %d too small", i);
            (i < 2 ? pl.p.in[i] : pl.p.out).offset = o.offset;
        }
        pl.p.shape[0] = N; pl.p.shape[1] = Cn; pl.p.ndim = 2; pl.p.total = N * Cn; pl.p.n_in = 2;
        pl.impl = IMPL_SOFTMAX_XENT;
        pl.n_inputs = 2;
        for (int i = 0; i < 2; ++i) { pl.in_dtype[i] = EB200_F32; pl.in_numel[i] = d->inputs[i].numel; pl.perm[i] = i; }
        for (int j = 0; j < KMAX_CONSTS; ++j) pl.dyn_input[j] = -1;
        pl.out_dtype = EB200_F32;
        pl.out_numel = d->output.numel;
        pl.scalar = d->scalar;
        pl.scratch_bytes = 4096;          // per-CTA loss partials and the ticket word
        pl.scratch_zero = true;
        pl.algo_bytes = 4 * (3 * N * Cn + 1);
        snprintf(pl.name, sizeof(pl.name), "softmax_xent_fwd_bwd");
        return EB200_OK;
    }
    EB_REQUIRE(d->ndim >= 0 && d->ndim <= EB200_MAX_DIMS, EB200_ERR_INVALID, "rank %d out of range", d->ndim);
    EB_REQUIRE(d->n_inputs >= 1 && d->n_inputs <= EB200_MAX_INPUTS, EB200_ERR_INVALID, "%d inputs out of range", d->n_inputs);
    EB_REQUIRE(d->n_insns >= 0 && d->n_insns <= EB200_MAX_INSNS, EB200_ERR_INVALID, "%d map instructions out of range", d->n_insns);
    for (int i = 0; i < d->ndim; ++i)
        EB_REQUIRE(d->shape[i] >= 0 && d->shape[i] < (1LL << 40), EB200_ERR_INVALID, "shape[%d] = %lld out of range", i, (long long)d->shape[i]);
    for (int i = 0; i <= d->n_inputs; ++i) {
        const eb200_operand& o = i < d->n_inputs ? d->inputs[i] : d->output;
        EB_REQUIRE(dtype_size(o.dtype) != 0, EB200_ERR_INVALID, "operand %d has unknown dtype %d", i, o.dtype);
        EB_REQUIRE(o.n_bounds >= 0 && o.n_bounds <= EB200_MAX_BOUNDS, EB200_ERR_INVALID, "operand %d has %d bounds", i, o.n_bounds);
        EB_REQUIRE(o.numel >= 0, EB200_ERR_INVALID, "operand %d has negative numel", i);
        EB_REQUIRE(o.dtype != EB200_I64, EB200_ERR_UNSUPPORTED, "i64 tensors are not served by any kernel class yet");
    }
    EB_REQUIRE(d->output.n_bounds == 0, EB200_ERR_INVALID, "the store operand cannot carry bounds");
    int st = check_program(d);
    if (st) return st;

    const bool is_reduce = d->kclass == EB200_K_REDUCE;
    const bool is_scan = d->kclass == EB200_K_SCAN;
    if (is_reduce || is_scan) {
        EB_REQUIRE(d->reduce_op >= EB200_R_SUM && d->reduce_op <= EB200_R_PROD, EB200_ERR_INVALID, "reduce op %d", d->reduce_op);
        EB_REQUIRE(d->reduce_axis >= 0 && d->reduce_axis < d->ndim, EB200_ERR_INVALID, "reduce axis %d of rank %d", d->reduce_axis, d->ndim);
    } else {
        EB_REQUIRE(d->reduce_op == EB200_R_NONE, EB200_ERR_INVALID, "reduce op on a non-reduce kernel");
    }
    if (d->n_insns == 0)
        EB_REQUIRE(d->kclass != EB200_K_ELEMENTWISE || d->n_inputs == 1, EB200_ERR_INVALID, "empty map needs exactly one input");

    // ---- address range validation: never let a kernel index outside a buffer
    long long total = 1;
    for (int i = 0; i < d->ndim; ++i) total *= d->shape[i];
    if (total > 0) {
        for (int i = 0; i <= d->n_inputs; ++i) {
            const eb200_operand& o = i < d->n_inputs ? d->inputs[i] : d->output;
            long long lo, hi;
            if (o.n_bounds) {
                // a masked load is only dereferenced where every bound holds: validate
                // the addresses of exactly those iterations
                int r = masked_range(o, d->shape, d->ndim, total, &lo, &hi);
                if (r == 0) continue;   // the bounds never hold together: nothing is loaded
                EB_REQUIRE(r > 0, EB200_ERR_BOUNDS,
                           "input %d: bound conditions of this form cannot be validated against the buffer size", i);
            } else {
                int skip = (i == d->n_inputs && is_reduce) ? d->reduce_axis : -1;
                affine_range(o.strides, o.offset, d->shape, d->ndim, skip, &lo, &hi);
            }
            EB_REQUIRE(lo >= 0 && hi < o.numel, EB200_ERR_BOUNDS,
                       "%s %d addresses elements [%lld, %lld] of a buffer of %lld",
                       i < d->n_inputs ? "input" : "output", i < d->n_inputs ? i : 0, lo, hi, (long long)o.numel);
        }
    }

    // ---- normalise: drop extent-1 dims and provably true bounds, collapse
    int keep[KMAX_DIMS], nk = 0, raxis = -1;
    for (int i = 0; i < d->ndim; ++i) {
        bool is_r = (is_reduce || is_scan) && i == d->reduce_axis;
        if (d->shape[i] != 1 || is_r) {
            if (is_r) raxis = nk;
            keep[nk++] = i;
        }
    }
    std::vector<Op> ops(d->n_inputs + 1);
    long long shape[KMAX_DIMS];
    for (int j = 0; j < nk; ++j) shape[j] = d->shape[keep[j]];
    for (int i = 0; i <= d->n_inputs; ++i) {
        const eb200_operand& o = i < d->n_inputs ? d->inputs[i] : d->output;
        Op& q = ops[i];
        q.dtype = o.dtype; q.offset = o.offset; q.numel = o.numel; q.pad = o.pad_value;
        for (int j = 0; j < nk; ++j) q.strides[j] = o.strides[keep[j]];
        if (i == d->n_inputs && raxis >= 0 && is_reduce) q.strides[raxis] = 0;
        for (int b = 0; b < o.n_bounds; ++b) {
            eb200_bound nb{};
            for (int j = 0; j < nk; ++j) nb.coef[j] = o.bounds[b].coef[keep[j]];
            nb.c = o.bounds[b].c; nb.lo = o.bounds[b].lo; nb.hi = o.bounds[b].hi;
            long long lo, hi;
            affine_range(nb.coef, nb.c, shape, nk, -1, &lo, &hi);
            if (lo >= nb.lo && hi < nb.hi) continue;  // always true
            q.bounds.push_back(nb);
        }
    }
    if (nk == 0) {  // a single element: keep one extent-1 dim so kernels always have a rank
        nk = 1;
        shape[0] = 1;
        for (auto& q : ops) {
            q.strides[0] = 0;
            for (auto& b : q.bounds) b.coef[0] = 0;
        }
    }
    // collapse dim j (outer) into j+1 (inner) when every operand walks them as one
    for (int j = nk - 2; j >= 0; --j) {
        if (j == raxis || j + 1 == raxis) continue;
        bool ok = true;
        for (auto& q : ops) {
            if (q.strides[j] != q.strides[j + 1] * shape[j + 1]) { ok = false; break; }
            for (auto& b : q.bounds)
                if (b.coef[j] != b.coef[j + 1] * shape[j + 1]) { ok = false; break; }
            if (!ok) break;
        }
        if (!ok) continue;
        // the merged dim keeps the inner strides and takes the product extent;
        // it lands at position j once dim j is removed
        shape[j + 1] *= shape[j];
        for (int t = j; t < nk - 1; ++t) shape[t] = shape[t + 1];
        for (auto& q : ops) {
            for (int t = j; t < nk - 1; ++t) q.strides[t] = q.strides[t + 1];
            for (auto& b : q.bounds)
                for (int t = j; t < nk - 1; ++t) b.coef[t] = b.coef[t + 1];
        }
        if (raxis > j) --raxis;
        --nk;
    }

    // a scan walks the axis and every dim after it as ONE sequence
    // (src/lowerer/loop_gen.rs:237-327): fold that tail into the axis where all
    // operands walk it contiguously
    while (is_scan && raxis >= 0 && raxis + 1 < nk) {
        const int j = raxis;
        bool ok = true;
        for (auto& q : ops) {
            if (q.strides[j] != q.strides[j + 1] * shape[j + 1]) { ok = false; break; }
            for (auto& b : q.bounds)
                if (b.coef[j] != b.coef[j + 1] * shape[j + 1]) { ok = false; break; }
            if (!ok) break;
        }
        if (!ok) break;
        shape[j + 1] *= shape[j];
        for (int t = j; t < nk - 1; ++t) shape[t] = shape[t + 1];
        for (auto& q : ops) {
            for (int t = j; t < nk - 1; ++t) q.strides[t] = q.strides[t + 1];
            for (auto& b : q.bounds)
                for (int t = j; t < nk - 1; ++t) b.coef[t] = b.coef[t + 1];
        }
        --nk;
    }

    Plan& pl = *plan;
    pl = Plan();
    KParams& p = pl.p;
    memset(&p, 0, sizeof(p));
    p.ndim = nk;
    p.n_in = d->n_inputs;
    p.total = total;
    for (int j = 0; j < KMAX_DIMS; ++j) p.shape[j] = j < nk ? shape[j] : 1;     // dims past the rank: extent 1 (strides stay 0)
    // magic numbers for exact n / shape[j], n < 2^31: M = ceil(2^(31+l) / s) < 2^32 with l = ceil(log2 s)
    for (int j = 0; j < KMAX_DIMS; ++j) {
        const unsigned long long sj = j < nk && shape[j] >= 1 && shape[j] < (1LL << 31) ? (unsigned long long)shape[j] : 1ULL;
        int l = 0;
        while ((1ULL << l) < sj) ++l;
        p.dmul[j] = (unsigned)((((1ULL << (31 + l)) + sj - 1) / sj));
        p.dshr[j] = (unsigned)(31 + l);
    }
    p.raxis = raxis;
    p.rop = d->reduce_op;
    p.rlen = raxis >= 0 ? shape[raxis] : 1;
    p.kept = raxis >= 0 ? (p.rlen ? total / p.rlen : 0) : total;
    if (raxis >= 0 && p.rlen == 0) {
        long long k = 1;
        for (int j = 0; j < nk; ++j) if (j != raxis) k *= shape[j];
        p.kept = k;
    }
    if (is_scan) {
        // rows = the dims before the axis; a row = the axis and everything after it
        p.rlen = 1; p.kept = 1;
        for (int j = 0; j < nk; ++j) (j < raxis ? p.kept : p.rlen) *= shape[j];
    }
    p.splits = 1;
    p.chunk = p.rlen;
    p.tuning = d->flags;
    int nb_total = 0;
    for (int i = 0; i <= d->n_inputs; ++i) {
        KOperand& ko = i < d->n_inputs ? p.in[i] : p.out;
        const Op& q = ops[i];
        ko.ptr = nullptr; ko.offset = q.offset; ko.dtype = q.dtype; ko.pad = q.pad;
        for (int j = 0; j < nk; ++j) ko.strides[j] = q.strides[j];
        ko.bound_begin = nb_total; ko.n_bounds = (int)q.bounds.size();
        EB_REQUIRE(nb_total + ko.n_bounds <= KMAX_BOUNDS, EB200_ERR_UNSUPPORTED, "more than %d live bound conditions in one kernel", KMAX_BOUNDS);
        for (auto& b : q.bounds) {
            KBound& kb = p.bounds[nb_total++];
            for (int j = 0; j < nk; ++j) kb.coef[j] = b.coef[j];
            kb.c = b.c; kb.lo = b.lo; kb.hi = b.hi;
        }
    }
    if (d->n_insns == 0) {
        p.n_insns = 1;
        p.prog[0].op = EB200_OP_LOAD; p.prog[0].arg = 0; p.prog[0].imm = 0.f;
    } else {
        p.n_insns = d->n_insns;
        for (int i = 0; i < d->n_insns; ++i) {
            p.prog[i].op = (short)d->prog[i].op; p.prog[i].arg = (short)d->prog[i].arg; p.prog[i].imm = d->prog[i].imm;
        }
    }
    pl.n_inputs = d->n_inputs;
    for (int i = 0; i < d->n_inputs; ++i) { pl.in_dtype[i] = d->inputs[i].dtype; pl.in_numel[i] = d->inputs[i].numel; }
    pl.out_dtype = d->output.dtype;
    pl.out_numel = d->output.numel;
    pl.scalar = d->scalar;
    for (int i = 0; i < 7; ++i) pl.hyper[i] = d->hyper[i];

    // ---- algorithmic traffic: every operand element that is addressed, once
    {
        int64_t bytes = 0;
        for (int i = 0; i <= d->n_inputs; ++i) {
            const KOperand& ko = i < d->n_inputs ? p.in[i] : p.out;
            int64_t n = 1;
            for (int j = 0; j < nk; ++j) if (ko.strides[j] != 0) n *= shape[j];
            if (i == d->n_inputs && raxis < 0 && d->kclass != EB200_K_SCATTER) n = total;
            if (d->kclass == EB200_K_SCATTER && i == d->n_inputs) n = d->output.numel;
            if (total == 0) n = 0;
            bytes += n * dtype_size(ko.dtype);
        }
        pl.algo_bytes = bytes;
    }

    // ---- 128-bit legality along the innermost collapsed dim
    // (`half_ok`: the elementwise kernel also moves f16 / bf16 operands four at a time, with 64-bit accesses)
    auto vec_ok = [&](const KOperand& ko, int inner, bool is_store, bool half_ok = false) -> bool {
        const bool dt_ok = ko.dtype == EB200_F32 || (half_ok && (ko.dtype == EB200_F16 || ko.dtype == EB200_BF16));
        if (!dt_ok || ko.n_bounds) return false;
        long long s = ko.strides[inner];
        if (s == 0) return !is_store;
        if (s != 1) return false;
        if (ko.offset % 4) return false;
        for (int j = 0; j < nk; ++j) if (j != inner && ko.strides[j] % 4) return false;
        return true;
    };

    // ---- one-element f32 operands become launch-time constants (read once per
    //      thread instead of once per element); the remaining operands are
    //      renumbered by first use in the map, so equal expressions meet the
    //      same compiled functor whatever order their inputs were declared in
    for (int j = 0; j < KMAX_CONSTS; ++j) pl.dyn_input[j] = -1;
    for (int i = 0; i < KMAX_IN; ++i) pl.perm[i] = i;
    if (d->kclass == EB200_K_ELEMENTWISE || d->kclass == EB200_K_REDUCE || d->kclass == EB200_K_SCAN) {
        KOperand old_in[KMAX_IN];
        for (int i = 0; i < KMAX_IN; ++i) old_in[i] = p.in[i];
        // (1) expression tree from the postfix program; one-element loads marked constant
        struct Node { short op, arg; float imm; int kid[3]; int nk; int dyn; };
        std::vector<Node> nodes;
        std::vector<int> stack;
        for (int pc = 0; pc < p.n_insns; ++pc) {
            const KInsn& ins = p.prog[pc];
            Node nd{ins.op, ins.arg, ins.imm, {-1, -1, -1}, 0, -1};
            int pop = 0;
            switch (ins.op) {
                case EB200_OP_LOAD: {
                    const KOperand& ko = old_in[ins.arg];
                    bool one = ko.dtype == EB200_F32 && ko.n_bounds == 0;
                    for (int j = 0; j < nk && one; ++j) one = ko.strides[j] == 0;
                    if (one) { nd.op = EB200_OP_CONST; nd.dyn = ins.arg; }
                    break;
                }
                case EB200_OP_CONST: break;
                case EB200_OP_SELECT: case EB200_OP_FMA: pop = 3; break;
                case EB200_OP_RECIP: case EB200_OP_SQRT: case EB200_OP_LOG2: case EB200_OP_EXP2:
                case EB200_OP_SIN: case EB200_OP_FLOOR: case EB200_OP_NOT: case EB200_OP_CAST: pop = 1; break;
                default: pop = 2; break;
            }
            nd.nk = pop;
            for (int c = pop - 1; c >= 0; --c) { nd.kid[c] = stack.back(); stack.pop_back(); }
            // (2) commutative ops: constant operand last
            if (pop == 2 && (nd.op == EB200_OP_ADD || nd.op == EB200_OP_MUL || nd.op == EB200_OP_MAX) &&
                nodes[nd.kid[0]].op == EB200_OP_CONST && nodes[nd.kid[1]].op != EB200_OP_CONST)
                std::swap(nd.kid[0], nd.kid[1]);
            nodes.push_back(nd);
            stack.push_back((int)nodes.size() - 1);
        }
        // (3) re-emit: inputs renumbered by first use, constants given slots in order
        int canon[KMAX_IN];
        for (int i = 0; i < KMAX_IN; ++i) canon[i] = -1;
        int n_kin = 0, nc = 0, n_out = 0;
        bool too_many = false;
        std::vector<int> order;   // iterative post-order
        {
            std::vector<std::pair<int, int>> st;
            st.push_back({stack.back(), 0});
            while (!st.empty()) {
                auto& top = st.back();
                const Node& nd = nodes[top.first];
                if (top.second < nd.nk) { int k = nd.kid[top.second++]; st.push_back({k, 0}); }
                else { order.push_back(top.first); st.pop_back(); }
            }
        }
        for (int id : order) {
            const Node& nd = nodes[id];
            KInsn ins{nd.op, nd.arg, nd.imm};
            if (nd.op == EB200_OP_LOAD) {
                const int i = nd.arg;
                if (canon[i] < 0) { canon[i] = n_kin; pl.perm[n_kin] = i; p.in[n_kin] = old_in[i]; ++n_kin; }
                ins.arg = (short)canon[i];
            } else if (nd.op == EB200_OP_CONST) {
                // equal constants share a slot (the same literal bits, or the same element of the same
                // tensor), so repeated subexpressions -- tanh's exp inside its gradient, say -- are
                // textually identical in the compiled functor and evaluated once
                int slot = -1;
                for (int j = 0; j < nc && slot < 0; ++j) {
                    if (nd.dyn >= 0) { if (pl.dyn_input[j] == nd.dyn && pl.dyn_offset[j] == old_in[nd.dyn].offset) slot = j; }
                    else if (pl.dyn_input[j] < 0 && memcmp(&p.consts[j], &nd.imm, sizeof(float)) == 0) slot = j;
                }
                if (slot < 0) {
                    if (nc >= KMAX_CONSTS) { too_many = true; break; }
                    slot = nc++;
                    if (nd.dyn >= 0) { pl.dyn_input[slot] = nd.dyn; pl.dyn_offset[slot] = old_in[nd.dyn].offset; p.consts[slot] = 0.0f; }
                    else p.consts[slot] = nd.imm;
                }
                ins.arg = (short)slot;
                if (nd.dyn >= 0) ins.imm = 0.0f;
            }
            p.prog[n_out++] = ins;
        }
        EB_REQUIRE(!too_many, EB200_ERR_UNSUPPORTED, "map uses more than %d constants", KMAX_CONSTS);
        p.n_insns = n_out;
        p.n_in = n_kin;
        p.n_consts = nc;
    }

    // ---- classify
    const bool identity = p.n_insns == 1 && p.prog[0].op == EB200_OP_LOAD && p.n_in == 1;
    switch (d->kclass) {
        case EB200_K_SGD: {
            EB_REQUIRE(d->n_inputs == 2 && nk <= 1, EB200_ERR_UNSUPPORTED, "sgd kernel wants two flat f32 inputs");
            for (int i = 0; i < 2; ++i)
                EB_REQUIRE(p.in[i].dtype == EB200_F32 && (total <= 1 || p.in[i].strides[0] == 1), EB200_ERR_UNSUPPORTED, "sgd operands must be flat f32");
            EB_REQUIRE(p.out.dtype == EB200_F32 && (total <= 1 || p.out.strides[0] == 1), EB200_ERR_UNSUPPORTED, "sgd output must be flat f32");
            pl.impl = IMPL_SGD;
            snprintf(pl.name, sizeof(pl.name), "sgd_update");
            break;
        }
        case EB200_K_SGD_MOMENTUM:
        case EB200_K_ADAM: {
            const bool adam = d->kclass == EB200_K_ADAM;
            const int nf = adam ? 4 : 3;     // flat f32 inputs: p, g, (m,) v
            EB_REQUIRE(d->n_inputs == (adam ? 5 : 3) && nk <= 1, EB200_ERR_UNSUPPORTED,
                       adam ? "adam wants p, g, m, v and the step counter" : "sgd with momentum wants p, g and v");
            for (int i = 0; i < nf; ++i)
                EB_REQUIRE(p.in[i].dtype == EB200_F32 && (total <= 1 || p.in[i].strides[0] == 1), EB200_ERR_UNSUPPORTED, "optimizer operands must be flat f32");
            EB_REQUIRE(p.out.dtype == EB200_F32 && (total <= 1 || p.out.strides[0] == 1), EB200_ERR_UNSUPPORTED, "optimizer output must be flat f32");
            if (adam) {
                EB_REQUIRE(p.in[4].dtype == EB200_I32 && p.in[4].strides[0] == 0, EB200_ERR_UNSUPPORTED, "adam's step counter is one I32 element");
                pl.impl = IMPL_ADAM;
                pl.scratch_bytes = 256;      // the ticket word that picks the last CTA
                pl.scratch_zero = true;
                pl.algo_bytes = 28 * total;
                snprintf(pl.name, sizeof(pl.name), "adam_update");
            } else {
                pl.impl = IMPL_SGD_MOMENTUM;
                pl.algo_bytes = 20 * total;
                snprintf(pl.name, sizeof(pl.name), "sgd_momentum_update");
            }
            break;
        }
        case EB200_K_SCAN: {
            EB_REQUIRE(p.out.dtype == EB200_F32, EB200_ERR_UNSUPPORTED, "scan writes f32");
            pl.impl = IMPL_SCAN;
            const bool tail_flat = raxis == nk - 1;
            bool v = tail_flat && p.rlen % 4 == 0 && p.rlen >= 4 && vec_ok(p.out, raxis, true);
            for (int i = 0; v && i < p.n_in; ++i) v = vec_ok(p.in[i], raxis, false);
            p.vec = v ? 4 : 1;
            pl.scratch_bytes = scan_scratch_floats(p, sm_count) * 4;
            pl.launches = pl.scratch_bytes ? 2 : 1;
            if (pl.scratch_bytes) pl.algo_bytes += (pl.algo_bytes - 4 * total > 0 ? pl.algo_bytes - 4 * total : 0);   // the two-pass form reads its inputs twice
            snprintf(pl.name, sizeof(pl.name), "scan_%s_v%d", pl.scratch_bytes ? "tiles" : (p.rlen <= 1024 ? "warp_rows" : "cta_rows"), p.vec);
            break;
        }
        case EB200_K_SCATTER: {
            EB_REQUIRE(d->n_inputs == 1 && identity, EB200_ERR_UNSUPPORTED, "scatter takes one input and no map");
            EB_REQUIRE(p.in[0].dtype == EB200_F32 && p.out.dtype == EB200_F32, EB200_ERR_UNSUPPORTED, "scatter-add is f32 only");
            pl.impl = IMPL_SCATTER;
            pl.launches = 2;
            snprintf(pl.name, sizeof(pl.name), "scatter_add");
            // A fold -- the scatter-add unfold's gradient lowers to (src/grad/rules.rs:40-53): iteration dims
            // (..., Ho, Wo, KH, KW), the output addressed as h = ho*sh + kh*dh, w = wo*sw + kw*dw inside dense planes --
            // can be turned around: every output element sums the few windows that cover it.  No atomics, and the
            // terms are added in the order the reference's sequential loop adds them.
            if (nk >= 4 && !p.in[0].n_bounds && total < (1LL << 31)) {
                const long long a = p.out.strides[nk - 4], b = p.out.strides[nk - 3], c = p.out.strides[nk - 2], e = p.out.strides[nk - 1];
                const long long Ho = shape[nk - 4], Wo = shape[nk - 3], KH = shape[nk - 2], KW = shape[nk - 1];
                bool ok = a > 0 && b > 0 && c > 0 && e > 0 && KH <= 16 && KW <= 16;
                // (windows that do not overlap -- a pooling gradient, window = stride -- put at most one term into every
                // element: they stay on the scatter kernel, which reads its input in order, with plain stores instead
                // of atomics; as a gather they measured 304 / 903 us against 251 / 788 us for the atomic scatter.
                // Overlapping 3x3 windows: 1 328 us with atomics, 534 us as a gather.)
                const bool overlap = c * (KH - 1) >= a || e * (KW - 1) >= b;
                long long pitch = 0, sh = 0, dh = 0, wout = 0, hout = 0;
                if (ok) {
                    long long x = a, y = c;
                    while (y) { const long long t = x % y; x = y; y = t; }
                    pitch = x;                                   // gcd(a, c): the row pitch of the output planes
                    sh = a / pitch; dh = c / pitch;
                    wout = b * (Wo - 1) + e * (KW - 1) + 1;
                    hout = sh * (Ho - 1) + dh * (KH - 1) + 1;
                    ok = wout <= pitch && hout < (1LL << 30) && wout < (1LL << 30) && b < (1LL << 20) && e < (1LL << 20) &&
                         sh < (1LL << 20) && dh < (1LL << 20);
                }
                // the dims in front of the windows address disjoint planes
                if (ok) {
                    int order[KMAX_DIMS], m = 0;
                    for (int j = 0; j < nk - 4; ++j) if (shape[j] > 1) order[m++] = j;
                    std::sort(order, order + m, [&](int u, int v) { return p.out.strides[u] < p.out.strides[v]; });
                    long long span = hout * pitch;
                    for (int j = 0; j < m && ok; ++j) {
                        ok = p.out.strides[order[j]] >= span;
                        span = p.out.strides[order[j]] * shape[order[j]];
                    }
                    long long outer = 1;
                    for (int j = 0; j < nk - 4; ++j) outer *= shape[j];
                    ok = ok && outer * hout * wout < (1LL << 31);
                }
                if (ok && !overlap) {
                    pl.scatter_plain = 1;            // every output element receives at most one term: 0 + v, no atomic needed
                } else if (ok) {
                    pl.impl = IMPL_FOLD_GATHER;
                    pl.fold_pitch = pitch;
                    pl.fold_sh = (int)sh; pl.fold_dh = (int)dh; pl.fold_sw = (int)b; pl.fold_dw = (int)e;
                    pl.fold_hout = (int)hout; pl.fold_wout = (int)wout;
                    snprintf(pl.name, sizeof(pl.name), "scatter_add_as_gather");
                }
            }
            break;
        }
        case EB200_K_COPY:
            EB_REQUIRE(d->n_inputs == 1 && identity, EB200_ERR_INVALID, "copy takes one input and no map");
            EB_REQUIRE(p.in[0].dtype == p.out.dtype, EB200_ERR_UNSUPPORTED, "copy cannot change dtype");
            /* fallthrough */
        case EB200_K_ELEMENTWISE: {
            pl.impl = IMPL_EW;
            // batched 2-D transpose: output contiguous, input unit-stride on a
            // dim that is not the innermost one
            bool tr = identity && p.in[0].dtype == p.out.dtype && !p.in[0].n_bounds && nk >= 2 &&
                      dtype_size(p.out.dtype) == 4 && p.in[0].strides[nk - 1] != 1;
            if (tr) {
                long long acc = 1;
                for (int j = nk - 1; j >= 0; --j) { if (p.out.strides[j] != acc) tr = false; acc *= shape[j]; }
            }
            int rdim = -1;
            if (tr) {
                for (int j = 0; j < nk - 1; ++j) if (p.in[0].strides[j] == 1) { rdim = j; break; }
                if (rdim < 0 || shape[rdim] < 16 || shape[nk - 1] < 16) tr = false;
            }
            if (tr) {
                pl.impl = IMPL_TRANSPOSE;
                p.raxis = rdim;  // the dim the input is contiguous along
                snprintf(pl.name, sizeof(pl.name), "transpose_copy");
            } else {
                int inner = nk - 1;
                bool v = nk >= 1 && shape[inner] % 4 == 0 && vec_ok(p.out, inner, true, true);
                for (int i = 0; v && i < p.n_in; ++i) v = vec_ok(p.in[i], inner, false, true);
                p.vec = v ? 4 : 1;
                snprintf(pl.name, sizeof(pl.name), "ew_chain_v%d", p.vec);
                if (!v && nk >= 2 && total % 4 == 0 && total >= 1024) {
                    // "groups of four": the output is a plain contiguous f32 array, so a thread can own four
                    // consecutive elements (one index decomposition, one 128-bit store) even when some
                    // operand is strided, broadcast or masked along the inner dims: those are read element
                    // by element, operands laid out like the iteration space with one 128-bit load
                    auto flat = [&](const KOperand& ko) {
                        if (ko.dtype != EB200_F32 || ko.n_bounds || ko.offset % 4) return false;
                        long long acc = 1;
                        for (int j = nk - 1; j >= 0; --j) { if (shape[j] > 1 && ko.strides[j] != acc) return false; acc *= shape[j]; }
                        return true;
                    };
                    // worth it when some operand comes in with 128-bit loads, or when the rank is high
                    int n_flat = 0;
                    for (int i = 0; i < p.n_in; ++i) n_flat += flat(p.in[i]) ? 1 : 0;
                    // (measured: rank-4 kernels with every operand strided lose ~12 % in groups of four, rank 5-6
                    // ones, whose scalar form decomposes six indices per element, gain 15 %)
                    if (flat(p.out) && (n_flat > 0 || nk >= 5)) {
                        p.vec = 2;
                        for (int i = 0; i < p.n_in; ++i) {
                            p.in[i].flat = flat(p.in[i]) ? 1 : 0;
                            // stepping to the next element in row-major order ticks some dim d and wraps the
                            // dims after it: the operand's address moves by this much
                            for (int dd = 0; dd < KMAX_DIMS; ++dd) {
                                long long dl = dd < nk ? p.in[i].strides[dd] : 0;
                                for (int e2 = dd + 1; e2 < nk; ++e2) dl -= (shape[e2] - 1) * p.in[i].strides[e2];
                                p.in[i].delta[dd] = dl;
                            }
                        }
                        snprintf(pl.name, sizeof(pl.name), "ew_chain_g4");
                    }
                }
            }
            break;
        }
        case EB200_K_REDUCE: {
            // a contraction is served as a GEMM only when some GEMM kernel's grid can hold it
            // (grid.z carries batch x splits, grid.y the column tiles of the f32 kernel);
            // anything else stays a plain reduce
            auto gemm_fits = [&](const GemmShape& g) {
                if ((d->flags & 8) == 0 && gemm_tc_supported(g) && 2 * g.batch * g.m * g.n * g.k >= (1LL << 22)) return true;
                return g.batch <= 65535 && (g.n + 63) / 64 <= 65535;
            };
            if (try_gemm(p, &pl, d->gemm_mode) && gemm_fits(pl.gemm)) {
                pl.algo_flops = 2 * pl.gemm.batch * pl.gemm.m * pl.gemm.n * pl.gemm.k;
                // tensor cores when the operand layout allows it and the problem
                // is more than a few tiles of work; f32 FFMA tiles otherwise
                const bool force_simt = (d->flags & 8) != 0;
                GemmShape& g = pl.gemm;
                const bool tc = g.half || (!force_simt && gemm_tc_supported(g) && pl.algo_flops >= (1LL << 22));
                // split-K when the output has too few tiles to fill the machine
                // (weight gradients: small M x N, K = batch)
                {
                    const long long tm = tc ? 128 : 64, tn = tc ? 128 : 64;
                    const long long tiles = ((g.m + tm - 1) / tm) * ((g.n + tn - 1) / tn) * g.batch;
                    const long long kblocks = (g.k + 31) / 32;
                    if (tiles < sm_count && kblocks >= 16 && (d->flags & 16) == 0 && !g.half) {
                        // (a handful of output tiles -- a [10, 128] weight gradient over a batch of 512 -- may cut k down to two
                        // blocks per CTA: otherwise two or four CTAs walk the whole of k one block after the other)
                        long long s = std::min<long long>((2LL * sm_count + tiles - 1) / tiles, kblocks / (tiles <= 4 && !tc ? 2 : 8));
                        s = std::min<long long>(s, 65535 / std::max<long long>(1, g.batch));
                        if (s > 1) {
                            long long per = (kblocks + s - 1) / s;
                            s = (kblocks + per - 1) / per;
                            g.splits = (int)s;
                            g.k_chunk = per * 32;
                        }
                    }
                }
                long long scratch_floats = 0;
                if (tc) {
                    pl.impl = IMPL_GEMM_TC;
                    const bool three = g.mode == EB200_GEMM_3XTF32 && !g.half;
                    g.convert = gemm_tc_convert(g, d->flags);
                    if (three && g.convert != 3) {
                        // hi / lo copies of every operand that is not split inside the kernel, one pre-pass each
                        long long a_span, b_span;
                        gemm_tc_scratch(g, &a_span, &b_span);
                        if (!(g.convert & 1)) { scratch_floats += 2 * a_span; pl.launches += 1; }
                        if (!(g.convert & 2)) { scratch_floats += 2 * b_span; pl.launches += 1; }
                    }
                    // name: arithmetic mode, then which dim of A and of B is contiguous (k, m / k, n)
                    snprintf(pl.name, sizeof(pl.name), "gemm_tcgen05_%s_%c%c%s",
                             g.half == EB200_F16 ? "f16" : g.half == EB200_BF16 ? "bf16" : three ? "3xtf32" : "tf32",
                             g.a_sk == 1 ? 'k' : 'm', g.b_sk == 1 ? 'k' : 'n', g.splits > 1 ? "_splitk" : "");
                } else if (!force_simt && gemm_tall_supported(g) && (d->flags & 16) == 0) {
                    pl.impl = IMPL_GEMM_TALL;
                    g.splits = 2 * sm_count;          // one partial per CTA, two CTAs per SM
                    g.k_chunk = 0;
                    snprintf(pl.name, sizeof(pl.name), "gemm_tall_f32_splitk");
                } else {
                    pl.impl = IMPL_GEMM_SIMT;
                    snprintf(pl.name, sizeof(pl.name), "gemm_simt_f32%s", g.splits > 1 ? "_splitk" : "");
                }
                if (g.splits > 1) {
                    g.partial_off = scratch_floats;
                    scratch_floats += (long long)g.splits * g.batch * g.m * g.n;
                    pl.launches += 1;
                }
                pl.scratch_bytes = scratch_floats * 4;
                break;
            }
            if ((d->flags & 16384) != 0) {
                // sibling fusion (descriptor flag bit 14): besides this row reduce, the kernel also produces the column
                // maximum and the transposed copy of the one full-size operand it reads
                EB_REQUIRE(raxis == nk - 1 && nk == 2 && p.rop == EB200_R_SUM && p.n_in == 1, EB200_ERR_UNSUPPORTED,
                           "sibling fusion wants a sum over the rows of one [R, C] operand (other operands one-element)");
                const KOperand& x = p.in[0];
                EB_REQUIRE(x.dtype == EB200_F32 && !x.n_bounds && x.strides[1] == 1 && x.strides[0] == shape[1] && x.offset % 4 == 0 &&
                           shape[0] % 64 == 0 && shape[1] % 64 == 0, EB200_ERR_UNSUPPORTED,
                           "sibling fusion wants a contiguous f32 operand with R and C multiples of 64");
                const long long R = shape[0], Cc = shape[1];
                EB_REQUIRE(d->output.numel - d->output.offset >= R + Cc + R * Cc && d->output.offset % 4 == 0, EB200_ERR_BOUNDS,
                           "sibling fusion writes [y (R) | z (C) | t (C*R)] into its output");
                pl.impl = IMPL_SIBLINGS;
                pl.sib_rows = R; pl.sib_cols = Cc;
                pl.scratch_bytes = siblings_scratch_floats(R, Cc) * 4;
                pl.launches = 2;
                pl.algo_bytes = 4 * (2 * R * Cc + R + Cc);
                snprintf(pl.name, sizeof(pl.name), "siblings_rowsum_colmax_transpose");
                pl.chain = find_chain(p.prog, p.n_insns);
                return EB200_OK;
            }
            if (raxis == nk - 1) {
                pl.impl = IMPL_REDUCE_INNER;
                bool v = p.rlen % 4 == 0 && p.rlen >= 4;
                for (int i = 0; v && i < p.n_in; ++i) v = vec_ok(p.in[i], raxis, false);
                p.vec = v ? 4 : 1;
                pl.threads_per_row = p.rlen <= 64 ? 1 : (p.rlen <= 16384 ? 32 : 256);
                // short vectorised rows (an MLP's [65536, 256] . w): eight lanes per row, four rows per warp -- a warp per
                // row would leave every lane two dependent loads and nothing else in flight
                if (p.vec == 4 && p.rlen > 64 && p.rlen < 512 && p.kept >= 4096) pl.threads_per_row = 8;
                // (a row group that fills whole waves of CTAs -- 128 threads per row make 6.92 waves of config 2's
                // 8192 rows where a warp per row makes 1.73 -- measured SLOWER: 51.8 us against 47.1 us; the warp
                // form has no block barrier and keeps more rows in flight per SM)
                // tuning override (desc.flags bits 0-1): 1 -> thread, 2 -> warp, 3 -> CTA per row
                if ((d->flags & 7) == 1) pl.threads_per_row = 1;
                if ((d->flags & 7) == 2) pl.threads_per_row = 32;
                if ((d->flags & 7) == 3) pl.threads_per_row = 256;
                if ((d->flags & 7) == 4) pl.threads_per_row = 128;
                if ((d->flags & 7) == 5) pl.threads_per_row = 8;
                // few long rows: split each row over several CTAs, finish in a second pass
                long long ctas = pl.threads_per_row == 256 ? p.kept : 0;
                if (pl.threads_per_row == 256 && ctas < 2LL * sm_count && p.rlen >= 65536) {
                    long long want = (4LL * sm_count + ctas - 1) / std::max(1LL, ctas);
                    long long maxs = p.rlen / 16384;
                    int s = (int)std::max(1LL, std::min(want, std::min(maxs, 1024LL)));
                    if (s > 1) {
                        long long chunk = (p.rlen + s - 1) / s;
                        chunk = (chunk + 3) / 4 * 4;
                        s = (int)((p.rlen + chunk - 1) / chunk);
                        p.splits = s;
                        p.chunk = chunk;
                        pl.scratch_bytes = (int64_t)s * p.kept * 4;
                        pl.launches = 2;
                    }
                }
                snprintf(pl.name, sizeof(pl.name), "reduce_inner_t%d_v%d%s", pl.threads_per_row, p.vec, p.splits > 1 ? "_split" : "");
            } else {
                pl.impl = IMPL_REDUCE_OUTER;
                int inner = nk - 1;
                bool v = shape[inner] % 4 == 0 && vec_ok(p.out, inner, true);
                for (int i = 0; v && i < p.n_in; ++i) v = vec_ok(p.in[i], inner, false);
                p.vec = v ? 4 : 1;
                // enough thread blocks to fill the machine: split the reduce dim
                long long threads = p.kept / p.vec;
                long long blocks = (threads + 255) / 256;
                // few kept elements: a CTA is (kept / 4) column threads x row lanes (flag 16 keeps the plain form)
                pl.narrow = p.vec == 4 && threads <= 128 && p.rlen >= 256 && !(d->flags & 16);
                if (blocks < 4LL * sm_count && p.rlen >= 64) {
                    // one full wave: 4 resident CTAs per SM, all with equal work
                    long long want = (4LL * sm_count) / std::max(1LL, blocks);
                    // narrow: every CTA needs enough rows for its lanes (4 steps of 4 rows each at least)
                    const long long min_rows = pl.narrow ? 16LL * (256 / std::max(1LL, threads)) : 16;
                    int s = (int)std::max(1LL, std::min(want, std::min(p.rlen / min_rows, 1024LL)));
                    if (s > 1) {
                        long long chunk = (p.rlen + s - 1) / s;
                        s = (int)((p.rlen + chunk - 1) / chunk);
                        p.splits = s;
                        p.chunk = chunk;
                        pl.scratch_bytes = (int64_t)s * p.kept * 4;
                        pl.launches = 2;
                    }
                }
                if (p.splits <= 1) p.chunk = p.rlen;
                snprintf(pl.name, sizeof(pl.name), "reduce_outer_%sv%d%s", pl.narrow ? "narrow_" : "", p.vec, p.splits > 1 ? "_split" : "");
            }
            break;
        }
    }
    if (pl.impl == IMPL_EW || pl.impl == IMPL_REDUCE_INNER || pl.impl == IMPL_REDUCE_OUTER || pl.impl == IMPL_SCAN) {
        pl.chain = find_chain(p.prog, p.n_insns);
    }
    return EB200_OK;
}

}  // namespace eb200
