// Evaluation of `map` expressions on the device.
//
// A map is the expression tree of a lowered kernel over Wildcard inputs
// (src/graph/ops.rs:69-95).  Two evaluators exist behind one interface:
//
//  * compiled functors (chains_gen.inc) for the expression shapes the build
//    knows about: the expression is ordinary C++ the compiler keeps in
//    registers, constants come from KParams::consts;
//  * Interp, a postfix bytecode interpreter, serves every other expression.
//
// Semantics follow what the reference renders for its C backend
// (src/backend/renderer.rs:268-441, crates/backend-c/src/renderer.rs:181-206):
// fmaxf, sqrtf, log2f, exp2f, sinf, floorf, `1.0f / x`; comparisons and logic
// yield 1 or 0; Select tests its condition against zero.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"

namespace eb200 {

__device__ __forceinline__ float op_lt(float a, float b) { return a < b ? 1.0f : 0.0f; }
__device__ __forceinline__ float op_and(float a, float b) { return (a != 0.0f && b != 0.0f) ? 1.0f : 0.0f; }
__device__ __forceinline__ float op_not(float a) { return a == 0.0f ? 1.0f : 0.0f; }
__device__ __forceinline__ float op_select(float c, float t, float e) { return c != 0.0f ? t : e; }
// 1.0f / x, correctly rounded (the same value the division gives) in fewer instructions
__device__ __forceinline__ float op_recip(float a) { return __frcp_rn(a); }
// exp2 / log2 on the special-function unit: relative error below 2^-22 (2.4e-7), well inside the
// 1e-5 the elementwise contract allows.  Fused chains such as tanh and its gradient evaluate
// several of these per element and are bound by the FP32 pipe, not by HBM: the library
// routines (exp2f / log2f, with their range handling) cost four times as many instructions.
__device__ __forceinline__ float op_exp2(float a) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));      // (results below 2^-126 flush to zero)
    return r;
}
__device__ __forceinline__ float op_log2(float a) {
    float r;
    asm("lg2.approx.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}
__device__ __forceinline__ float op_rem(float a, float b) {
    long long x = (long long)a, y = (long long)b;
    return y ? (float)(x % y) : 0.0f;
}
__device__ __forceinline__ float op_idiv(float a, float b) {
    long long x = (long long)a, y = (long long)b;
    return y ? (float)(x / y) : 0.0f;
}
__device__ __forceinline__ float op_cast(float a, int dtype) {
    if (dtype == EB200_F32) return a;
    if (dtype == EB200_BOOL) return a != 0.0f ? 1.0f : 0.0f;
    if (dtype == EB200_F16) return __half2float(__float2half_rn(a));
    if (dtype == EB200_BF16) return __bfloat162float(__float2bfloat16_rn(a));
    return truncf(a);
}

// ---- typed element access ---------------------------------------------------------
__device__ __forceinline__ float load_elem(const KOperand& o, long long idx) {
    switch (o.dtype) {
        case EB200_F32: return reinterpret_cast<const float*>(o.ptr)[idx];
        case EB200_BOOL: return (float)reinterpret_cast<const unsigned char*>(o.ptr)[idx];
        case EB200_I32: return (float)reinterpret_cast<const int*>(o.ptr)[idx];
        case EB200_F16: return __half2float(reinterpret_cast<const __half*>(o.ptr)[idx]);
        case EB200_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(o.ptr)[idx]);
        default: return 0.0f;
    }
}

__device__ __forceinline__ void store_elem(const KOperand& o, long long idx, float v) {
    switch (o.dtype) {
        case EB200_F32: reinterpret_cast<float*>(o.ptr)[idx] = v; break;
        case EB200_BOOL: reinterpret_cast<unsigned char*>(o.ptr)[idx] = (unsigned char)(v != 0.0f); break;
        case EB200_I32: reinterpret_cast<int*>(o.ptr)[idx] = (int)v; break;
        case EB200_F16: reinterpret_cast<__half*>(o.ptr)[idx] = __float2half_rn(v); break;
        case EB200_BF16: reinterpret_cast<__nv_bfloat16*>(o.ptr)[idx] = __float2bfloat16_rn(v); break;
        default: break;
    }
}

// Bound conditions of a padded view: all of lo <= c + coef.idx < hi.
__device__ __forceinline__ bool bounds_ok(const KParams& p, const KOperand& o, const long long* idx) {
    for (int b = 0; b < o.n_bounds; ++b) {
        const KBound& kb = p.bounds[o.bound_begin + b];
        long long e = kb.c;
#pragma unroll
        for (int d = 0; d < KMAX_DIMS; ++d)
            if (d < p.ndim) e += kb.coef[d] * idx[d];
        if (e < kb.lo || e >= kb.hi) return false;
    }
    return true;
}

// ---- bytecode interpreter ---------------------------------------------------------
struct Interp {
    static constexpr bool kCompiled = false;
    static constexpr bool kSpecial = false;
    static constexpr int kNin = KMAX_IN;
    static constexpr int kNconst = KMAX_CONSTS;
    __device__ __forceinline__ static int nin(const KParams& p) { return p.n_in; }

    template <int V>
    __device__ static void eval(const KParams& p, const float (*in)[V], float* out, const float* cl) {
        float st[KSTACK][V];
        int sp = 0;
        for (int pc = 0; pc < p.n_insns; ++pc) {
            const KInsn ins = p.prog[pc];
            switch (ins.op) {
                case EB200_OP_LOAD:
#pragma unroll
                    for (int v = 0; v < V; ++v) st[sp][v] = in[ins.arg][v];
                    ++sp; break;
                case EB200_OP_CONST:
#pragma unroll
                    for (int v = 0; v < V; ++v) st[sp][v] = cl[ins.arg];
                    ++sp; break;
#define EB_BIN(OPC, EXPR)                                                       \
    case OPC:                                                                   \
        --sp;                                                                   \
        _Pragma("unroll") for (int v = 0; v < V; ++v) {                         \
            float a = st[sp - 1][v], b = st[sp][v];                             \
            st[sp - 1][v] = (EXPR);                                             \
        }                                                                       \
        break;
#define EB_UN(OPC, EXPR)                                                        \
    case OPC:                                                                   \
        _Pragma("unroll") for (int v = 0; v < V; ++v) {                         \
            float a = st[sp - 1][v];                                            \
            st[sp - 1][v] = (EXPR);                                             \
        }                                                                       \
        break;
                EB_BIN(EB200_OP_ADD, a + b)
                EB_BIN(EB200_OP_MUL, a * b)
                EB_BIN(EB200_OP_MAX, fmaxf(a, b))
                EB_BIN(EB200_OP_LT, op_lt(a, b))
                EB_BIN(EB200_OP_AND, op_and(a, b))
                EB_BIN(EB200_OP_REM, op_rem(a, b))
                EB_BIN(EB200_OP_IDIV, op_idiv(a, b))
                EB_UN(EB200_OP_RECIP, op_recip(a))
                EB_UN(EB200_OP_SQRT, sqrtf(a))
                EB_UN(EB200_OP_LOG2, op_log2(a))
                EB_UN(EB200_OP_EXP2, op_exp2(a))
                EB_UN(EB200_OP_SIN, sinf(a))
                EB_UN(EB200_OP_FLOOR, floorf(a))
                EB_UN(EB200_OP_NOT, op_not(a))
                EB_UN(EB200_OP_CAST, op_cast(a, ins.arg))
#undef EB_BIN
#undef EB_UN
                case EB200_OP_SELECT:
                    sp -= 2;
#pragma unroll
                    for (int v = 0; v < V; ++v) st[sp - 1][v] = op_select(st[sp - 1][v], st[sp][v], st[sp + 1][v]);
                    break;
                case EB200_OP_FMA:
                    sp -= 2;
#pragma unroll
                    for (int v = 0; v < V; ++v) st[sp - 1][v] = fmaf(st[sp - 1][v], st[sp][v], st[sp + 1][v]);
                    break;
                default: break;
            }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) out[v] = st[0][v];
    }
};

// ---- compiled functors ------------------------------------------------------------
// A generated `struct ChainN { static constexpr int NIN; static float f(w, c); }`
// is wrapped into the evaluator interface here.
template <class C>
struct Compiled {
    static constexpr bool kCompiled = true;
    static constexpr bool kSpecial = C::SPECIAL != 0;   // evaluates exp2 / log2 / recip / sqrt / sin: long dependent chains
    static constexpr int kNin = C::NIN > 0 ? C::NIN : 1;
    static constexpr int kNconst = C::NCONST > 0 ? C::NCONST : 1;
    __device__ __forceinline__ static int nin(const KParams&) { return C::NIN; }

    template <int V>
    __device__ __forceinline__ static void eval(const KParams& p, const float (*in)[V], float* out, const float* cl) {
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float w[C::NIN > 0 ? C::NIN : 1];
#pragma unroll
            for (int i = 0; i < C::NIN; ++i) w[i] = in[i][v];
            out[v] = C::f(w, cl);
        }
    }
};

#include "chains_gen.inc"

// Constant table of a launch: literal constants of the map, and one-element
// tensor operands, which the plan turns into constants read once per thread.
template <class F>
__device__ __forceinline__ void load_consts(const KParams& p, float* cl) {
#pragma unroll
    for (int j = 0; j < F::kNconst; ++j) {
        cl[j] = 0.0f;
        if (j < p.n_consts) cl[j] = p.cptr[j] ? __ldg(p.cptr[j]) : p.consts[j];
    }
}

// Reduce combiners (src/graph/node.rs:29-77).
template <int ROP> struct Red;
template <> struct Red<EB200_R_SUM> {
    __device__ __forceinline__ static float identity() { return 0.0f; }
    __device__ __forceinline__ static float combine(float a, float b) { return a + b; }
};
template <> struct Red<EB200_R_MAX> {
    __device__ __forceinline__ static float identity() { return -INFINITY; }
    __device__ __forceinline__ static float combine(float a, float b) { return fmaxf(a, b); }
};
template <> struct Red<EB200_R_MIN> {
    __device__ __forceinline__ static float identity() { return INFINITY; }
    __device__ __forceinline__ static float combine(float a, float b) { return a < b ? a : b; }
};
template <> struct Red<EB200_R_PROD> {
    __device__ __forceinline__ static float identity() { return 1.0f; }
    __device__ __forceinline__ static float combine(float a, float b) { return a * b; }
};

__device__ __forceinline__ float red_identity(int rop) {
    switch (rop) {
        case EB200_R_MAX: return -INFINITY;
        case EB200_R_MIN: return INFINITY;
        case EB200_R_PROD: return 1.0f;
        default: return 0.0f;
    }
}
__device__ __forceinline__ float red_combine(int rop, float a, float b) {
    switch (rop) {
        case EB200_R_MAX: return fmaxf(a, b);
        case EB200_R_MIN: return a < b ? a : b;
        case EB200_R_PROD: return a * b;
        default: return a + b;
    }
}

}  // namespace eb200
