// ew_chain: fused elementwise chains (kernel class E_, src/lowerer/lower.rs:504-522)
// and strided gathers (class C_, lower.rs:448-501) that are not transposes.
//
// The reference renders a scalar nested loop per arithmetic node.  Here one
// launch evaluates a whole composed chain: each thread owns 4 consecutive
// elements along the innermost collapsed dim and moves them with 128-bit
// loads/stores, four such vectors in flight per thread; broadcast operands
// (stride 0) are read once per vector and one-element operands once per thread.
// The kernel is instantiated per collapsed rank (1, 2, 3, any) so the common
// cases carry no index arithmetic beyond what their rank needs.
// HBM-bound: algorithmic bytes = 4 B x (elements read + elements written).
#include "expr.cuh"
#include "index.cuh"

namespace eb200 {

constexpr int EW_U = 4;  // independent 128-bit vectors in flight per thread

// H16: some operand is stored as f16 / bf16 (kernels without such operands carry none of the type handling)
template <class F, int ND, bool H16>
__device__ __forceinline__ void load_vec4(const KParams& p, long long e, float (*in)[4]) {
    long long idx[KMAX_DIMS];
    if (ND != 1) decompose<ND>(p, e, idx);
    const int inner = ND > 0 ? ND - 1 : p.ndim - 1;
    const int n = F::nin(p);
#pragma unroll
    for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
        if (i >= n) break;
        const KOperand& o = p.in[i];
        const long long a = ND == 1 ? o.offset + e * o.strides[0] : operand_index<ND>(p, o, idx);
        if (H16 && o.dtype != EB200_F32) {
            // f16 / bf16 storage: four elements are one 64-bit load; the raw bits wait in in[i][0..1] and are
            // widened by widen_vec4 when the values are used, so that no load has a dependent instruction
            // between itself and the loads that follow it
            if (o.strides[inner] == 1) {
                const uint2 t = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned short*>(o.ptr) + a));
                in[i][0] = __uint_as_float(t.x); in[i][1] = __uint_as_float(t.y);
            } else {
                in[i][0] = load_elem(o, a);
            }
            continue;
        }
        const float* src = reinterpret_cast<const float*>(o.ptr) + a;
        if (o.strides[inner] == 1) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(src));
            in[i][0] = t.x; in[i][1] = t.y; in[i][2] = t.z; in[i][3] = t.w;
        } else {
            const float t = __ldg(src);
            in[i][0] = t; in[i][1] = t; in[i][2] = t; in[i][3] = t;
        }
    }
}

// second half of load_vec4 for 16-bit operands: raw bits -> four f32 values (a broadcast element -> four copies)
template <class F, int ND>
__device__ __forceinline__ void widen_vec4(const KParams& p, float (*in)[4]) {
    const int inner = ND > 0 ? ND - 1 : p.ndim - 1;
    const int n = F::nin(p);
#pragma unroll
    for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
        if (i >= n) break;
        const KOperand& o = p.in[i];
        if (o.dtype == EB200_F32) continue;
        if (o.strides[inner] == 1) {
            const unsigned x = __float_as_uint(in[i][0]), y = __float_as_uint(in[i][1]);
            if (o.dtype == EB200_F16) {
                const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&x));
                const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&y));
                in[i][0] = lo.x; in[i][1] = lo.y; in[i][2] = hi.x; in[i][3] = hi.y;
            } else {
                in[i][0] = __uint_as_float(x << 16); in[i][1] = __uint_as_float(x & 0xffff0000u);
                in[i][2] = __uint_as_float(y << 16); in[i][3] = __uint_as_float(y & 0xffff0000u);
            }
        } else {
            in[i][1] = in[i][0]; in[i][2] = in[i][0]; in[i][3] = in[i][0];
        }
    }
}

template <int ND, bool H16>
__device__ __forceinline__ void store_vec4(const KParams& p, long long e, const float* v) {
    long long a;
    if (ND == 1) {
        a = p.out.offset + e;
    } else {
        long long idx[KMAX_DIMS];
        decompose<ND>(p, e, idx);
        a = operand_index<ND>(p, p.out, idx);
    }
    if (!H16 || p.out.dtype == EB200_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out.ptr) + a) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        uint2 t;
        if (p.out.dtype == EB200_F16) {
            *reinterpret_cast<__half2*>(&t.x) = __floats2half2_rn(v[0], v[1]);
            *reinterpret_cast<__half2*>(&t.y) = __floats2half2_rn(v[2], v[3]);
        } else {
            *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
            *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
        }
        *reinterpret_cast<uint2*>(reinterpret_cast<unsigned short*>(p.out.ptr) + a) = t;
    }
}

// Vectors (or elements) in flight per thread: four for plain chains; two for chains that evaluate special
// functions -- their long dependent sequences want more resident warps (launch bounds: 4 CTAs per SM)
// rather than more work per thread.
// (16-bit operands move half the bytes per vector; their kernels are built for four CTAs per SM as well, so that
// twice the threads keep the same bytes in flight.)
// Kernels of rank 2 and more spend most of their instructions on index arithmetic per vector (broadcast rows and
// columns, strided operands): they, too, do better with more resident warps than with more vectors per thread
// (a [65536, 256] kernel with two broadcast operands: 42.8 us with four vectors and 2-3 CTAs per SM).
template <class F, bool H16, int ND = 1>
constexpr int ew_u() { return (F::kSpecial || ND != 1) ? 2 : EW_U; }

template <class F, int ND, bool H16>
__global__ void __launch_bounds__(256, (F::kSpecial || H16 || ND != 1) ? 4 : 1) ew_kernel(const __grid_constant__ KParams p) {
    constexpr int U = ew_u<F, H16, ND>();
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int n = F::nin(p);
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    if (p.vec == 4) {
        const long long nvec = p.total >> 2;
        // a CTA owns U consecutive 4 KB segments per iteration
        for (long long v0 = ((long long)blockIdx.x * U) * blockDim.x + threadIdx.x; v0 < nvec; v0 += U * stride) {
            float in[U][KMAX_IN][4];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long v = v0 + (long long)u * blockDim.x;
                if (v < nvec) load_vec4<F, ND, H16>(p, v << 2, in[u]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long v = v0 + (long long)u * blockDim.x;
                if (v < nvec) {
                    float r[4];
                    if (H16) widen_vec4<F, ND>(p, in[u]);
                    F::template eval<4>(p, in[u], r, cl);
                    store_vec4<ND, H16>(p, v << 2, r);
                }
            }
        }
    } else if (p.vec == 2) {
        // groups of four consecutive elements per thread (see the planner): one decomposition, the
        // multi-index then advances with carries; EW_G groups in flight
        constexpr int EW_G = 2;
        constexpr int RK = ND > 0 ? ND : KMAX_DIMS;
        const long long ngrp = p.total >> 2;
        for (long long g0 = ((long long)blockIdx.x * EW_G) * blockDim.x + threadIdx.x; g0 < ngrp; g0 += EW_G * stride) {
            float in[EW_G][KMAX_IN][4];
#pragma unroll
            for (int u = 0; u < EW_G; ++u) {
                const long long g = g0 + (long long)u * blockDim.x;
                if (g < ngrp) {
                    long long idx[KMAX_DIMS];
                    decompose<ND>(p, g << 2, idx);
                    // element addresses of the strided operands: computed once, then moved like an odometer
                    long long addr[KMAX_IN];
#pragma unroll
                    for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
                        if (i >= n) break;
                        addr[i] = p.in[i].flat ? 0 : operand_index<ND>(p, p.in[i], idx);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
                            if (i >= n) break;
                            const KOperand& o = p.in[i];
                            if (o.flat) {
                                if (j == 0) {
                                    const float4 t = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(o.ptr) + o.offset + (g << 2)));
                                    in[u][i][0] = t.x; in[u][i][1] = t.y; in[u][i][2] = t.z; in[u][i][3] = t.w;
                                }
                            } else if (o.n_bounds && !bounds_ok(p, o, idx)) {
                                in[u][i][j] = o.pad;
                            } else {
                                in[u][i][j] = load_elem(o, addr[i]);
                            }
                        }
                        if (j == 3) break;
                        // next element: innermost index + 1, carries outward; `tick` is the dim that moved
                        int tick = 0;
#pragma unroll
                        for (int d = RK - 1; d >= 0; --d) {
                            if (ND == 0 && d >= p.ndim) continue;
                            if (++idx[d] < p.shape[d]) { tick = d; break; }
                            idx[d] = 0;
                        }
#pragma unroll
                        for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
                            if (i >= n) break;
                            addr[i] += p.in[i].delta[tick];
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < EW_G; ++u) {
                const long long g = g0 + (long long)u * blockDim.x;
                if (g < ngrp) {
                    float r[4];
                    F::template eval<4>(p, in[u], r, cl);
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out.ptr) + p.out.offset + (g << 2)) = make_float4(r[0], r[1], r[2], r[3]);
                }
            }
        }
    } else {
        // scalar path: U independent elements per thread in flight (the loads of all of
        // them are issued before the first is evaluated); a CTA owns U consecutive
        // 256-element segments per iteration
        for (long long e0 = ((long long)blockIdx.x * U) * blockDim.x + threadIdx.x; e0 < p.total; e0 += U * stride) {
            float in[U][KMAX_IN][1];
            long long oa[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long e = e0 + (long long)u * blockDim.x;
                if (e < p.total) {
                    long long idx[KMAX_DIMS];
                    decompose<ND>(p, e, idx);
#pragma unroll
                    for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
                        if (i >= n) break;
                        const KOperand& o = p.in[i];
                        if (o.n_bounds && !bounds_ok(p, o, idx)) in[u][i][0] = o.pad;
                        else in[u][i][0] = load_elem(o, operand_index<ND>(p, o, idx));
                    }
                    oa[u] = operand_index<ND>(p, p.out, idx);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long e = e0 + (long long)u * blockDim.x;
                if (e < p.total) {
                    float r[1];
                    F::template eval<1>(p, in[u], r, cl);
                    store_elem(p.out, oa[u], r[0]);
                }
            }
        }
    }
}

// ---- flat kernels over 16-bit storage: eight elements per thread ---------------------------------------
// With f16 / bf16 operands a vector of four elements is 8 bytes: the four-wide kernel above runs out of issue
// slots (index arithmetic and loop control per vector) at 0.66 of the copy bandwidth.  For the flat case (one
// collapsed dim, every operand unit-stride or broadcast, 16-byte aligned) a thread takes eight elements: one
// 128-bit load per 16-bit operand, two per f32 operand, one 128-bit store of eight 16-bit results.
template <class F>
__global__ void __launch_bounds__(256, 4) ew16x8_kernel(const __grid_constant__ KParams p) {
    constexpr int U = F::kSpecial ? 1 : 2;
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int n = F::nin(p);
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    const long long nvec = p.total >> 3;
    for (long long v0 = ((long long)blockIdx.x * U) * blockDim.x + threadIdx.x; v0 < nvec; v0 += U * stride) {
        float lo[U][NI][4], hi[U][NI][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v >= nvec) break;
            const long long e = v << 3;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (i >= n) break;
                const KOperand& o = p.in[i];
                if (o.strides[0] == 0) {
                    lo[u][i][0] = load_elem(o, o.offset);
                } else if (o.dtype == EB200_F32) {
                    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(o.ptr) + o.offset + e);
                    const float4 a = __ldg(src), b = __ldg(src + 1);
                    lo[u][i][0] = a.x; lo[u][i][1] = a.y; lo[u][i][2] = a.z; lo[u][i][3] = a.w;
                    hi[u][i][0] = b.x; hi[u][i][1] = b.y; hi[u][i][2] = b.z; hi[u][i][3] = b.w;
                } else {        // raw bits now, widened below (no dependent instruction between the loads)
                    const uint4 t = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(o.ptr) + o.offset + e));
                    lo[u][i][0] = __uint_as_float(t.x); lo[u][i][1] = __uint_as_float(t.y);
                    lo[u][i][2] = __uint_as_float(t.z); lo[u][i][3] = __uint_as_float(t.w);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v >= nvec) break;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (i >= n) break;
                const KOperand& o = p.in[i];
                if (o.strides[0] == 0) {
                    const float t = lo[u][i][0];
#pragma unroll
                    for (int j = 0; j < 4; ++j) { lo[u][i][j] = t; hi[u][i][j] = t; }
                } else if (o.dtype != EB200_F32) {
                    unsigned w4[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) w4[j] = __float_as_uint(lo[u][i][j]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float a, b;
                        if (o.dtype == EB200_F16) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[j]));
                            a = f.x; b = f.y;
                        } else {
                            a = __uint_as_float(w4[j] << 16); b = __uint_as_float(w4[j] & 0xffff0000u);
                        }
                        if (j < 2) { lo[u][i][2 * j] = a; lo[u][i][2 * j + 1] = b; }
                        else { hi[u][i][2 * (j - 2)] = a; hi[u][i][2 * (j - 2) + 1] = b; }
                    }
                }
            }
            float r[8];
            F::template eval<4>(p, lo[u], r, cl);
            F::template eval<4>(p, hi[u], r + 4, cl);
            const long long e = v << 3;
            if (p.out.dtype == EB200_F32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out.ptr) + p.out.offset + e);
                dst[0] = make_float4(r[0], r[1], r[2], r[3]);
                dst[1] = make_float4(r[4], r[5], r[6], r[7]);
            } else {
                uint4 t;
                unsigned* tw = reinterpret_cast<unsigned*>(&t);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (p.out.dtype == EB200_F16) *reinterpret_cast<__half2*>(&tw[j]) = __floats2half2_rn(r[2 * j], r[2 * j + 1]);
                    else *reinterpret_cast<__nv_bfloat162*>(&tw[j]) = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(p.out.ptr) + p.out.offset + e) = t;
            }
        }
    }
}

template <class F>
static int launch_one(Device* dev, const KParams& p) {
    long long work = p.vec == 1 ? p.total : (p.total >> 2);
    if (work <= 0) return EB200_OK;
    // 16-bit operands on the vector path: instantiated for rank 1 and for any rank only
    bool h16 = false;
    if (p.vec == 4) {
        for (int i = 0; i < p.n_in; ++i) h16 = h16 || p.in[i].dtype == EB200_F16 || p.in[i].dtype == EB200_BF16;
        h16 = h16 || p.out.dtype == EB200_F16 || p.out.dtype == EB200_BF16;
    }
    // ranks 1-4 have their own instantiation; scalar kernels of rank 5 and 6 share the rank-6 one
    // (dims past the rank have extent 1 and stride 0); everything else takes the any-rank form
    int nd = 0;
    if (p.total < (1LL << 31)) nd = p.ndim <= 4 ? p.ndim : (p.ndim <= 6 && p.vec != 4 ? 6 : 0);
    if (p.vec == 2 && nd == 1) nd = 0;      // (rank 1 never plans groups of four; keep the switch total)
    if (h16 && nd != 1) nd = 0;
    const int u = (F::kSpecial || nd != 1) ? 2 : EW_U;      // ew_u<F, H16, ND>() of the instantiation that will run
    long long per_block = 256LL * (p.vec == 2 ? 2 : u);
    long long blocks = (work + per_block - 1) / per_block;
    long long cap = (long long)dev->prop.multiProcessorCount * 32;
    if (blocks > cap) blocks = cap;
    const unsigned g = (unsigned)blocks;
    if (h16) {
        // flat, a multiple of eight elements, every operand 16-byte aligned: eight elements per thread
        bool wide = nd == 1 && (p.total & 7) == 0;
        for (int i = 0; wide && i <= p.n_in; ++i) {
            const KOperand& o = i < p.n_in ? p.in[i] : p.out;
            if (o.strides[0] == 0 && i < p.n_in) continue;
            const int esz = o.dtype == EB200_F32 ? 4 : 2;
            wide = (o.dtype == EB200_F32 || o.dtype == EB200_F16 || o.dtype == EB200_BF16) && o.strides[0] == 1 &&
                   ((reinterpret_cast<uintptr_t>(o.ptr) + (uintptr_t)o.offset * esz) & 15) == 0;
        }
        if (wide) {
            const long long nv8 = p.total >> 3, per8 = 256LL * (F::kSpecial ? 1 : 2);
            const long long b8 = std::min<long long>((nv8 + per8 - 1) / per8, cap);
            ew16x8_kernel<F><<<(unsigned)b8, 256, 0, dev->stream>>>(p);
        } else if (nd == 1) ew_kernel<F, 1, true><<<g, 256, 0, dev->stream>>>(p);
        else ew_kernel<F, 0, true><<<g, 256, 0, dev->stream>>>(p);
    } else
    switch (nd) {
        case 1: ew_kernel<F, 1, false><<<g, 256, 0, dev->stream>>>(p); break;
        case 2: ew_kernel<F, 2, false><<<g, 256, 0, dev->stream>>>(p); break;
        case 3: ew_kernel<F, 3, false><<<g, 256, 0, dev->stream>>>(p); break;
        case 4: ew_kernel<F, 4, false><<<g, 256, 0, dev->stream>>>(p); break;
        case 6: ew_kernel<F, 6, false><<<g, 256, 0, dev->stream>>>(p); break;
        default: ew_kernel<F, 0, false><<<g, 256, 0, dev->stream>>>(p); break;
    }
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

int launch_ew(Device* dev, const Plan& plan, const KParams& p) {
    switch (plan.chain) {
#define X(i) case i: return launch_one<Compiled<Chain##i>>(dev, p);
        EB_FOR_EACH_CHAIN(X)
#undef X
        default: return launch_one<Interp>(dev, p);
    }
}

}  // namespace eb200
