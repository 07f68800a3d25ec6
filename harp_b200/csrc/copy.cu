// Data-movement kernels: transposing copies, scatter-add (fold) and the SGD update.
//
// transpose_copy  `x.permute(..).contiguous()` -- GraphNode::contiguous
//                 (src/graph/node.rs:431-445) lowers to an identity-map E_
//                 kernel over a permuted view, and un-inlinable views lower to
//                 C_ kernels (src/lowerer/lower.rs:448-501); both are nested
//                 scalar loops with strided reads in the reference.  Here: the
//                 input is unit-stride along dim R, the output along the last
//                 dim C; 64x64 tiles go through shared memory so both the
//                 global reads (along R) and writes (along C) are 128-bit and
//                 coalesced.  All other dims are batch.  Moves raw 32-bit words:
//                 bit-exact.  HBM-bound: 8 B per element.
// scatter_add     S_ kernels (src/lowerer/lower.rs:580-683): zero fill, then
//                 out[dst(idx)] += in[idx]; the CUDA renderer of the reference
//                 uses atomicAdd as well (crates/backend-cuda/src/renderer.rs:461-481).
// sgd_update      p - lr*g, the host loop of SGD::step
//                 (crates/nn/src/optim/sgd.rs:88-92) kept on the device; separate
//                 multiply and subtract roundings, like the Rust loop.
#include <stdlib.h>

#include <algorithm>

#include "expr.cuh"
#include "index.cuh"

namespace eb200 {

struct TrParams {
    int nbatch;                       // batch dims
    long long bshape[KMAX_DIMS];
    long long bin[KMAX_DIMS];         // input strides of batch dims
    long long bout[KMAX_DIMS];        // output strides of batch dims
    long long R, C;                   // extents
    long long in_sc;                  // input stride along C (input stride along R is 1)
    long long out_sr;                 // output stride along R (output stride along C is 1)
    long long in_off, out_off;
    long long tiles_r, tiles_c, tiles;
};

template <int TT>
__global__ void __launch_bounds__(256) transpose_kernel(const __grid_constant__ TrParams q,
                                                        const uint32_t* __restrict__ in,
                                                        uint32_t* __restrict__ out) {
    // tile[r][c] with an odd pitch: written column-wise while loading, read
    // row-wise while storing.  Within a warp 8 lanes span 32 words of the
    // contiguous dim and 4 lanes span 4 lines, so every shared-memory access of
    // a warp touches 32 distinct banks.
    extern __shared__ uint32_t tile_mem[];
    constexpr int P = TT + 1;
    constexpr int QN = TT / 32;        // 32-word segments along the contiguous dim
    constexpr int LPP = (8 / QN) * 4;  // lines covered per pass by the 8 warps
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tx = lane & 7, ty = lane >> 3;
    const int seg = (warp % QN) * 32;
    const int line0 = (warp / QN) * 4 + ty;
    for (long long t = blockIdx.x; t < q.tiles; t += gridDim.x) {
        long long rem = t;
        const long long tc = rem % q.tiles_c; rem /= q.tiles_c;
        const long long tr = rem % q.tiles_r; rem /= q.tiles_r;
        long long ibase = q.in_off, obase = q.out_off;
        for (int d = q.nbatch - 1; d >= 0; --d) {
            const long long i = rem % q.bshape[d];
            rem /= q.bshape[d];
            ibase += i * q.bin[d];
            obase += i * q.bout[d];
        }
        const long long r0 = tr * TT, c0 = tc * TT;
        // load: input lines have fixed c and are contiguous along r
#pragma unroll
        for (int pass = 0; pass < TT / LPP; ++pass) {
            const int cl = pass * LPP + line0;
            const int rl = seg + tx * 4;
            const long long c = c0 + cl, r = r0 + rl;
            if (c < q.C && r < q.R) {
                const long long a = ibase + c * q.in_sc + r;
                if (r + 3 < q.R && (a & 3) == 0) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(in + a));
                    tile_mem[rl * P + cl] = v.x; tile_mem[(rl + 1) * P + cl] = v.y;
                    tile_mem[(rl + 2) * P + cl] = v.z; tile_mem[(rl + 3) * P + cl] = v.w;
                } else {
                    for (int i = 0; i < 4 && r + i < q.R; ++i) tile_mem[(rl + i) * P + cl] = __ldg(in + a + i);
                }
            }
        }
        __syncthreads();
        // store: output lines have fixed r and are contiguous along c
#pragma unroll
        for (int pass = 0; pass < TT / LPP; ++pass) {
            const int rl = pass * LPP + line0;
            const int cl = seg + tx * 4;
            const long long r = r0 + rl, c = c0 + cl;
            if (r < q.R && c < q.C) {
                const long long a = obase + r * q.out_sr + c;
                const uint32_t* src = tile_mem + rl * P + cl;
                if (c + 3 < q.C && (a & 3) == 0) {
                    uint4 v;
                    v.x = src[0]; v.y = src[1]; v.z = src[2]; v.w = src[3];
                    *reinterpret_cast<uint4*>(out + a) = v;
                } else {
                    for (int i = 0; i < 4 && c + i < q.C; ++i) out[a + i] = src[i];
                }
            }
        }
        __syncthreads();
    }
}

// Persistent form for extents that are multiples of 64 with 16-byte aligned lines:
// a CTA walks tiles blockIdx.x, +gridDim.x, ...; while it writes tile i out of
// shared memory, the four 128-bit loads of tile i+1 are already in flight in
// registers, so the memory system never drains between a CTA's tiles.
__global__ void __launch_bounds__(256) transpose_pipe_kernel(const __grid_constant__ TrParams q,
                                                             const uint32_t* __restrict__ in,
                                                             uint32_t* __restrict__ out) {
    constexpr int TT = 64, P = TT + 1;
    __shared__ uint32_t tile_mem[TT * P];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tx = lane & 7, ty = lane >> 3;
    const int seg = (warp & 1) * 32;
    const int line0 = (warp >> 1) * 4 + ty;
    auto bases = [&](long long t, long long& ib, long long& ob) {
        long long rem = t;
        const long long tc = rem % q.tiles_c; rem /= q.tiles_c;
        const long long tr = rem % q.tiles_r; rem /= q.tiles_r;
        long long ibase = q.in_off, obase = q.out_off;
        for (int d = q.nbatch - 1; d >= 0; --d) {
            const long long i = rem % q.bshape[d];
            rem /= q.bshape[d];
            ibase += i * q.bin[d];
            obase += i * q.bout[d];
        }
        ib = ibase + tc * TT * q.in_sc + tr * TT;      // element (c0, r0) of the input
        ob = obase + tr * TT * q.out_sr + tc * TT;     // element (r0, c0) of the output
    };
    // two tiles of loads in flight: slot 0 = the tile to store next, slot 1 = the one after
    constexpr int DEPTH = 2;
    uint4 nxt[DEPTH][4];
    long long obq[DEPTH];
    long long ib, ob;
    const long long step = gridDim.x;
#pragma unroll
    for (int dpt = 0; dpt < DEPTH; ++dpt) {
        const long long tt = (long long)blockIdx.x + dpt * step;
        if (tt < q.tiles) {
            bases(tt, ib, ob);
            obq[dpt] = ob;
#pragma unroll
            for (int pass = 0; pass < 4; ++pass)
                nxt[dpt][pass] = __ldg(reinterpret_cast<const uint4*>(in + ib + (long long)(pass * 16 + line0) * q.in_sc + seg + tx * 4));
        }
    }
    for (long long t = blockIdx.x; t < q.tiles; t += step) {
        const long long ob_cur = obq[0];
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int cl = pass * 16 + line0, rl = seg + tx * 4;
            tile_mem[rl * P + cl] = nxt[0][pass].x; tile_mem[(rl + 1) * P + cl] = nxt[0][pass].y;
            tile_mem[(rl + 2) * P + cl] = nxt[0][pass].z; tile_mem[(rl + 3) * P + cl] = nxt[0][pass].w;
        }
        __syncthreads();
        // shift the queue and refill its tail
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) nxt[0][pass] = nxt[1][pass];
        obq[0] = obq[1];
        const long long tn = t + DEPTH * step;
        if (tn < q.tiles) {
            bases(tn, ib, ob);
            obq[1] = ob;
#pragma unroll
            for (int pass = 0; pass < 4; ++pass)
                nxt[1][pass] = __ldg(reinterpret_cast<const uint4*>(in + ib + (long long)(pass * 16 + line0) * q.in_sc + seg + tx * 4));
        }
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int rl = pass * 16 + line0, cl = seg + tx * 4;
            const uint32_t* src = tile_mem + rl * P + cl;
            uint4 v;
            v.x = src[0]; v.y = src[1]; v.z = src[2]; v.w = src[3];
            *reinterpret_cast<uint4*>(out + ob_cur + (long long)rl * q.out_sr + cl) = v;
        }
        __syncthreads();
    }
}

template <int TT>
static int launch_tr(Device* dev, TrParams& q, const uint32_t* in, uint32_t* out) {
    q.tiles_r = (q.R + TT - 1) / TT;
    q.tiles_c = (q.C + TT - 1) / TT;
    q.tiles *= q.tiles_r * q.tiles_c;   // q.tiles holds the batch count on entry
    if (q.tiles <= 0) return EB200_OK;
    const size_t smem = (size_t)TT * (TT + 1) * sizeof(uint32_t);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        EB_CHECK_CUDA(cudaFuncSetAttribute(transpose_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    long long blocks = q.tiles;
    const long long cap = (1LL << 31) - 1;
    if (blocks > cap) blocks = cap;
    transpose_kernel<TT><<<(unsigned)blocks, 256, smem, dev->stream>>>(q, in, out);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

int launch_transpose(Device* dev, const Plan& plan, const void* in, void* out) {
    const KParams& p = plan.p;
    const int rd = p.raxis, cd = p.ndim - 1;
    TrParams q{};
    q.nbatch = 0;
    for (int d = 0; d < p.ndim; ++d) {
        if (d == rd || d == cd) continue;
        q.bshape[q.nbatch] = p.shape[d];
        q.bin[q.nbatch] = p.in[0].strides[d];
        q.bout[q.nbatch] = p.out.strides[d];
        ++q.nbatch;
    }
    q.R = p.shape[rd];
    q.C = p.shape[cd];
    q.in_sc = p.in[0].strides[cd];
    q.out_sr = p.out.strides[rd];
    q.in_off = p.in[0].offset;
    q.out_off = p.out.offset;
    long long batch = 1;
    for (int d = 0; d < q.nbatch; ++d) batch *= q.bshape[d];
    q.tiles = batch;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(in);
    uint32_t* dst = reinterpret_cast<uint32_t*>(out);
    // 64x64 tiles: 8 resident CTAs per SM; 128x128 tiles measured 30 % slower
    // (3 CTAs per SM leave too few loads in flight)
    bool pipe = q.R % 64 == 0 && q.C % 64 == 0 && q.in_sc % 4 == 0 && q.out_sr % 4 == 0 &&
                q.in_off % 4 == 0 && q.out_off % 4 == 0;
    for (int d = 0; d < q.nbatch && pipe; ++d) pipe = q.bin[d] % 4 == 0 && q.bout[d] % 4 == 0;
    if (pipe && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        q.tiles_r = q.R / 64;
        q.tiles_c = q.C / 64;
        q.tiles *= q.tiles_r * q.tiles_c;
        if (q.tiles <= 0) return EB200_OK;
        const int per_sm = 8;
        const long long blocks = std::min<long long>(q.tiles, (long long)dev->prop.multiProcessorCount * per_sm);
        transpose_pipe_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(q, src, dst);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
        return EB200_OK;
    }
    return launch_tr<64>(dev, q, src, dst);
}

// ---- scatter-add ---------------------------------------------------------------------
__global__ void __launch_bounds__(256) fill_zero_kernel(float* __restrict__ out, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = 0.0f;
}

// PLAIN: the planner has shown that no two iteration points address the same output element (a fold of disjoint
// windows): the zero fill plus one add is a store of v + 0 (the + 0 keeps the sign of a zero term as the add would).
template <bool PLAIN>
__global__ void __launch_bounds__(256, 4) scatter_add_kernel(const __grid_constant__ KParams p) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    float* out = reinterpret_cast<float*>(p.out.ptr);
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < p.total; e += stride) {
        long long idx[KMAX_DIMS];
        decompose(p, e, idx);
        const KOperand& o = p.in[0];
        float v;
        if (o.n_bounds && !bounds_ok(p, o, idx)) v = o.pad;
        else v = load_elem(o, operand_index(p, o, idx));
        if (PLAIN) out[operand_index(p, p.out, idx)] = v + 0.0f;
        else atomicAdd(out + operand_index(p, p.out, idx), v);
    }
}

int launch_scatter(Device* dev, const Plan& plan, const KParams& p) {
    const long long cap = (long long)dev->prop.multiProcessorCount * 16;
    if (plan.out_numel > 0) {
        long long blocks = (plan.out_numel + 255) / 256;
        if (blocks > cap) blocks = cap;
        fill_zero_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(reinterpret_cast<float*>(p.out.ptr), plan.out_numel);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
    }
    if (p.total > 0) {
        long long blocks = (p.total + 255) / 256;
        if (blocks > cap) blocks = cap;
        if (plan.scatter_plain) scatter_add_kernel<true><<<(unsigned)blocks, 256, 0, dev->stream>>>(p);
        else scatter_add_kernel<false><<<(unsigned)blocks, 256, 0, dev->stream>>>(p);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
    }
    return EB200_OK;
}

// ---- fold as a gather ---------------------------------------------------------------------
// The scatter-add above serialises on atomics (a 3x3 fold adds nine terms into every element, from nine different
// threads).  When the scatter is a fold -- iteration dims (..., Ho, Wo, KH, KW), output element (h, w) =
// (ho*sh + kh*dh, wo*sw + kw*dw) of a dense plane -- each output element can collect its own terms instead: a thread
// per output element walks the windows that cover it, largest (kh, kw) first, which is the order of increasing
// (ho, wo) in which the reference's sequential loop nest adds them (src/lowerer/lower.rs:580-683): the result is
// bit-identical to that loop, independent of the launch.  Elements of the planes no window reaches (and the rest of
// the output buffer) keep the zero fill.
struct FastDiv {                 // exact n / d for n < 2^31: (n * mul) >> shr, with mul = ceil(2^(31+l) / d), l = ceil(log2 d)
    unsigned d, mul, shr;
};
static FastDiv make_fastdiv(unsigned d) {
    FastDiv f;
    f.d = d ? d : 1;
    int l = 0;
    while ((1ULL << l) < f.d) ++l;
    f.mul = (unsigned)((((1ULL << (31 + l)) + f.d - 1) / f.d));
    f.shr = (unsigned)(31 + l);
    return f;
}
__device__ __forceinline__ unsigned fdiv(unsigned n, const FastDiv& f) { return (unsigned)(((unsigned long long)n * f.mul) >> f.shr); }

struct FoldParams {
    int n_outer;
    FastDiv oshape[KMAX_DIMS];
    long long o_in[KMAX_DIMS], o_out[KMAX_DIMS];
    FastDiv hout, wout, sh, sw;
    unsigned Ho, Wo, KH, KW, dh, dw, total;
    long long pitch, in_ho, in_wo, in_kh, in_kw, in_off, out_off;
};

__global__ void __launch_bounds__(256) fold_gather_kernel(const __grid_constant__ FoldParams q, const float* __restrict__ in,
                                                          float* __restrict__ out) {
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < q.total; e += stride) {
        const unsigned t = fdiv(e, q.wout), w = e - t * q.wout.d;
        unsigned o = fdiv(t, q.hout);
        const unsigned h = t - o * q.hout.d;
        long long ib = q.in_off, ob = q.out_off + (long long)h * q.pitch + w;
#pragma unroll 1
        for (int j = q.n_outer - 1; j >= 0; --j) {
            const unsigned nx = fdiv(o, q.oshape[j]), ix = o - nx * q.oshape[j].d;
            ib += (long long)ix * q.o_in[j];
            ob += (long long)ix * q.o_out[j];
            o = nx;
        }
        float acc = 0.0f;
        for (int kh = (int)q.KH - 1; kh >= 0; --kh) {
            const int hh = (int)h - kh * (int)q.dh;
            if (hh < 0) continue;
            const unsigned ho = fdiv((unsigned)hh, q.sh);
            if (ho * q.sh.d != (unsigned)hh || ho >= q.Ho) continue;
            const long long rb = ib + (long long)ho * q.in_ho + (long long)kh * q.in_kh;
            for (int kw = (int)q.KW - 1; kw >= 0; --kw) {
                const int ww = (int)w - kw * (int)q.dw;
                if (ww < 0) continue;
                const unsigned wo = fdiv((unsigned)ww, q.sw);
                if (wo * q.sw.d != (unsigned)ww || wo >= q.Wo) continue;
                acc += __ldg(in + rb + (long long)wo * q.in_wo + (long long)kw * q.in_kw);
            }
        }
        out[ob] = acc;
    }
}

int launch_fold_gather(Device* dev, const Plan& plan, const KParams& p) {
    const long long cap = (long long)dev->prop.multiProcessorCount * 16;
    if (plan.out_numel > 0) {
        long long blocks = (plan.out_numel + 255) / 256;
        if (blocks > cap) blocks = cap;
        fill_zero_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(reinterpret_cast<float*>(p.out.ptr), plan.out_numel);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
    }
    if (p.total <= 0) return EB200_OK;
    const int nk = p.ndim;
    FoldParams q{};
    q.n_outer = nk - 4;
    long long outer = 1;
    for (int j = 0; j < nk - 4; ++j) {
        q.oshape[j] = make_fastdiv((unsigned)p.shape[j]);
        q.o_in[j] = p.in[0].strides[j];
        q.o_out[j] = p.out.strides[j];
        outer *= p.shape[j];
    }
    q.Ho = (unsigned)p.shape[nk - 4]; q.Wo = (unsigned)p.shape[nk - 3]; q.KH = (unsigned)p.shape[nk - 2]; q.KW = (unsigned)p.shape[nk - 1];
    q.in_ho = p.in[0].strides[nk - 4]; q.in_wo = p.in[0].strides[nk - 3]; q.in_kh = p.in[0].strides[nk - 2]; q.in_kw = p.in[0].strides[nk - 1];
    q.sh = make_fastdiv((unsigned)plan.fold_sh); q.sw = make_fastdiv((unsigned)plan.fold_sw); q.dh = (unsigned)plan.fold_dh; q.dw = (unsigned)plan.fold_dw;
    q.hout = make_fastdiv((unsigned)plan.fold_hout); q.wout = make_fastdiv((unsigned)plan.fold_wout);
    q.pitch = plan.fold_pitch;
    q.in_off = p.in[0].offset; q.out_off = p.out.offset;
    q.total = (unsigned)(outer * plan.fold_hout * plan.fold_wout);
    long long blocks = ((long long)q.total + 255) / 256;
    const long long cap2 = (long long)dev->prop.multiProcessorCount * 32;
    if (blocks > cap2) blocks = cap2;
    fold_gather_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(q, reinterpret_cast<const float*>(p.in[0].ptr), reinterpret_cast<float*>(p.out.ptr));
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

// ---- SGD ------------------------------------------------------------------------------
// `out` may be `p` itself (the update runs in place), so neither is __restrict__
// and p is read with plain loads.
__global__ void __launch_bounds__(256) sgd_kernel(const float* p, const float* __restrict__ g,
                                                  float* out, long long n, float lr) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const long long nvec = aligned ? (n >> 2) : 0;
    for (long long v = tid; v < nvec; v += stride) {
        const float4 a = reinterpret_cast<const float4*>(p)[v];
        const float4 b = __ldg(reinterpret_cast<const float4*>(g) + v);
        float4 r;
        r.x = __fsub_rn(a.x, __fmul_rn(lr, b.x));
        r.y = __fsub_rn(a.y, __fmul_rn(lr, b.y));
        r.z = __fsub_rn(a.z, __fmul_rn(lr, b.z));
        r.w = __fsub_rn(a.w, __fmul_rn(lr, b.w));
        reinterpret_cast<float4*>(out)[v] = r;
    }
    for (long long i = (nvec << 2) + tid; i < n; i += stride) out[i] = __fsub_rn(p[i], __fmul_rn(lr, g[i]));
}

int launch_sgd(Device* dev, const Plan& plan, const float* p, const float* g, float* out, long long n) {
    if (n <= 0) return EB200_OK;
    long long blocks = (n / 4 + 255) / 256 + 1;
    const long long cap = (long long)dev->prop.multiProcessorCount * 16;
    if (blocks > cap) blocks = cap;
    sgd_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(p, g, out, n, plan.scalar);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

}  // namespace eb200
