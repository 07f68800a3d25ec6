// Axis reductions with a fused pre-map (kernel class R_,
// src/lowerer/lower.rs:525-571; loop shape src/lowerer/loop_gen.rs:87-151;
// identities and combiners src/graph/node.rs:29-77).
//
// The reference runs `acc = op(acc, map(loads))` sequentially, reduce loop
// innermost.  Two kernels replace it:
//
//  reduce_inner  the reduce dim is the innermost collapsed dim (contiguous
//                rows).  A group of T threads (1, a warp, or a 256-thread CTA)
//                walks one row with 128-bit loads, four in flight per thread,
//                evaluates the map, and combines through warp shuffles and a
//                shared-memory tree.  Operands that do not move along the row
//                (stride 0) are read once per row.  Few very long rows are
//                split over several CTAs into scratch partials and finished by
//                reduce_finish.
//  reduce_outer  the reduce dim is strided (e.g. max over axis 0): each thread
//                owns 4 adjacent kept elements, so a warp reads 512 contiguous
//                bytes per reduce step; the reduce dim is split over
//                gridDim.y into scratch partials [split][kept] which
//                reduce_finish folds.  With one split it is also the generic
//                fallback for any reduce the other paths do not take.
//
// Both are HBM-bound: algorithmic bytes = 4 B x (input elements + outputs).
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "expr.cuh"
#include "index.cuh"

namespace eb200 {

#ifndef EB_RI_U1
#define EB_RI_U1 4
#endif

// idx[d] = v without dynamic register indexing
__device__ __forceinline__ void set_idx(long long* idx, int d, long long v) {
#pragma unroll
    for (int i = 0; i < KMAX_DIMS; ++i)
        if (i == d) idx[i] = v;
}

template <int T>
__device__ __forceinline__ float group_reduce(float v, int rop, float* smem) {
    if (T == 1) return v;
    // T < 32: several row groups share a warp, the exchange stays inside each group of T lanes
#pragma unroll
    for (int o = (T < 32 ? T : 32) / 2; o > 0; o >>= 1) v = red_combine(rop, v, __shfl_xor_sync(0xffffffffu, v, o));
    if (T <= 32) return v;
    // T is 128 or 256: the 256-thread CTA holds 256/T row groups of T/32 warps
    constexpr int WPG = T >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    const int g0 = (warp / WPG) * WPG;   // first warp of this thread's group
    float r = red_identity(rop);
#pragma unroll
    for (int w = 0; w < WPG; ++w) r = red_combine(rop, r, smem[g0 + w]);
    __syncthreads();
    return r;
}

__device__ __forceinline__ void ldg4(const float* src, float* dst) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(src));
    dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
}

__device__ __forceinline__ void splat4(float v, float* dst) { dst[0] = v; dst[1] = v; dst[2] = v; dst[3] = v; }


template <class F, int T>
__global__ void __launch_bounds__(256) reduce_inner_kernel(const __grid_constant__ KParams p, float* __restrict__ scratch) {
    __shared__ float smem[8];
    constexpr int ROWS = 256 / T;
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    // independent 128-bit loads in flight per thread and operand
    constexpr int RI_U = (F::kCompiled && NI == 1) ? EB_RI_U1 : 4;
    const int lane = threadIdx.x % T;
    const int sub = threadIdx.x / T;
    const int ra = p.raxis;
    const int n = F::nin(p);
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    const long long work = p.kept * p.splits;  // (row, split) pairs
    const long long nblk = (work + ROWS - 1) / ROWS;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
        const long long item = blk * ROWS + sub;
        const bool live = item < work;
        const long long row = live ? item / p.splits : 0;
        const int split = live ? (int)(item - row * p.splits) : 0;
        long long idx[KMAX_DIMS];
        decompose(p, row, idx, ra);
        const long long r0 = (long long)split * p.chunk;
        long long r1 = r0 + p.chunk;
        if (r1 > p.rlen) r1 = p.rlen;
        float acc = red_identity(p.rop);
        if (live) {
            if (p.vec == 4) {
                // per row: a pointer for operands that walk the row, a value for those that do not
                const float* rp[NI];
                float rc[NI];
                bool moves[NI];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    if (i >= n) break;
                    const float* b = reinterpret_cast<const float*>(p.in[i].ptr) + operand_index(p, p.in[i], idx);
                    moves[i] = p.in[i].strides[ra] == 1;
                    rp[i] = b;
                    rc[i] = moves[i] ? 0.0f : __ldg(b);
                }
                float a4[4];
#pragma unroll
                for (int v = 0; v < 4; ++v) a4[v] = acc;
                const long long step = (long long)T * 4;
                long long c = r0 + lane * 4;
                for (; c + (RI_U - 1) * step < r1; c += RI_U * step) {
                    float in[RI_U][NI][4];
#pragma unroll
                    for (int u = 0; u < RI_U; ++u) {
#pragma unroll
                        for (int i = 0; i < NI; ++i) {
                            if (i >= n) break;
                            if (moves[i]) ldg4(rp[i] + c + u * step, in[u][i]);
                            else splat4(rc[i], in[u][i]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < RI_U; ++u) {
                        float v4[4];
                        F::template eval<4>(p, in[u], v4, cl);
#pragma unroll
                        for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], v4[v]);
                    }
                }
                for (; c < r1; c += step) {
                    float in[NI][4], v4[4];
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        if (i >= n) break;
                        if (moves[i]) ldg4(rp[i] + c, in[i]);
                        else splat4(rc[i], in[i]);
                    }
                    F::template eval<4>(p, in, v4, cl);
#pragma unroll
                    for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], v4[v]);
                }
                acc = red_combine(p.rop, red_combine(p.rop, a4[0], a4[1]), red_combine(p.rop, a4[2], a4[3]));
            } else {
                for (long long c = r0 + lane; c < r1; c += T) {
                    set_idx(idx, ra, c);
                    float in[NI][1], v[1];
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        if (i >= n) break;
                        const KOperand& o = p.in[i];
                        if (o.n_bounds && !bounds_ok(p, o, idx)) in[i][0] = o.pad;
                        else in[i][0] = load_elem(o, operand_index(p, o, idx));
                    }
                    F::template eval<1>(p, in, v, cl);
                    acc = red_combine(p.rop, acc, v[0]);
                }
                set_idx(idx, ra, 0);
            }
        }
        acc = group_reduce<T>(acc, p.rop, smem);
        if (live && lane == 0) {
            if (p.splits > 1) scratch[(long long)split * p.kept + row] = acc;
            else store_elem(p.out, operand_index(p, p.out, idx), acc);
        }
    }
}

// ---- row reduce with TMA staging -------------------------------------------------------
// For long contiguous rows with one streaming operand: every warp owns rows and a
// private 4-slot ring of 2 KB chunks in shared memory.  Lane 0 keeps the ring full
// with bulk async copies (cp.async.bulk, completion on an mbarrier per slot); the
// warp evaluates the map on a chunk as soon as it lands and refills the slot.
// 16 warps x 8 KB = 128 KB in flight per SM with no registers tied up in loads
// and no CTA-wide barrier anywhere.  Waits are bounded like the GEMM's.
constexpr int RT_WARPS = 32, RT_CH = 512, RT_ST = 3;   // warps per CTA, floats per chunk, slots per warp
constexpr unsigned RT_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t rt_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <class F>
__global__ void __launch_bounds__(RT_WARPS * 32, 1) reduce_inner_tma_kernel(const __grid_constant__ KParams p) {
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    extern __shared__ __align__(128) unsigned char rt_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* ring = reinterpret_cast<float*>(rt_raw) + (size_t)warp * RT_ST * RT_CH;
    uint64_t* bars = reinterpret_cast<uint64_t*>(rt_raw + (size_t)RT_WARPS * RT_ST * RT_CH * 4) + warp * RT_ST;
    const int ra = p.raxis;
    const int n = F::nin(p);
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    int mov = 0;                                   // the one operand that walks the row
#pragma unroll
    for (int i = 0; i < NI; ++i)
        if (i < n && p.in[i].strides[ra] == 1) mov = i;
    if (lane == 0) {
        for (int s = 0; s < RT_ST; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(rt_smem(&bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const long long wstride = (long long)gridDim.x * RT_WARPS;
    const long long first = (long long)blockIdx.x * RT_WARPS + warp;
    const int cpr = (int)((p.rlen + RT_CH - 1) / RT_CH);          // chunks per row
    // producer cursor (lane 0): next chunk to request
    long long prow = first;
    int pchunk = 0;
    const float* pbase = nullptr;
    unsigned issued = 0, consumed = 0;
    bool ok = true;
    auto issue = [&]() {                            // lane 0 only
        if (prow >= p.kept) return;
        if (pchunk == 0) {
            long long pidx[KMAX_DIMS];
            decompose(p, prow, pidx, ra);
            pbase = reinterpret_cast<const float*>(p.in[mov].ptr) + operand_index(p, p.in[mov], pidx);
        }
        const int s = issued % RT_ST;
        const long long c0 = (long long)pchunk * RT_CH;
        const unsigned bytes = (unsigned)(min((long long)RT_CH, p.rlen - c0) * 4);
        const uint32_t bar = rt_smem(&bars[s]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // our reads of this slot precede the copy
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(rt_smem(ring + (size_t)s * RT_CH)), "l"(pbase + c0), "r"(bytes), "r"(bar) : "memory");
        ++issued;
        if (++pchunk == cpr) { pchunk = 0; prow += wstride; }
    };
    if (lane == 0)
        for (int s = 0; s < RT_ST; ++s) issue();
    for (long long row = first; row < p.kept && ok; row += wstride) {
        long long idx[KMAX_DIMS];
        decompose(p, row, idx, ra);
        float rc[NI];                               // operands that do not move along the row: one value per row
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            if (i >= n) break;
            rc[i] = (i == mov) ? 0.0f : __ldg(reinterpret_cast<const float*>(p.in[i].ptr) + operand_index(p, p.in[i], idx));
        }
        float a4[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) a4[v] = red_identity(p.rop);
        for (int ch = 0; ch < cpr && ok; ++ch) {
            const int s = consumed % RT_ST;
            const unsigned parity = (consumed / RT_ST) & 1u;
            const uint32_t bar = rt_smem(&bars[s]);
            unsigned done = 0;
            for (unsigned spin = 0; spin < RT_SPIN_LIMIT && !done; ++spin) {
                asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                             : "=r"(done) : "r"(bar), "r"(parity) : "memory");
            }
            if (!done) {
                if (p.error_flag) atomicExch(p.error_flag, 1);
                ok = false;
                break;
            }
            const long long c0 = (long long)ch * RT_CH;
            const int len = (int)min((long long)RT_CH, p.rlen - c0);
            const float* src = ring + (size_t)s * RT_CH;
            // 512 floats = 4 vectors per lane, all evaluated together
            float in[4][NI][4];
            bool have[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = u * 128 + lane * 4;
                have[u] = e < len;
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    if (i >= n) break;
                    if (i == mov) {
                        const float4 t = have[u] ? *reinterpret_cast<const float4*>(src + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                        in[u][i][0] = t.x; in[u][i][1] = t.y; in[u][i][2] = t.z; in[u][i][3] = t.w;
                    } else {
                        splat4(rc[i], in[u][i]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (!have[u]) continue;
                float v4[4];
                F::template eval<4>(p, in[u], v4, cl);
#pragma unroll
                for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], v4[v]);
            }
            __syncwarp();                            // every lane has consumed its part of the slot
            ++consumed;
            if (lane == 0) issue();                  // refill it; three other slots are still in flight
        }
        float acc = red_combine(p.rop, red_combine(p.rop, a4[0], a4[1]), red_combine(p.rop, a4[2], a4[3]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc = red_combine(p.rop, acc, __shfl_xor_sync(0xffffffffu, acc, o));
        if (lane == 0 && ok) store_elem(p.out, operand_index(p, p.out, idx), acc);
    }
    // a warp that gave up still has copies in flight into its ring: wait for them (bounded)
    if (!ok && lane == 0) {
        for (unsigned c = consumed; c < issued; ++c) {
            const uint32_t bar = rt_smem(&bars[c % RT_ST]);
            unsigned done = 0;
            for (unsigned spin = 0; spin < RT_SPIN_LIMIT && !done; ++spin)
                asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                             : "=r"(done) : "r"(bar), "r"((c / RT_ST) & 1u) : "memory");
        }
    }
}

#ifndef EB_RO_U
#define EB_RO_U 4
#endif
constexpr int RO_U = EB_RO_U;  // reduce steps in flight per thread

template <class F>
__global__ void __launch_bounds__(256) reduce_outer_kernel(const __grid_constant__ KParams p, float* __restrict__ scratch) {
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    const int ra = p.raxis;
    const int n = F::nin(p);
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    const int split = blockIdx.y;
    const long long r0 = (long long)split * p.chunk;
    long long r1 = r0 + p.chunk;
    if (r1 > p.rlen) r1 = p.rlen;
    const long long nwork = p.vec == 4 ? (p.kept >> 2) : p.kept;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long wv = (long long)blockIdx.x * blockDim.x + threadIdx.x; wv < nwork; wv += stride) {
        const long long k = p.vec == 4 ? (wv << 2) : wv;
        long long idx[KMAX_DIMS];
        decompose(p, k, idx, ra);
        if (p.vec == 4) {
            const int inner = p.ndim - 1;
            // per thread: operands are a vector along the kept dim, or one value
            // broadcast over it; each may or may not move with the reduce index
            const float* bp[NI];
            long long rs[NI];
            bool isvec[NI];
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (i >= n) break;
                bp[i] = reinterpret_cast<const float*>(p.in[i].ptr) + operand_index(p, p.in[i], idx) + r0 * p.in[i].strides[ra];
                rs[i] = p.in[i].strides[ra];
                isvec[i] = p.in[i].strides[inner] == 1;
            }
            float a4[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) a4[v] = red_identity(p.rop);
            long long r = r0;
            for (; r + RO_U <= r1; r += RO_U) {
                float in[RO_U][NI][4];
#pragma unroll
                for (int u = 0; u < RO_U; ++u) {
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        if (i >= n) break;
                        if (isvec[i]) ldg4(bp[i], in[u][i]);
                        else splat4(__ldg(bp[i]), in[u][i]);
                        bp[i] += rs[i];
                    }
                }
#pragma unroll
                for (int u = 0; u < RO_U; ++u) {
                    float v4[4];
                    F::template eval<4>(p, in[u], v4, cl);
#pragma unroll
                    for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], v4[v]);
                }
            }
            for (; r < r1; ++r) {
                float in[NI][4], v4[4];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    if (i >= n) break;
                    if (isvec[i]) ldg4(bp[i], in[i]);
                    else splat4(__ldg(bp[i]), in[i]);
                    bp[i] += rs[i];
                }
                F::template eval<4>(p, in, v4, cl);
#pragma unroll
                for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], v4[v]);
            }
            const float4 res = make_float4(a4[0], a4[1], a4[2], a4[3]);
            if (p.splits > 1) *reinterpret_cast<float4*>(scratch + (long long)split * p.kept + k) = res;
            else *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out.ptr) + operand_index(p, p.out, idx)) = res;
        } else {
            float acc = red_identity(p.rop);
            for (long long r = r0; r < r1; ++r) {
                set_idx(idx, ra, r);
                float in[NI][1], v[1];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    if (i >= n) break;
                    const KOperand& o = p.in[i];
                    if (o.n_bounds && !bounds_ok(p, o, idx)) in[i][0] = o.pad;
                    else in[i][0] = load_elem(o, operand_index(p, o, idx));
                }
                F::template eval<1>(p, in, v, cl);
                acc = red_combine(p.rop, acc, v[0]);
            }
            set_idx(idx, ra, 0);
            if (p.splits > 1) scratch[(long long)split * p.kept + k] = acc;
            else store_elem(p.out, operand_index(p, p.out, idx), acc);
        }
    }
}

// The same reduce for NARROW outputs (at most 128 vectors of 4 kept elements, e.g. a bias
// gradient [rows, 32] -> [32]): with a thread per vector only a few threads of a CTA
// would work.  Here the CTA's 256 threads are (kept / 4) column threads x row lanes;
// a warp reads whole consecutive rows (coalesced), every lane folds the rows
// lane, lane + L, ... of the CTA's row chunk, and the lanes are combined through
// shared memory in lane order (deterministic).  Built for four CTAs per SM: the planner sizes the row split as
// one wave of 4 x SMs CTAs.
template <class F>
__global__ void __launch_bounds__(256, 4) reduce_outer_narrow_kernel(const __grid_constant__ KParams p, float* __restrict__ scratch) {
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    const int ra = p.raxis;
    const int n = F::nin(p);
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    __shared__ float part[256][4];
    const int nwork = (int)(p.kept >> 2);
    const int lanes = 256 / nwork;
    const int lane_r = threadIdx.x / nwork, tc = threadIdx.x - lane_r * nwork;
    const int split = blockIdx.y;
    const long long r0 = (long long)split * p.chunk;
    long long r1 = r0 + p.chunk;
    if (r1 > p.rlen) r1 = p.rlen;
    float a4[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) a4[v] = red_identity(p.rop);
    long long idx[KMAX_DIMS];
    decompose(p, (long long)tc << 2, idx, ra);
    if (lane_r < lanes) {
        const int inner = p.ndim - 1;
        const float* bp[NI];
        long long rs[NI];
        bool isvec[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            if (i >= n) break;
            rs[i] = p.in[i].strides[ra] * lanes;
            bp[i] = reinterpret_cast<const float*>(p.in[i].ptr) + operand_index(p, p.in[i], idx) + (r0 + lane_r) * p.in[i].strides[ra];
            isvec[i] = p.in[i].strides[inner] == 1;
        }
        long long r = r0 + lane_r;
        for (; r + (long long)(RO_U - 1) * lanes < r1; r += (long long)RO_U * lanes) {
            float in[RO_U][NI][4];
#pragma unroll
            for (int u = 0; u < RO_U; ++u) {
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    if (i >= n) break;
                    if (isvec[i]) ldg4(bp[i], in[u][i]);
                    else splat4(__ldg(bp[i]), in[u][i]);
                    bp[i] += rs[i];
                }
            }
#pragma unroll
            for (int u = 0; u < RO_U; ++u) {
                float v4[4];
                F::template eval<4>(p, in[u], v4, cl);
#pragma unroll
                for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], v4[v]);
            }
        }
        for (; r < r1; r += lanes) {
            float in[NI][4], v4[4];
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (i >= n) break;
                if (isvec[i]) ldg4(bp[i], in[i]);
                else splat4(__ldg(bp[i]), in[i]);
                bp[i] += rs[i];
            }
            F::template eval<4>(p, in, v4, cl);
#pragma unroll
            for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], v4[v]);
        }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) part[threadIdx.x][v] = a4[v];
    __syncthreads();
    if (lane_r == 0) {
        for (int l = 1; l < lanes; ++l)
#pragma unroll
            for (int v = 0; v < 4; ++v) a4[v] = red_combine(p.rop, a4[v], part[l * nwork + tc][v]);
        const float4 res = make_float4(a4[0], a4[1], a4[2], a4[3]);
        if (p.splits > 1) *reinterpret_cast<float4*>(scratch + (long long)split * p.kept + ((long long)tc << 2)) = res;
        else *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out.ptr) + operand_index(p, p.out, idx)) = res;
    }
}

// Folds scratch partials [splits][kept] into the output operand.
__global__ void __launch_bounds__(256) reduce_finish_kernel(const __grid_constant__ KParams p, const float* __restrict__ scratch) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < p.kept; k += stride) {
        float acc = red_identity(p.rop);
        for (int s = 0; s < p.splits; ++s) acc = red_combine(p.rop, acc, scratch[(long long)s * p.kept + k]);
        long long idx[KMAX_DIMS];
        decompose(p, k, idx, p.raxis);
        store_elem(p.out, operand_index(p, p.out, idx), acc);
    }
}

// The same fold for few kept elements and many splits (a bias gradient: 256 columns, ~600 row blocks): one thread
// per column would walk its partials alone, one dependent load after the other.  Here a CTA is 32 columns x 8
// split lanes: lane j folds splits j, j + 8, ... (in order), the eight partial results are folded in lane order
// through shared memory -- a fixed order, so the result does not depend on the launch.
__global__ void __launch_bounds__(256) reduce_finish_wide_kernel(const __grid_constant__ KParams p, const float* __restrict__ scratch) {
    __shared__ float part[8][33];
    const int col = threadIdx.x & 31, lane_s = threadIdx.x >> 5;
    for (long long k0 = (long long)blockIdx.x * 32; k0 < p.kept; k0 += (long long)gridDim.x * 32) {
        const long long k = k0 + col;
        float acc = red_identity(p.rop);
        if (k < p.kept) {
#pragma unroll 4
            for (int s = lane_s; s < p.splits; s += 8) acc = red_combine(p.rop, acc, __ldg(scratch + (long long)s * p.kept + k));
        }
        part[lane_s][col] = acc;
        __syncthreads();
        if (lane_s == 0 && k < p.kept) {
            float r = part[0][col];
#pragma unroll
            for (int j = 1; j < 8; ++j) r = red_combine(p.rop, r, part[j][col]);
            long long idx[KMAX_DIMS];
            decompose(p, k, idx, p.raxis);
            store_elem(p.out, operand_index(p, p.out, idx), r);
        }
        __syncthreads();
    }
}

template <class F>
static int launch_one(Device* dev, const Plan& plan, const KParams& p, float* scratch, bool finish) {
    const int sms = dev->prop.multiProcessorCount;
    if (p.kept <= 0) return EB200_OK;
    if (plan.impl == IMPL_REDUCE_INNER) {
        const int T = plan.threads_per_row;
        const long long work = p.kept * p.splits;
        const long long rows = 256 / T;
        long long blocks = (work + rows - 1) / rows;
        long long cap = (long long)sms * 64;
        if (blocks > cap) blocks = cap;
        int moving = 0;
        for (int i = 0; i < p.n_in; ++i) moving += p.in[i].strides[p.raxis] == 1;
        // Staging rows through shared memory with bulk async copies is opt-in
        // (descriptor flag 32): on B200 it measured 5.05 TB/s against 6.15 TB/s for
        // the direct 128-bit loads on [8192, 8192] rows.
        const bool tma = (p.tuning & 32) && T == 32 && p.vec == 4 && p.splits == 1 && moving == 1 && p.rlen >= 2048 &&
                         p.error_flag != nullptr && p.kept >= sms;
        if (tma) {
            const size_t smem = (size_t)RT_WARPS * RT_ST * RT_CH * 4 + RT_WARPS * RT_ST * 8;
            static unsigned long long configured_devices = 0;      // function attributes are per device
            const unsigned long long dev_bit = 1ULL << (dev->index & 63);
            if (!(configured_devices & dev_bit)) {
                EB_CHECK_CUDA(cudaFuncSetAttribute(reduce_inner_tma_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured_devices |= dev_bit;
            }
            long long g = std::min<long long>(sms, (p.kept + RT_WARPS - 1) / RT_WARPS);
            reduce_inner_tma_kernel<F><<<(unsigned)g, RT_WARPS * 32, smem, dev->stream>>>(p);
        } else
        if (T == 1) reduce_inner_kernel<F, 1><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        else if (T == 8) reduce_inner_kernel<F, 8><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        else if (T == 32) reduce_inner_kernel<F, 32><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        else if (T == 128) reduce_inner_kernel<F, 128><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        else reduce_inner_kernel<F, 256><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
    } else {
        const long long nwork = p.vec == 4 ? (p.kept >> 2) : p.kept;
        long long bx = (nwork + 255) / 256;
        long long cap = (long long)sms * 32;
        if (bx > cap) bx = cap;
        dim3 grid((unsigned)bx, (unsigned)p.splits);
        if (plan.narrow) reduce_outer_narrow_kernel<F><<<dim3(1, (unsigned)p.splits), 256, 0, dev->stream>>>(p, scratch);
        else reduce_outer_kernel<F><<<grid, 256, 0, dev->stream>>>(p, scratch);
    }
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    if (p.splits > 1 && finish) {
        long long blocks = (p.kept + 255) / 256;
        long long cap = (long long)sms * 8;
        if (blocks > cap) blocks = cap;
        if (p.splits >= 32 && p.kept <= 32LL * sms)
            reduce_finish_wide_kernel<<<(unsigned)((p.kept + 31) / 32), 256, 0, dev->stream>>>(p, scratch);
        else
            reduce_finish_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
    }
    return EB200_OK;
}

// `finish` false leaves the partials of a split reduction in scratch (the caller folds them,
// e.g. fused with an all-reduce).
int launch_reduce(Device* dev, const Plan& plan, const KParams& p, void* scratch, bool finish) {
    float* s = reinterpret_cast<float*>(scratch);
    EB_REQUIRE(p.splits == 1 || s, EB200_ERR_INVALID, "split reduction launched without scratch");
    switch (plan.chain) {
#define X(i) case i: return launch_one<Compiled<Chain##i>>(dev, plan, p, s, finish);
        EB_FOR_EACH_CHAIN(X)
#undef X
        default: return launch_one<Interp>(dev, plan, p, s, finish);
    }
}

}  // namespace eb200

// ---- column reduce without any allocation ------------------------------------------------
//
// eb200_reduce_cols_static serves callers that hold device memory but must not
// allocate any: code running where cudaMalloc is off limits because it
// synchronises the whole device (a latency-critical serving loop, a callback
// between captured graphs) or because all device memory already belongs to the
// caller's own arena.  Such callers cannot use eb200_kernel_create, whose split
// reductions take their partial-result scratch from the device pool.  Here the
// scratch is a fixed array inside the library image instead.
namespace eb200 {

constexpr long long kStaticScratchFloats = 1LL << 19;  // 2 MiB, resident on every device that loads the library
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

struct StaticDevice {
    bool ready = false;
    float* scratch = nullptr;   // device address of g_static_scratch on this device
    int sms = 0;
};
static StaticDevice g_static_dev[64];
static std::mutex g_static_mutex;

}  // namespace eb200

extern "C" int eb200_reduce_cols_static(const float* x, int64_t rows, int64_t cols, int reduce_op,
                                        float* out, void* stream) {
    using namespace eb200;
    EB_REQUIRE(x && out, EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(rows >= 1 && cols >= 1, EB200_ERR_INVALID, "rows and cols must be positive");
    EB_REQUIRE(reduce_op >= EB200_R_SUM && reduce_op <= EB200_R_PROD, EB200_ERR_INVALID, "reduce op %d", reduce_op);
    int devid = -1;
    EB_CHECK_CUDA(cudaGetDevice(&devid));
    EB_REQUIRE(devid >= 0 && devid < 64, EB200_ERR_UNSUPPORTED, "device ordinal %d out of range", devid);
    StaticDevice& sd = g_static_dev[devid];
    {
        // One-time set-up per device, with that device current.  The array's name
        // is only a host-side stand-in: kernels need the address the runtime
        // reports for this device.
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!sd.ready) {
            float* ptr = nullptr;
            EB_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch));
            EB_REQUIRE(ptr != nullptr, EB200_ERR_CUDA, "no device address for the static scratch array");
            int sms = 0;
            EB_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, devid));
            sd.scratch = ptr;
            sd.sms = sms;
            sd.ready = true;
        }
    }
    // the same descriptor eb200_kernel_create would get for max/sum over axis 0 of [rows, cols]
    eb200_kernel_desc d;
    memset(&d, 0, sizeof(d));
    d.kclass = EB200_K_REDUCE;
    d.ndim = 2;
    d.shape[0] = rows; d.shape[1] = cols;
    d.n_inputs = 1;
    d.reduce_op = reduce_op;
    d.reduce_axis = 0;
    d.inputs[0].dtype = EB200_F32; d.inputs[0].strides[0] = cols; d.inputs[0].strides[1] = 1; d.inputs[0].numel = rows * cols;
    d.output.dtype = EB200_F32; d.output.strides[0] = 0; d.output.strides[1] = 1; d.output.numel = cols;
    Plan plan;
    int st = build_plan(&d, sd.sms, &plan);
    if (st) return st;
    EB_REQUIRE(plan.impl == IMPL_REDUCE_INNER || plan.impl == IMPL_REDUCE_OUTER, EB200_ERR_UNSUPPORTED,
               "shape [%lld, %lld] is not served by a reduce kernel", (long long)rows, (long long)cols);
    EB_REQUIRE(plan.scratch_bytes <= kStaticScratchFloats * (long long)sizeof(float), EB200_ERR_UNSUPPORTED,
               "reduce of [%lld, %lld] needs %lld bytes of scratch; the static scratch holds %lld",
               (long long)rows, (long long)cols, (long long)plan.scratch_bytes,
               (long long)(kStaticScratchFloats * sizeof(float)));
    EB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               EB200_ERR_INVALID, "x and out must be 16-byte aligned");
    Device dev;
    dev.index = devid;
    dev.stream = reinterpret_cast<cudaStream_t>(stream);
    dev.prop.multiProcessorCount = sd.sms;
    KParams p = plan.p;
    p.in[0].ptr = reinterpret_cast<char*>(const_cast<float*>(x));
    p.out.ptr = reinterpret_cast<char*>(out);
    // every partial [split][column] is written by the first kernel before the
    // second reads it, so nothing in the scratch has to start at zero
    return launch_reduce(&dev, plan, p, sd.scratch);
}
