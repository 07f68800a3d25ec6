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
#include <string.h>

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
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = red_combine(rop, v, __shfl_xor_sync(0xffffffffu, v, o));
    if (T == 32) return v;
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

constexpr int RO_U = 4;  // reduce steps in flight per thread

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

template <class F>
static int launch_one(Device* dev, const Plan& plan, const KParams& p, float* scratch) {
    const int sms = dev->prop.multiProcessorCount;
    if (p.kept <= 0) return EB200_OK;
    if (plan.impl == IMPL_REDUCE_INNER) {
        const int T = plan.threads_per_row;
        const long long work = p.kept * p.splits;
        const long long rows = 256 / T;
        long long blocks = (work + rows - 1) / rows;
        long long cap = (long long)sms * 64;
        if (blocks > cap) blocks = cap;
        if (T == 1) reduce_inner_kernel<F, 1><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        else if (T == 32) reduce_inner_kernel<F, 32><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        else if (T == 128) reduce_inner_kernel<F, 128><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        else reduce_inner_kernel<F, 256><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
    } else {
        const long long nwork = p.vec == 4 ? (p.kept >> 2) : p.kept;
        long long bx = (nwork + 255) / 256;
        long long cap = (long long)sms * 32;
        if (bx > cap) bx = cap;
        dim3 grid((unsigned)bx, (unsigned)p.splits);
        reduce_outer_kernel<F><<<grid, 256, 0, dev->stream>>>(p, scratch);
    }
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    if (p.splits > 1) {
        long long blocks = (p.kept + 255) / 256;
        long long cap = (long long)sms * 8;
        if (blocks > cap) blocks = cap;
        reduce_finish_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(p, scratch);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
    }
    return EB200_OK;
}

int launch_reduce(Device* dev, const Plan& plan, const KParams& p, void* scratch) {
    float* s = reinterpret_cast<float*>(scratch);
    EB_REQUIRE(p.splits == 1 || s, EB200_ERR_INVALID, "split reduction launched without scratch");
    switch (plan.chain) {
#define X(i) case i: return launch_one<Compiled<Chain##i>>(dev, plan, p, s);
        EB_FOR_EACH_CHAIN(X)
#undef X
        default: return launch_one<Interp>(dev, plan, p, s);
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
