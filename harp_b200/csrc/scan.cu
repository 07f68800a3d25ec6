// Cumulative (scan) kernels, class P_ (src/lowerer/lower.rs:691-735).
//
// The reference's loop nest (src/lowerer/loop_gen.rs:237-327) declares ONE
// accumulator per index of the dims before the scan axis and then walks the
// scan axis AND every dim after it, storing the accumulator at each position:
//
//     for outer...: acc = identity
//         for s in axis: for inner...: acc = op(acc, map(loads)); out[...] = acc
//
// so a "row" of the scan is the row-major sequence over (axis, inner dims); with
// the axis innermost this is the ordinary cumsum / cumprod / cummax.  That
// sequence semantics is what is served here:
//
//  scan_rows    many rows: a warp (rows up to 1024 elements) or a 256-thread CTA
//               per row walks it in chunks of 16 elements per thread: thread-local
//               scan, warp shuffle scan, cross-warp offsets through shared
//               memory, a running carry between chunks.  8 B per element
//               (one read, one write): HBM-bound.
//  scan_tiles   few long rows: every row is cut into tiles of 8192 elements; a
//               first kernel reduces each tile to one total, a second kernel
//               folds the totals before its tile and scans the tile with that
//               prefix.  12 B per element (the input is read twice), no
//               device-side waiting between CTAs, results independent of the
//               launch configuration.
//
// Sums are reassociated (tree order inside a chunk), like every parallel sum
// here; max / min are exact.
#include <algorithm>

#include "expr.cuh"
#include "index.cuh"

namespace eb200 {

constexpr int SCAN_TILE = 8192;     // elements per tile of the two-pass form

// The scan op as a template parameter (ROP >= 0: the plain cumsum / cummax / cummin / cumprod of one
// operand, the common case) or read from the parameters (ROP < 0: every fused-map chain).  With the op
// known at compile time the shuffle scan is a third of the instructions: the kernels are issue bound.
template <int ROP> __device__ __forceinline__ float scan_comb(int rop, float a, float b) { return Red<ROP>::combine(a, b); }
template <> __device__ __forceinline__ float scan_comb<-1>(int rop, float a, float b) { return red_combine(rop, a, b); }
template <int ROP> __device__ __forceinline__ float scan_ident(int rop) { return Red<ROP>::identity(); }
template <> __device__ __forceinline__ float scan_ident<-1>(int rop) { return red_identity(rop); }

// One element of the row: map over the loads at linear index e (through the
// operands' views, masked loads included).
template <class F>
__device__ __forceinline__ float scan_elem(const KParams& p, long long e, const float* cl) {
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    const int n = F::nin(p);
    long long idx[KMAX_DIMS];
    decompose(p, e, idx);
    float in[NI][1], v[1];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        if (i >= n) break;
        const KOperand& o = p.in[i];
        if (o.n_bounds && !bounds_ok(p, o, idx)) in[i][0] = o.pad;
        else in[i][0] = load_elem(o, operand_index(p, o, idx));
    }
    F::template eval<1>(p, in, v, cl);
    return v[0];
}

// Four consecutive elements of a row whose operands are unit-stride (or
// broadcast) along the flattened tail: 128-bit loads.
template <class F>
__device__ __forceinline__ void scan_vec4(const KParams& p, const long long* ridx, long long pos, const float* cl, float* x) {
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    const int n = F::nin(p);
    const int ra = p.raxis;
    float in[NI][4];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        if (i >= n) break;
        const float* b = reinterpret_cast<const float*>(p.in[i].ptr) + operand_index(p, p.in[i], ridx);
        if (p.in[i].strides[ra] == 1) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(b + pos));
            in[i][0] = t.x; in[i][1] = t.y; in[i][2] = t.z; in[i][3] = t.w;
        } else {
            const float t = __ldg(b);
            in[i][0] = t; in[i][1] = t; in[i][2] = t; in[i][3] = t;
        }
    }
    F::template eval<4>(p, in, x, cl);
}

// Scans positions [pos0, pos1) of `row` with a group of T threads (a warp or the
// whole 256-thread CTA), starting from `carry`; returns the carry after pos1.
// `store` false only accumulates (the tile-total pass).
template <class F, int T, bool STORE, int ROP>
__device__ __forceinline__ float scan_segment(const KParams& p, const float* cl, long long row, long long pos0, long long pos1,
                                              float carry, float* smem) {
    const int rop = p.rop;
    const int lane = threadIdx.x % T;
    const int wlane = threadIdx.x & 31;
    const float ident = scan_ident<ROP>(rop);
    long long ridx[KMAX_DIMS];
    if (p.vec == 4) {
        decompose(p, row * p.rlen, ridx);          // index of the row's first element; the tail dim is 0
    }
    // SV vectors of four consecutive elements per thread and chunk: one thread-local scan of 4 * SV elements, ONE
    // shuffle scan and one pair of block barriers per chunk (the kernels are bound by their instruction stream),
    // SV independent 128-bit loads in flight
    constexpr int SV = 4, PER = 4 * SV;
    for (long long chunk = pos0; chunk < pos1; chunk += (long long)T * PER) {
        const long long my = chunk + (long long)lane * PER;
        float x[PER];
        if (p.vec == 4) {
#pragma unroll
            for (int v = 0; v < SV; ++v) {
                if (my + 4 * v < pos1) scan_vec4<F>(p, ridx, my + 4 * v, cl, x + 4 * v);          // rlen and tile bounds are multiples of 4
                else { x[4 * v] = ident; x[4 * v + 1] = ident; x[4 * v + 2] = ident; x[4 * v + 3] = ident; }
            }
        } else {
#pragma unroll
            for (int j = 0; j < PER; ++j) x[j] = my + j < pos1 ? scan_elem<F>(p, row * p.rlen + my + j, cl) : ident;
        }
#pragma unroll
        for (int j = 1; j < PER; ++j) x[j] = scan_comb<ROP>(rop, x[j - 1], x[j]);
        // inclusive scan of the thread totals across the warp
        float incl = x[PER - 1];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, incl, o);
            if (wlane >= o) incl = scan_comb<ROP>(rop, t, incl);
        }
        float excl = __shfl_up_sync(0xffffffffu, incl, 1);
        if (wlane == 0) excl = ident;
        float total;                                  // of the whole chunk
        if (T == 32) {
            total = __shfl_sync(0xffffffffu, incl, 31);
        } else {
            const int warp = threadIdx.x >> 5;
            if (wlane == 31) smem[warp] = incl;
            __syncthreads();
            float before = ident;
            total = ident;
#pragma unroll
            for (int w = 0; w < T / 32; ++w) {
                const float t = smem[w];
                if (w < warp) before = scan_comb<ROP>(rop, before, t);
                total = scan_comb<ROP>(rop, total, t);
            }
            __syncthreads();
            excl = scan_comb<ROP>(rop, before, excl);
        }
        if (STORE && my < pos1) {
            const float base = scan_comb<ROP>(rop, carry, excl);
            if (p.vec == 4) {
                float* o = reinterpret_cast<float*>(p.out.ptr) + operand_index(p, p.out, ridx) + my;
#pragma unroll
                for (int v = 0; v < SV; ++v) {
                    if (my + 4 * v < pos1)
                        *reinterpret_cast<float4*>(o + 4 * v) =
                            make_float4(scan_comb<ROP>(rop, base, x[4 * v]), scan_comb<ROP>(rop, base, x[4 * v + 1]),
                                        scan_comb<ROP>(rop, base, x[4 * v + 2]), scan_comb<ROP>(rop, base, x[4 * v + 3]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    if (my + j >= pos1) break;
                    long long idx[KMAX_DIMS];
                    decompose(p, row * p.rlen + my + j, idx);
                    store_elem(p.out, operand_index(p, p.out, idx), scan_comb<ROP>(rop, base, x[j]));
                }
            }
        }
        carry = scan_comb<ROP>(rop, carry, total);
    }
    return carry;
}

template <class F, int T, int ROP>
__global__ void __launch_bounds__(256) scan_rows_kernel(const __grid_constant__ KParams p) {
    __shared__ float smem[8];
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    constexpr int ROWS = 256 / T;
    const int sub = threadIdx.x / T;
    const long long nblk = (p.kept + ROWS - 1) / ROWS;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
        const long long row = blk * ROWS + sub;
        // T == 256: the whole CTA walks one row (barriers inside are uniform); T == 32: a warp per row
        if (row < p.kept) scan_segment<F, T, true, ROP>(p, cl, row, 0, p.rlen, scan_ident<ROP>(p.rop), smem);
    }
}

// grid = (tiles, rows): total of every tile
template <class F, int ROP>
__global__ void __launch_bounds__(256) scan_tile_total_kernel(const __grid_constant__ KParams p, float* __restrict__ totals, int tiles) {
    __shared__ float smem[8];
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    const long long row = blockIdx.y;
    const long long pos0 = (long long)blockIdx.x * SCAN_TILE;
    const long long pos1 = min(pos0 + SCAN_TILE, p.rlen);
    const float t = scan_segment<F, 256, false, ROP>(p, cl, row, pos0, pos1, scan_ident<ROP>(p.rop), smem);
    if (threadIdx.x == 0) totals[row * tiles + blockIdx.x] = t;
}

// grid = (tiles, rows): fold the totals of the tiles before this one (in tile
// order, so every CTA of a row sees the same prefixes), then scan the tile
template <class F, int ROP>
__global__ void __launch_bounds__(256) scan_tile_apply_kernel(const __grid_constant__ KParams p, const float* __restrict__ totals, int tiles) {
    __shared__ float smem[8];
    __shared__ float prefix_s;
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    const long long row = blockIdx.y;
    if (threadIdx.x < 32) {
        // a warp folds the earlier totals: lane l takes a contiguous slice, slices combine in lane order
        const int n = blockIdx.x, per = (n + 31) / 32;
        float acc = red_identity(p.rop);
        for (int i = threadIdx.x * per; i < min(n, (int)(threadIdx.x + 1) * per); ++i) acc = red_combine(p.rop, acc, totals[row * tiles + i]);
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, acc, o);
            if ((int)threadIdx.x >= o) acc = red_combine(p.rop, t, acc);
        }
        if (threadIdx.x == 31) prefix_s = acc;
    }
    __syncthreads();
    const long long pos0 = (long long)blockIdx.x * SCAN_TILE;
    const long long pos1 = min(pos0 + SCAN_TILE, p.rlen);
    scan_segment<F, 256, true, ROP>(p, cl, row, pos0, pos1, prefix_s, smem);
}

long long scan_scratch_floats(const KParams& p, int sms) {
    if (p.kept <= 0 || p.rlen <= 0) return 0;
    if (p.kept >= 2LL * sms || p.rlen < 4LL * SCAN_TILE) return 0;
    return p.kept * ((p.rlen + SCAN_TILE - 1) / SCAN_TILE);
}

template <class F, int ROP>
static int launch_scan_one(Device* dev, const Plan& plan, const KParams& p, float* scratch) {
    const int sms = dev->prop.multiProcessorCount;
    if (p.kept <= 0 || p.rlen <= 0) return EB200_OK;
    if (plan.scratch_bytes > 0) {
        EB_REQUIRE(scratch, EB200_ERR_INVALID, "tiled scan launched without scratch");
        const int tiles = (int)((p.rlen + SCAN_TILE - 1) / SCAN_TILE);
        EB_REQUIRE(p.kept <= 65535, EB200_ERR_UNSUPPORTED, "tiled scan over %lld rows", p.kept);
        dim3 grid((unsigned)tiles, (unsigned)p.kept);
        scan_tile_total_kernel<F, ROP><<<grid, 256, 0, dev->stream>>>(p, scratch, tiles);
        count_launch();
        scan_tile_apply_kernel<F, ROP><<<grid, 256, 0, dev->stream>>>(p, scratch, tiles);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
        return EB200_OK;
    }
    const bool warp_rows = p.rlen <= 1024;
    const long long rows_per = warp_rows ? 8 : 1;
    long long blocks = (p.kept + rows_per - 1) / rows_per;
    blocks = std::min<long long>(blocks, (long long)sms * 8);
    if (warp_rows) scan_rows_kernel<F, 32, ROP><<<(unsigned)blocks, 256, 0, dev->stream>>>(p);
    else scan_rows_kernel<F, 256, ROP><<<(unsigned)blocks, 256, 0, dev->stream>>>(p);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

int launch_scan(Device* dev, const Plan& plan, const KParams& p, void* scratch) {
    float* s = reinterpret_cast<float*>(scratch);
    if (plan.chain == 0) {          // the identity map: the scan op is a template parameter
        switch (p.rop) {
            case EB200_R_SUM: return launch_scan_one<Compiled<Chain0>, EB200_R_SUM>(dev, plan, p, s);
            case EB200_R_MAX: return launch_scan_one<Compiled<Chain0>, EB200_R_MAX>(dev, plan, p, s);
            case EB200_R_MIN: return launch_scan_one<Compiled<Chain0>, EB200_R_MIN>(dev, plan, p, s);
            default: return launch_scan_one<Compiled<Chain0>, EB200_R_PROD>(dev, plan, p, s);
        }
    }
    switch (plan.chain) {
#define X(i) case i: return launch_scan_one<Compiled<Chain##i>, -1>(dev, plan, p, s);
        EB_FOR_EACH_CHAIN(X)
#undef X
        default: return launch_scan_one<Interp, -1>(dev, plan, p, s);
    }
}

}  // namespace eb200
