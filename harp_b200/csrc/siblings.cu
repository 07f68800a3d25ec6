// Sibling fusion: three roots of one realize that read the same [R, C] tensor, in ONE pass.
//
// eclat lowers every surviving graph node to a kernel of its own (src/lowerer/lower.rs:335-388),
// so a graph with the roots
//     y = sum(map(x, ...), axis 1)    (R_, reduce dim innermost)
//     z = max(x, axis 0)              (R_, reduce dim strided)
//     t = x.permute(1, 0).contiguous()  (E_ over the permuted view)
// reads x three times.  When the three are realized together the loads can be shared: every CTA
// takes 64 x 64 tiles of x (128-bit loads, two tiles in flight in registers), and from the one
// copy in registers it
//   * adds map(x) along its 64 columns   -> one partial per row and tile column,
//   * takes the maximum down its 64 rows -> one partial per column and tile row,
//   * writes the tile transposed through odd-pitch shared memory (128-bit stores).
// A second kernel folds the partials in tile order (deterministic).  Algorithmic traffic: x once
// in, t once out (8 B per element) instead of 16 B for the three separate kernels; the partials
// add 16 B per 64 elements.  HBM-bound.
#include <algorithm>

#include "expr.cuh"

namespace eb200 {

struct SibParams {
    long long R, C;            // x is [R][C], contiguous along C
    long long tiles_r, tiles_c, tiles;
    float* y_part;             // [tiles_c][R]
    float* z_part;             // [tiles_r][C]
    float* y; float* z; float* t;     // outputs: y [R], z [C], t [C][R]
};

template <class F>
__global__ void __launch_bounds__(256) siblings_kernel(const __grid_constant__ KParams p, const __grid_constant__ SibParams q,
                                                       const float* __restrict__ x) {
    constexpr int TT = 64, P = TT + 1;
    constexpr int NI = F::kCompiled ? F::kNin : KMAX_IN;
    __shared__ float tile_mem[TT * P];
    __shared__ float row_half[2][TT];          // [column half][row of the tile]
    __shared__ float col_quarter[4][TT];       // [warp pair][column of the tile]
    float cl[F::kNconst];
    load_consts<F>(p, cl);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tx = lane & 7, ty = lane >> 3;
    const int seg = (warp & 1) * 32;           // which half of the tile's columns this warp holds
    const int line0 = (warp >> 1) * 4 + ty;    // row of the tile (plus 16 per pass)
    const int n = F::nin(p);
    auto base_of = [&](long long t_, long long& r0, long long& c0) {
        c0 = (t_ % q.tiles_c) * TT;
        r0 = (t_ / q.tiles_c) * TT;
    };
    constexpr int DEPTH = 2;
    float4 nxt[DEPTH][4];
    const long long step = gridDim.x;
#pragma unroll
    for (int dpt = 0; dpt < DEPTH; ++dpt) {
        const long long tt = (long long)blockIdx.x + dpt * step;
        if (tt < q.tiles) {
            long long r0, c0;
            base_of(tt, r0, c0);
#pragma unroll
            for (int pass = 0; pass < 4; ++pass)
                nxt[dpt][pass] = __ldg(reinterpret_cast<const float4*>(x + (r0 + pass * 16 + line0) * q.C + c0 + seg + tx * 4));
        }
    }
    for (long long t_ = blockIdx.x; t_ < q.tiles; t_ += step) {
        long long r0, c0;
        base_of(t_, r0, c0);
        float cmax[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const float4 v = nxt[0][pass];
            const int rl = pass * 16 + line0, cc = seg + tx * 4;
            // transposed staging: t[c][r] = x[r][c]
            tile_mem[cc * P + rl] = v.x; tile_mem[(cc + 1) * P + rl] = v.y;
            tile_mem[(cc + 2) * P + rl] = v.z; tile_mem[(cc + 3) * P + rl] = v.w;
            cmax[0] = fmaxf(cmax[0], v.x); cmax[1] = fmaxf(cmax[1], v.y);
            cmax[2] = fmaxf(cmax[2], v.z); cmax[3] = fmaxf(cmax[3], v.w);
            // the row map on this thread's four columns; operand 0 of the (renumbered) map is x,
            // every other operand reached the kernel as a launch-time constant
            float in[NI][4], m4[4];
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (i >= n) break;
                in[i][0] = v.x; in[i][1] = v.y; in[i][2] = v.z; in[i][3] = v.w;
            }
            F::template eval<4>(p, in, m4, cl);
            float rs = (m4[0] + m4[1]) + (m4[2] + m4[3]);
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            rs += __shfl_xor_sync(0xffffffffu, rs, 4);
            if (tx == 0) row_half[warp & 1][rl] = rs;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            cmax[j] = fmaxf(cmax[j], __shfl_xor_sync(0xffffffffu, cmax[j], 8));
            cmax[j] = fmaxf(cmax[j], __shfl_xor_sync(0xffffffffu, cmax[j], 16));
        }
        if (ty == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) col_quarter[warp >> 1][seg + tx * 4 + j] = cmax[j];
        }
        __syncthreads();
        // shift the queue and refill its tail
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) nxt[0][pass] = nxt[1][pass];
        const long long tn = t_ + DEPTH * step;
        if (tn < q.tiles) {
            long long rn, cn;
            base_of(tn, rn, cn);
#pragma unroll
            for (int pass = 0; pass < 4; ++pass)
                nxt[1][pass] = __ldg(reinterpret_cast<const float4*>(x + (rn + pass * 16 + line0) * q.C + cn + seg + tx * 4));
        }
        // partials of this tile
        if (threadIdx.x < TT) {
            const int i = threadIdx.x;
            q.y_part[(t_ % q.tiles_c) * q.R + r0 + i] = row_half[0][i] + row_half[1][i];
        } else if (threadIdx.x < 2 * TT) {
            const int i = threadIdx.x - TT;
            q.z_part[(t_ / q.tiles_c) * q.C + c0 + i] =
                fmaxf(fmaxf(col_quarter[0][i], col_quarter[1][i]), fmaxf(col_quarter[2][i], col_quarter[3][i]));
        }
        // transposed tile out: row cl of t (a column of x), 64 consecutive rows of x
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int cl_ = pass * 16 + line0, rl = seg + tx * 4;
            const float* src = tile_mem + cl_ * P + rl;
            *reinterpret_cast<float4*>(q.t + (c0 + cl_) * q.R + r0 + rl) = make_float4(src[0], src[1], src[2], src[3]);
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) siblings_finish_kernel(const __grid_constant__ SibParams q) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < q.R + q.C; i += stride) {
        if (i < q.R) {
            float acc = 0.0f;
            for (long long tc = 0; tc < q.tiles_c; ++tc) acc += q.y_part[tc * q.R + i];
            q.y[i] = acc;
        } else {
            const long long c = i - q.R;
            float acc = -INFINITY;
            for (long long tr = 0; tr < q.tiles_r; ++tr) acc = fmaxf(acc, q.z_part[tr * q.C + c]);
            q.z[c] = acc;
        }
    }
}

long long siblings_scratch_floats(long long R, long long C) { return (C / 64) * R + (R / 64) * C; }

template <class F>
static int launch_siblings_one(Device* dev, const KParams& p, const SibParams& q, const float* x) {
    // persistent CTAs: exactly as many as are resident at once (a second wave would start only when
    // first-wave CTAs have finished their whole share of the tiles)
    int per_sm = 0;
    EB_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, siblings_kernel<F>, 256, 0));
    const long long blocks = std::min<long long>(q.tiles, (long long)dev->prop.multiProcessorCount * std::max(1, per_sm));
    siblings_kernel<F><<<(unsigned)blocks, 256, 0, dev->stream>>>(p, q, x);
    count_launch();
    long long fb = std::min<long long>((q.R + q.C + 255) / 256, (long long)dev->prop.multiProcessorCount * 8);
    siblings_finish_kernel<<<(unsigned)fb, 256, 0, dev->stream>>>(q);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

// p: the plan parameters of the row reduce (its map, constants); x: the full-size operand;
// out: [y (R, padded to 64) | z (C, padded to 64) | t (C * R)]
int launch_siblings(Device* dev, const Plan& plan, const KParams& p, const float* x, float* out, void* scratch) {
    EB_REQUIRE(scratch, EB200_ERR_INVALID, "sibling fusion launched without scratch");
    SibParams q{};
    q.R = plan.sib_rows; q.C = plan.sib_cols;
    q.tiles_r = q.R / 64; q.tiles_c = q.C / 64; q.tiles = q.tiles_r * q.tiles_c;
    q.y_part = reinterpret_cast<float*>(scratch);
    q.z_part = q.y_part + q.tiles_c * q.R;
    q.y = out;
    q.z = out + (q.R + 63) / 64 * 64;
    q.t = q.z + (q.C + 63) / 64 * 64;
    EB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q.t) & 15) == 0, EB200_ERR_INVALID,
               "sibling fusion needs 16-byte aligned buffers");
    switch (plan.chain) {
#define X(i) case i: return launch_siblings_one<Compiled<Chain##i>>(dev, p, q, x);
        EB_FOR_EACH_CHAIN(X)
#undef X
        default: return launch_siblings_one<Interp>(dev, p, q, x);
    }
}

}  // namespace eb200
