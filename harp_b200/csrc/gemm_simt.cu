// gemm_simt: dense contraction on the FP32 pipes.
//
// The reference has no f32 matmul op: `C = A.B` is spelled
// unsqueeze -> expand -> mul -> sum(axis=K) (crates/nn/src/functional/linear.rs:27-56,
// examples/matmul_demo.rs:43-60) and lowers to an R_ kernel whose body is
// `acc = acc + A[..] * B[..]` in a sequential triple loop.  The classifier
// recognises that pattern from operand strides (plan.cpp) and hands it here or
// to the tensor-core kernel.  This kernel keeps full f32 products and adds
// each output's terms in increasing k, like the reference loop, so it is the
// f32-faithful path for shapes or strides the tensor-core kernel does not take.
// 64x64 output tile per CTA, 16-deep k slices through shared memory, 4x4
// register micro-tile per thread; any A/B/C strides, batched over gridDim.z.
#include <algorithm>

#include "common.h"

namespace eb200 {

constexpr int GM = 64, GN = 64, GK = 16;

__global__ void __launch_bounds__(256) gemm_simt_kernel(const __grid_constant__ GemmShape g,
                                                        const float* __restrict__ A,
                                                        const float* __restrict__ B,
                                                        float* __restrict__ C) {
    __shared__ float As[GK][GM + 4];
    __shared__ float Bs[GK][GN + 4];
    const int t = threadIdx.x;
    const long long m0 = (long long)blockIdx.x * GM, n0 = (long long)blockIdx.y * GN;
    const long long bz = blockIdx.z / g.splits;
    const long long split = blockIdx.z % g.splits;
    const long long kbeg = split * g.k_chunk;
    const long long kend = g.splits > 1 ? min(g.k, kbeg + g.k_chunk) : g.k;
    const float* Ab = A + g.a_off + bz * g.a_sb;
    const float* Bb = B + g.b_off + bz * g.b_sb;
    // with split-K the CTA writes a dense [m][n] partial; the caller passes the partial buffer as C
    float* Cb = g.splits > 1 ? C + (long long)blockIdx.z * g.m * g.n : C + g.c_off + bz * g.c_sb;
    const long long c_sm = g.splits > 1 ? g.n : g.c_sm, c_sn = g.splits > 1 ? 1 : g.c_sn;
    const int ty = t >> 4, tx = t & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    const bool a_kfast = g.a_sk == 1;
    const bool b_nfast = g.b_sn == 1;
    for (long long k0 = kbeg; k0 < kend; k0 += GK) {
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            int m, k;
            if (a_kfast) { m = (t >> 4) + pass * 16; k = t & 15; }
            else { k = (t >> 6) + pass * 4; m = t & 63; }
            const long long gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < g.m && gk < kend) ? __ldg(Ab + gm * g.a_sm + gk * g.a_sk) : 0.0f;
            int n, kb;
            if (b_nfast) { kb = (t >> 6) + pass * 4; n = t & 63; }
            else { n = (t >> 4) + pass * 16; kb = t & 15; }
            const long long gn = n0 + n, gkb = k0 + kb;
            Bs[kb][n] = (gn < g.n && gkb < kend) ? __ldg(Bb + gkb * g.b_sk + gn * g.b_sn) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long gm = m0 + ty * 4 + i;
        if (gm >= g.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long gn = n0 + tx * 4 + j;
            if (gn < g.n) Cb[gm * c_sm + gn * c_sn] = acc[i][j];
        }
    }
}

// Sums split-K partials [batch][splits][m][n] into C through its strides, in
// increasing split order (deterministic).
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const __grid_constant__ GemmShape g,
                                                            const float* __restrict__ P, float* __restrict__ C) {
    const long long mn = g.m * g.n, total = g.batch * mn;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const long long bz = e / mn, r = e - bz * mn;
        const long long row = r / g.n, col = r - row * g.n;
        const float* src = P + bz * g.splits * mn + r;
        float acc = 0.0f;
        for (int s = 0; s < g.splits; ++s) acc += src[(long long)s * mn];
        C[g.c_off + bz * g.c_sb + row * g.c_sm + col * g.c_sn] = acc;
    }
}

// The same for few outputs and many splits (per-CTA partials of the tall kernels, per-stream
// partials of the streaming weight gradients): a warp per output, lane l adds the splits
// l, l + 32, ... in increasing order, the lanes are folded by a fixed shuffle tree.  The plain
// kernel would leave each of a few hundred threads with hundreds of dependent-latency loads.
__global__ void __launch_bounds__(256) splitk_reduce_warp_kernel(const __grid_constant__ GemmShape g,
                                                                 const float* __restrict__ P, float* __restrict__ C) {
    const long long mn = g.m * g.n, total = g.batch * mn;
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long e = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; e < total; e += warps) {
        const long long bz = e / mn, r = e - bz * mn;
        const long long row = r / g.n, col = r - row * g.n;
        const float* src = P + bz * g.splits * mn + r;
        float acc = 0.0f;
        for (int s = lane; s < g.splits; s += 32) acc += src[(long long)s * mn];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) C[g.c_off + bz * g.c_sb + row * g.c_sm + col * g.c_sn] = acc;
    }
}

int launch_splitk_reduce(Device* dev, const GemmShape& g, const float* partials, float* c) {
    const long long total = g.batch * g.m * g.n;
    const long long cap = (long long)dev->prop.multiProcessorCount * 16;
    if (g.splits >= 64 && total * 32 <= cap * 256) {
        long long blocks = (total * 32 + 255) / 256;
        splitk_reduce_warp_kernel<<<(unsigned)std::max(1LL, blocks), 256, 0, dev->stream>>>(g, partials, c);
    } else {
        long long blocks = (total + 255) / 256;
        if (blocks > cap) blocks = cap;
        splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(g, partials, c);
    }
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

// Tall-and-skinny weight gradients: C[m][n] = sum_k A[k][m] * B[k][n] with m, n <= 32 and k in
// the millions (conv1 of config 4: dW[32][9] over 2.8 M output positions).  The output is one
// tile, so the generic kernels leave the machine idle; here every warp of the grid owns a
// contiguous run of k: lane = m (one coalesced row of A per k), B's row is read with
// warp-uniform loads, n accumulators live in registers.  Warps are summed through shared
// memory in warp order, CTAs through the split-K partial buffer in CTA order (deterministic).
template <int NB>
__global__ void __launch_bounds__(256) gemm_tall_kernel(const __grid_constant__ GemmShape g, const float* __restrict__ A,
                                                        const float* __restrict__ B, float* __restrict__ P) {
    __shared__ float part[8][32][NB + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * 8;
    const long long per = (g.k + warps - 1) / warps;
    const long long k0 = ((long long)blockIdx.x * 8 + warp) * per;
    const long long k1 = k0 + per < g.k ? k0 + per : g.k;
    const bool mine = lane < g.m;
    const int n = (int)g.n;
    float acc[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[j] = 0.0f;
    const float* ap = A + g.a_off + (mine ? lane : 0);
    const float* bp = B + g.b_off;
    long long k = k0;
    for (; k + 4 <= k1; k += 4) {
        float a[4], b[4][NB];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            a[u] = mine ? __ldg(ap + (k + u) * g.a_sk) : 0.0f;
#pragma unroll
            for (int j = 0; j < NB; ++j) b[u][j] = j < n ? __ldg(bp + (k + u) * g.b_sk + j) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < NB; ++j) acc[j] = fmaf(a[u], b[u][j], acc[j]);
    }
    for (; k < k1; ++k) {
        const float a = mine ? __ldg(ap + k * g.a_sk) : 0.0f;
#pragma unroll
        for (int j = 0; j < NB; ++j) acc[j] = fmaf(a, j < n ? __ldg(bp + k * g.b_sk + j) : 0.0f, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) part[warp][lane][j] = acc[j];
    __syncthreads();
    for (int e = threadIdx.x; e < (int)g.m * n; e += 256) {
        const int row = e / n, col = e - row * n;
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) sum += part[w][row][col];
        P[(long long)blockIdx.x * g.m * g.n + e] = sum;
    }
}

bool gemm_tall_supported(const GemmShape& g) {
    return g.batch == 1 && g.m >= 1 && g.m <= 32 && g.n >= 1 && g.n <= 32 && g.a_sm == 1 && g.b_sn == 1 && g.k >= 16384;
}

int launch_gemm_tall(Device* dev, const Plan& plan, const float* a, const float* b, float* c, void* scratch) {
    const GemmShape& g = plan.gemm;
    EB_REQUIRE(scratch && g.splits >= 1, EB200_ERR_INVALID, "tall GEMM launched without scratch");
    float* partials = reinterpret_cast<float*>(scratch) + g.partial_off;
    const unsigned grid = (unsigned)g.splits;
    if (g.n <= 4) gemm_tall_kernel<4><<<grid, 256, 0, dev->stream>>>(g, a, b, partials);
    else if (g.n <= 8) gemm_tall_kernel<8><<<grid, 256, 0, dev->stream>>>(g, a, b, partials);
    else if (g.n <= 16) gemm_tall_kernel<16><<<grid, 256, 0, dev->stream>>>(g, a, b, partials);
    else gemm_tall_kernel<32><<<grid, 256, 0, dev->stream>>>(g, a, b, partials);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return launch_splitk_reduce(dev, g, partials, c);
}

int launch_gemm_simt(Device* dev, const Plan& plan, const float* a, const float* b, float* c, void* scratch) {
    const GemmShape& g = plan.gemm;
    if (g.m <= 0 || g.n <= 0 || g.batch <= 0) return EB200_OK;
    EB_REQUIRE(g.batch * g.splits <= 65535, EB200_ERR_UNSUPPORTED, "batch %lld x splits %d exceeds grid.z", g.batch, g.splits);
    const long long by = (g.n + GN - 1) / GN;
    EB_REQUIRE(by <= 65535, EB200_ERR_UNSUPPORTED, "n = %lld exceeds grid.y tiles", g.n);
    dim3 grid((unsigned)((g.m + GM - 1) / GM), (unsigned)by, (unsigned)(g.batch * g.splits));
    float* partials = g.splits > 1 ? reinterpret_cast<float*>(scratch) + g.partial_off : nullptr;
    EB_REQUIRE(g.splits == 1 || scratch, EB200_ERR_INVALID, "split-K launched without scratch");
    gemm_simt_kernel<<<grid, 256, 0, dev->stream>>>(g, a, b, g.splits > 1 ? partials : c);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    if (g.splits > 1) return launch_splitk_reduce(dev, g, partials, c);
    return EB200_OK;
}

}  // namespace eb200
