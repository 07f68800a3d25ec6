// max_pool2d with stride = window, forward and gradient, one kernel each.
//
// eclat spells the function as unfold -> max over the window dims
// (crates/nn/src/functional/pool.rs:117-160) and reaches its gradient through the
// max-reduce VJP (mask times gradient, src/grad/rules.rs:379-399) and unfold's VJP, a
// scatter-add (src/grad/rules.rs:40-53).  With stride = window every input element sits in
// at most one window, so both directions are permutation-free streaming passes:
//   forward   y[p][i][j]  = fold of max over the k x k taps x[p][i*k + a][j*k + b], row-major
//             tap order; with the ReLU flag each tap is max(x, 0) first
//   gradient  gx[p][h][w] = (tap < y[p][h/k][w/k]) ? 0 : g[p][h/k][w/k] on covered elements,
//             0 on rows / columns no window covers; with the ReLU flag the activation's own
//             mask follows: gx = x < 0 ? 0 : gx
// Every thread owns one window: it reads the k rows of its window with 64-bit loads when
// k = 2 and the rows are 8-byte aligned (scalar loads otherwise) and, in the gradient, writes
// them back the same way; four windows per thread are in flight.  HBM-bound: the forward
// moves 4 B per covered input element + 4 B per output element, the gradient 8 B per input
// element + 8 B per window.
#include <algorithm>

#include "common.h"

namespace eb200 {

struct PoolParams {
    long long plane;            // H * W
    unsigned H, W, Ho, Wo;      // input plane, full windows per plane
    unsigned Hc, Wc;            // windows per plane counting the partial ones (gradient: they receive zeros)
    unsigned total;             // windows the launch walks
};

constexpr int POOL_U = 4;

template <int K, bool VEC, bool RELU>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const __grid_constant__ PoolParams q, const float* __restrict__ x,
                                                          float* __restrict__ y) {
    const unsigned per_plane = q.Ho * q.Wo;
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned o0 = blockIdx.x * (POOL_U * blockDim.x) + threadIdx.x; o0 < q.total; o0 += POOL_U * stride) {
        float t[POOL_U][K * K];
#pragma unroll
        for (int u = 0; u < POOL_U; ++u) {
            const unsigned o = o0 + u * blockDim.x;
            if (o >= q.total) break;
            const unsigned p = o / per_plane, r = o - p * per_plane;
            const unsigned i = r / q.Wo, j = r - i * q.Wo;
            const float* src = x + (long long)p * q.plane + (long long)(i * K) * q.W + j * K;
            if (VEC) {
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const float2 v = __ldg(reinterpret_cast<const float2*>(src + (long long)a * q.W));
                    t[u][a * 2] = v.x; t[u][a * 2 + 1] = v.y;
                }
            } else {
#pragma unroll
                for (int a = 0; a < K; ++a)
#pragma unroll
                    for (int b = 0; b < K; ++b) t[u][a * K + b] = __ldg(src + (long long)a * q.W + b);
            }
        }
#pragma unroll
        for (int u = 0; u < POOL_U; ++u) {
            const unsigned o = o0 + u * blockDim.x;
            if (o >= q.total) break;
            float m = RELU ? fmaxf(t[u][0], 0.0f) : t[u][0];
#pragma unroll
            for (int a = 1; a < K * K; ++a) m = fmaxf(m, RELU ? fmaxf(t[u][a], 0.0f) : t[u][a]);
            y[o] = m;
        }
    }
}

template <bool RELU>
__device__ __forceinline__ float pool_grad_one(float x, float y, float g) {
    float r = ((RELU ? fmaxf(x, 0.0f) : x) < y) ? 0.0f : g;
    if (RELU) r = x < 0.0f ? 0.0f : r;
    return r;
}

template <int K, bool VEC, bool RELU>
__global__ void __launch_bounds__(256) maxpool_grad_kernel(const __grid_constant__ PoolParams q, const float* __restrict__ g,
                                                           const float* __restrict__ x, const float* __restrict__ y,
                                                           float* __restrict__ gx) {
    const unsigned per_plane = q.Hc * q.Wc;
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned o0 = blockIdx.x * (POOL_U * blockDim.x) + threadIdx.x; o0 < q.total; o0 += POOL_U * stride) {
        float t[POOL_U][K * K], gy[POOL_U][2];
        long long base[POOL_U];
        unsigned rows[POOL_U], cols[POOL_U];       // rows / columns of the window that lie inside the plane
        bool full[POOL_U];
#pragma unroll
        for (int u = 0; u < POOL_U; ++u) {
            const unsigned o = o0 + u * blockDim.x;
            if (o >= q.total) break;
            const unsigned p = o / per_plane, r = o - p * per_plane;
            const unsigned i = r / q.Wc, j = r - i * q.Wc;
            base[u] = (long long)p * q.plane + (long long)(i * K) * q.W + j * K;
            rows[u] = min((unsigned)K, q.H - i * K);
            cols[u] = min((unsigned)K, q.W - j * K);
            full[u] = i < q.Ho && j < q.Wo;
            if (full[u]) {
                const long long w = ((long long)p * q.Ho + i) * q.Wo + j;
                gy[u][0] = __ldg(g + w);
                gy[u][1] = __ldg(y + w);
                if (VEC) {
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const float2 v = __ldg(reinterpret_cast<const float2*>(x + base[u] + (long long)a * q.W));
                        t[u][a * 2] = v.x; t[u][a * 2 + 1] = v.y;
                    }
                } else {
#pragma unroll
                    for (int a = 0; a < K; ++a)
#pragma unroll
                        for (int b = 0; b < K; ++b) t[u][a * K + b] = __ldg(x + base[u] + (long long)a * q.W + b);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < POOL_U; ++u) {
            const unsigned o = o0 + u * blockDim.x;
            if (o >= q.total) break;
            float* dst = gx + base[u];
            if (full[u]) {
                if (VEC) {
#pragma unroll
                    for (int a = 0; a < 2; ++a)
                        *reinterpret_cast<float2*>(dst + (long long)a * q.W) =
                            make_float2(pool_grad_one<RELU>(t[u][a * 2], gy[u][1], gy[u][0]),
                                        pool_grad_one<RELU>(t[u][a * 2 + 1], gy[u][1], gy[u][0]));
                } else {
#pragma unroll
                    for (int a = 0; a < K; ++a)
#pragma unroll
                        for (int b = 0; b < K; ++b)
                            dst[(long long)a * q.W + b] = pool_grad_one<RELU>(t[u][a * K + b], gy[u][1], gy[u][0]);
                }
            } else {
                // a window cut by the plane's edge: no gradient reaches its elements
                for (unsigned a = 0; a < rows[u]; ++a)
                    for (unsigned b = 0; b < cols[u]; ++b) dst[(long long)a * q.W + b] = 0.0f;
            }
        }
    }
}

template <int K, bool VEC>
static void launch_pool_k(Device* dev, const PoolParams& q, int flags, unsigned blocks, const float* a, const float* b,
                          const float* c, float* out) {
    const bool relu = (flags & 1) != 0;
    if (flags & 2) {
        if (relu) maxpool_grad_kernel<K, VEC, true><<<blocks, 256, 0, dev->stream>>>(q, a, b, c, out);
        else maxpool_grad_kernel<K, VEC, false><<<blocks, 256, 0, dev->stream>>>(q, a, b, c, out);
    } else {
        if (relu) maxpool_fwd_kernel<K, VEC, true><<<blocks, 256, 0, dev->stream>>>(q, a, out);
        else maxpool_fwd_kernel<K, VEC, false><<<blocks, 256, 0, dev->stream>>>(q, a, out);
    }
}

// forward: a = x; gradient: a = g, b = x, c = y
int launch_maxpool(Device* dev, const Plan& plan, const float* a, const float* b, const float* c, float* out) {
    const long long P = plan.pool[0], H = plan.pool[1], W = plan.pool[2], K = plan.pool[3];
    const bool grad = (plan.pool_flags & 2) != 0;
    PoolParams q{};
    q.plane = H * W;
    q.H = (unsigned)H; q.W = (unsigned)W;
    q.Ho = (unsigned)(H / K); q.Wo = (unsigned)(W / K);
    q.Hc = (unsigned)((H + K - 1) / K); q.Wc = (unsigned)((W + K - 1) / K);
    const long long total = grad ? P * q.Hc * q.Wc : P * q.Ho * q.Wo;
    EB_REQUIRE(total > 0 && total < (1LL << 31), EB200_ERR_UNSUPPORTED, "max_pool2d over %lld windows", total);
    q.total = (unsigned)total;
    const float* xin = grad ? b : a;
    // 64-bit accesses: window of 2, every row of every plane 8-byte aligned
    const bool vec = K == 2 && (W & 1) == 0 && (q.plane & 1) == 0 && (reinterpret_cast<uintptr_t>(xin) & 7) == 0 &&
                     (!grad || (reinterpret_cast<uintptr_t>(out) & 7) == 0);
    const long long per_block = 256LL * POOL_U;
    const unsigned blocks = (unsigned)std::min<long long>((total + per_block - 1) / per_block, (long long)dev->prop.multiProcessorCount * 32);
    switch (K) {
        case 1: launch_pool_k<1, false>(dev, q, plan.pool_flags, blocks, a, b, c, out); break;
        case 2:
            if (vec) launch_pool_k<2, true>(dev, q, plan.pool_flags, blocks, a, b, c, out);
            else launch_pool_k<2, false>(dev, q, plan.pool_flags, blocks, a, b, c, out);
            break;
        case 3: launch_pool_k<3, false>(dev, q, plan.pool_flags, blocks, a, b, c, out); break;
        default: launch_pool_k<4, false>(dev, q, plan.pool_flags, blocks, a, b, c, out); break;
    }
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

}  // namespace eb200
