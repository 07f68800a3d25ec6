// Device-resident optimizer steps over flat parameter / gradient buffers.
//
// The reference updates parameters on the host: every step reads each gradient
// back, runs a Rust `for` loop and uploads a fresh tensor
// (crates/nn/src/optim/optimizer.rs:100-131).  Its two stateful rules are
// restated here as single kernels whose state (velocity, moments, step counter)
// never leaves the device:
//
//   SGD with momentum  crates/nn/src/optim/sgd.rs:84-89
//       v = momentum * v - lr * g;  p = p + v
//   Adam               crates/nn/src/optim/adam.rs:104-147
//       m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g
//       p = p - lr * (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps)
//
// The host loops are IEEE f32 (Rust never contracts a*b+c), so every operation
// is an explicitly rounded intrinsic in the reference's order and the results
// are bit-identical to the host loop.  12 B (momentum: 20 B, Adam: 28 B) of
// traffic per parameter: HBM-bound streaming kernels.
#include <algorithm>

#include "common.h"

namespace eb200 {

// f32::powi as the Rust runtime computes it (repeated squaring, products taken
// from the lowest set bit of the exponent upwards).
__device__ __forceinline__ float powi_f32(float a, int b) {
    const bool recip = b < 0;
    unsigned n = recip ? 0u - (unsigned)b : (unsigned)b;
    float r = 1.0f;
    while (true) {
        if (n & 1u) r = __fmul_rn(r, a);
        n >>= 1;
        if (n == 0) break;
        a = __fmul_rn(a, a);
    }
    return recip ? __fdiv_rn(1.0f, r) : r;
}

__device__ __forceinline__ float momentum_step(float p, float g, float& v, float lr, float momentum) {
    v = __fsub_rn(__fmul_rn(momentum, v), __fmul_rn(lr, g));
    return __fadd_rn(p, v);
}

// 128-bit accesses when every buffer is 16-byte aligned (flat parameter buffers are); `out` may be `p`.
__global__ void __launch_bounds__(256) sgd_momentum_kernel(const float* p, const float* __restrict__ g, float* v, float* out,
                                                           long long n, float lr, float momentum) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(v) |
                           reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const long long nvec = aligned ? (n >> 2) : 0;
    for (long long i = tid; i < nvec; i += stride) {
        const float4 pv = reinterpret_cast<const float4*>(p)[i];
        const float4 gv = __ldg(reinterpret_cast<const float4*>(g) + i);
        float4 vv = reinterpret_cast<float4*>(v)[i];
        float4 r;
        r.x = momentum_step(pv.x, gv.x, vv.x, lr, momentum); r.y = momentum_step(pv.y, gv.y, vv.y, lr, momentum);
        r.z = momentum_step(pv.z, gv.z, vv.z, lr, momentum); r.w = momentum_step(pv.w, gv.w, vv.w, lr, momentum);
        reinterpret_cast<float4*>(v)[i] = vv;
        reinterpret_cast<float4*>(out)[i] = r;
    }
    for (long long i = (nvec << 2) + tid; i < n; i += stride) {
        float vi = v[i];
        out[i] = momentum_step(p[i], g[i], vi, lr, momentum);
        v[i] = vi;
    }
}

struct AdamConsts { float lr, beta1, beta2, eps, omb1, omb2, bc1, bc2; };

__device__ __forceinline__ float adam_step(float p, float g, float& m, float& v, const AdamConsts& c) {
    m = __fadd_rn(__fmul_rn(c.beta1, m), __fmul_rn(c.omb1, g));
    v = __fadd_rn(__fmul_rn(c.beta2, v), __fmul_rn(__fmul_rn(c.omb2, g), g));
    const float m_hat = __fdiv_rn(m, c.bc1), v_hat = __fdiv_rn(v, c.bc2);
    return __fsub_rn(p, __fdiv_rn(__fmul_rn(c.lr, m_hat), __fadd_rn(__fsqrt_rn(v_hat), c.eps)));
}

__global__ void __launch_bounds__(256) adam_kernel(const float* p, const float* __restrict__ g, float* m, float* v, int* t,
                                                   float* out, long long n, float lr, float beta1, float beta2, float eps,
                                                   unsigned* ticket) {
    // every CTA reads the old step count before the last CTA to finish replaces it
    const int step = *reinterpret_cast<volatile int*>(t) + 1;
    AdamConsts c;
    c.lr = lr; c.beta1 = beta1; c.beta2 = beta2; c.eps = eps;
    c.bc1 = __fsub_rn(1.0f, powi_f32(beta1, step));
    c.bc2 = __fsub_rn(1.0f, powi_f32(beta2, step));
    c.omb1 = __fsub_rn(1.0f, beta1); c.omb2 = __fsub_rn(1.0f, beta2);
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                           reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const long long nvec = aligned ? (n >> 2) : 0;
    for (long long i = tid; i < nvec; i += stride) {
        const float4 pv = reinterpret_cast<const float4*>(p)[i];
        const float4 gv = __ldg(reinterpret_cast<const float4*>(g) + i);
        float4 mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
        float4 r;
        r.x = adam_step(pv.x, gv.x, mv.x, vv.x, c); r.y = adam_step(pv.y, gv.y, mv.y, vv.y, c);
        r.z = adam_step(pv.z, gv.z, mv.z, vv.z, c); r.w = adam_step(pv.w, gv.w, mv.w, vv.w, c);
        reinterpret_cast<float4*>(m)[i] = mv;
        reinterpret_cast<float4*>(v)[i] = vv;
        reinterpret_cast<float4*>(out)[i] = r;
    }
    for (long long i = (nvec << 2) + tid; i < n; i += stride) {
        float mi = m[i], vi = v[i];
        out[i] = adam_step(p[i], g[i], mi, vi, c);
        m[i] = mi; v[i] = vi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            *t = step;
            *ticket = 0u;
            __threadfence();
        }
    }
}

static unsigned optim_blocks(Device* dev, long long n) {
    long long blocks = (n / 4 + 255) / 256 + 1;
    const long long cap = (long long)dev->prop.multiProcessorCount * 16;
    return (unsigned)std::max(1LL, std::min(blocks, cap));
}

int launch_sgd_momentum(Device* dev, const Plan& plan, const float* p, const float* g, float* v, float* out, long long n) {
    if (n <= 0) return EB200_OK;
    sgd_momentum_kernel<<<optim_blocks(dev, n), 256, 0, dev->stream>>>(p, g, v, out, n, plan.scalar, plan.hyper[0]);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

int launch_adam(Device* dev, const Plan& plan, const float* p, const float* g, float* m, float* v, int* t, float* out,
                long long n, void* scratch) {
    EB_REQUIRE(scratch, EB200_ERR_INVALID, "Adam launched without its ticket word");
    if (n <= 0) return EB200_OK;
    adam_kernel<<<optim_blocks(dev, n), 256, 0, dev->stream>>>(p, g, m, v, t, out, n, plan.scalar, plan.hyper[0], plan.hyper[1],
                                                               plan.hyper[2], reinterpret_cast<unsigned*>(scratch));
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

}  // namespace eb200

// ---- log-softmax + cross-entropy, forward and backward -------------------------------------
// The reference composes the loss from a dozen tiny kernels (row max, subtract, exp, row sum,
// ln, subtract, multiply by the one-hot targets, two sums, scale: crates/nn/src/functional/
// activation.rs:174-187, loss.rs:32-65) and its gradient from as many again.  On [N, 10]
// logits each of them is launch latency only.  Here one kernel does both directions in the
// reference's arithmetic (exp = exp2(x * log2e), ln = log2(x) * (1 / log2e), classes summed
// in index order): a thread per row, per-CTA loss partials added in CTA order by the last
// CTA to finish (deterministic).
namespace eb200 {

constexpr int XENT_MAX_CTAS = 512;

__global__ void __launch_bounds__(256) softmax_xent_kernel(const float* __restrict__ logits, const float* __restrict__ onehot,
                                                           float* __restrict__ out, int n, int c, float scale,
                                                           float* partials, unsigned* ticket) {
    const float log2e = 1.4426950408889634f;       // std::f32::consts::LOG2_E
    const float inv_log2e = 1.0f / log2e;
    __shared__ float warp_sum[8];
    float* grad = out + 64;
    float local = 0.0f;
    for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < n; row += gridDim.x * blockDim.x) {
        const float* x = logits + (long long)row * c;
        const float* t = onehot + (long long)row * c;
        float m = -INFINITY;
        for (int j = 0; j < c; ++j) m = fmaxf(m, x[j]);
        float s = 0.0f, tsum = 0.0f;
        for (int j = 0; j < c; ++j) { s += exp2f((x[j] - m) * log2e); tsum += t[j]; }
        const float lse = log2f(s) * inv_log2e;
        const float inv_s = 1.0f / s;
        float acc = 0.0f;
        for (int j = 0; j < c; ++j) {
            const float z = x[j] - m;
            acc += t[j] * (z - lse);
            grad[(long long)row * c + j] = scale * (t[j] - exp2f(z * log2e) * inv_s * tsum);
        }
        local += acc;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float cta = 0.0f;
        for (int w = 0; w < 8; ++w) cta += warp_sum[w];
        partials[blockIdx.x] = cta;
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            float total = 0.0f;
            for (unsigned b = 0; b < gridDim.x; ++b) total += __ldcg(partials + b);
            out[0] = scale * total;
            *ticket = 0u;
            __threadfence();
        }
    }
}

int launch_softmax_xent(Device* dev, const Plan& plan, const float* logits, const float* onehot, float* out, void* scratch) {
    EB_REQUIRE(scratch, EB200_ERR_INVALID, "softmax cross-entropy launched without scratch");
    const int n = (int)plan.p.shape[0], c = (int)plan.p.shape[1];
    float* partials = reinterpret_cast<float*>(scratch);
    unsigned* ticket = reinterpret_cast<unsigned*>(partials + XENT_MAX_CTAS);
    const unsigned grid = (unsigned)std::max(1, std::min(XENT_MAX_CTAS, (n + 255) / 256));
    softmax_xent_kernel<<<grid, 256, 0, dev->stream>>>(logits, onehot, out, n, c, plan.scalar, partials, ticket);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

}  // namespace eb200
