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
#include "expr.cuh"
#include "index.cuh"

namespace eb200 {

constexpr int TT = 64;  // tile edge

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

__global__ void __launch_bounds__(256) transpose_kernel(const __grid_constant__ TrParams q,
                                                        const uint32_t* __restrict__ in,
                                                        uint32_t* __restrict__ out) {
    __shared__ uint32_t tile[TT][TT + 1];
    const int tx = threadIdx.x & 15;   // 16 vectors of 4 across the tile
    const int ty = threadIdx.x >> 4;   // 16 rows per pass
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
        // load: rows of the tile are input lines (fixed c), contiguous along r
#pragma unroll
        for (int pass = 0; pass < TT / 16; ++pass) {
            const int cl = ty + pass * 16;
            const int rl = tx * 4;
            const long long c = c0 + cl, r = r0 + rl;
            if (c < q.C && r < q.R) {
                const long long a = ibase + c * q.in_sc + r;
                if (r + 3 < q.R && (a & 3) == 0) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(in + a));
                    tile[cl][rl] = v.x; tile[cl][rl + 1] = v.y; tile[cl][rl + 2] = v.z; tile[cl][rl + 3] = v.w;
                } else {
                    for (int i = 0; i < 4 && r + i < q.R; ++i) tile[cl][rl + i] = __ldg(in + a + i);
                }
            }
        }
        __syncthreads();
        // store: rows of the output (fixed r), contiguous along c
#pragma unroll
        for (int pass = 0; pass < TT / 16; ++pass) {
            const int rl = ty + pass * 16;
            const int cl = tx * 4;
            const long long r = r0 + rl, c = c0 + cl;
            if (r < q.R && c < q.C) {
                const long long a = obase + r * q.out_sr + c;
                if (c + 3 < q.C && (a & 3) == 0) {
                    uint4 v;
                    v.x = tile[cl][rl]; v.y = tile[cl + 1][rl]; v.z = tile[cl + 2][rl]; v.w = tile[cl + 3][rl];
                    *reinterpret_cast<uint4*>(out + a) = v;
                } else {
                    for (int i = 0; i < 4 && c + i < q.C; ++i) out[a + i] = tile[cl + i][rl];
                }
            }
        }
        __syncthreads();
    }
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
    q.tiles_r = (q.R + TT - 1) / TT;
    q.tiles_c = (q.C + TT - 1) / TT;
    long long batch = 1;
    for (int d = 0; d < q.nbatch; ++d) batch *= q.bshape[d];
    q.tiles = batch * q.tiles_r * q.tiles_c;
    if (q.tiles <= 0) return EB200_OK;
    long long blocks = q.tiles;
    const long long cap = (1LL << 31) - 1;
    if (blocks > cap) blocks = cap;
    transpose_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(q, reinterpret_cast<const uint32_t*>(in),
                                                               reinterpret_cast<uint32_t*>(out));
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

// ---- scatter-add ---------------------------------------------------------------------
__global__ void __launch_bounds__(256) fill_zero_kernel(float* __restrict__ out, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = 0.0f;
}

__global__ void __launch_bounds__(256) scatter_add_kernel(const __grid_constant__ KParams p) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    float* out = reinterpret_cast<float*>(p.out.ptr);
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < p.total; e += stride) {
        long long idx[KMAX_DIMS];
        decompose(p, e, idx);
        const KOperand& o = p.in[0];
        float v;
        if (o.n_bounds && !bounds_ok(p, o, idx)) v = o.pad;
        else v = load_elem(o, operand_index(p, o, idx));
        atomicAdd(out + operand_index(p, p.out, idx), v);
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
        scatter_add_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(p);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
    }
    return EB200_OK;
}

// ---- SGD ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) sgd_kernel(const float* __restrict__ p, const float* __restrict__ g,
                                                  float* __restrict__ out, long long n, float lr) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const long long nvec = aligned ? (n >> 2) : 0;
    for (long long v = tid; v < nvec; v += stride) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p) + v);
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
