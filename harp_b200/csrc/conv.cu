// conv2d_igemm: convolution as an implicit GEMM on the tensor cores.
//
// The reference spells conv2d as pad -> unfold -> permute -> contiguous -> broadcast
// multiply -> sum (crates/nn/src/functional/conv.rs:113-184): two materialised
// copies of the 9x-inflated window tensor and a scalar triple loop.  Here the
// window tensor never exists: out[(n,oh,ow), co] = sum_k A[(n,oh,ow), k] * W[co, k]
// with k = (c, kh, kw) in the reference's order, where the 128 x 32 A tile of each
// k block is gathered straight from x into shared memory by four warps, written
// in the 128-byte-swizzled K-major layout the tensor core expects (the layout a
// TMA load would have produced), while TMA brings the matching weight tile.
// tcgen05.mma kind::tf32 accumulates in tensor memory; the same four warps then
// run the epilogue: bias, optional ReLU, 128-bit stores of [M, Co] rows.
// 3xTF32 splits A into hi/lo on the fly in the gather (no extra pass); the
// weights are split (and padded to a multiple of 32 in K) by a tiny prep kernel.
// Stride 1, symmetric zero padding.  All mbarrier waits are bounded.
#include <stdlib.h>

#include <algorithm>

#include "tc_ptx.cuh"

namespace eb200 {

struct ConvParams {
    int N, C, H, W, Co, KH, KW, pad;
    int Ho, Wo;
    long long M;        // N * Ho * Wo
    int K, Kpad;        // C * KH * KW, rounded up to 32
    int relu, has_bias, three_pass, stages;
    int tap_mask;       // KH * KW <= 32: the table carries one bit per window tap
    int* error_flag;
};

constexpr int CV_THREADS = 192;   // warp 0: TMA (weights), warp 1: MMA, warps 2-5: gather, then epilogue
constexpr int CV_MAX_K = 2048;

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u); }

template <int BN>
__global__ void __launch_bounds__(CV_THREADS, 3)
conv2d_igemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_wlo,
                    const __grid_constant__ ConvParams q, const float* __restrict__ x,
                    const float* __restrict__ bias, float* __restrict__ out) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int B_TILE = BN * TC_BK * 4;
    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + B_TILE);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)q.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + q.stages;
    uint64_t* acc_bar = empty_bar + q.stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    int2* ktab = reinterpret_cast<int2*>(tmem_slot + 2);     // per k: {offset into x, tap bit (or kh | kw << 16)}

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long m0 = (long long)blockIdx.x * TC_BM;
    const int n0 = (int)blockIdx.y * BN;
    const int num_kb = q.Kpad / TC_BK;

    for (int k = threadIdx.x; k < q.Kpad; k += CV_THREADS) {
        int2 e = make_int2(0, 0);
        if (k < q.K) {
            const int c = k / (q.KH * q.KW), r = k - c * q.KH * q.KW;
            const int kh = r / q.KW, kw = r - kh * q.KW;
            e.x = (c * q.H + kh) * q.W + kw;
            e.y = q.tap_mask ? (int)(1u << (kh * q.KW + kw)) : (kh | (kw << 16));
        }
        ktab[k] = e;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < q.stages; ++s) { mbar_init(&full_bar[s], 129); mbar_init(&empty_bar[s], 1); }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, BN < 32 ? 32 : BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % q.stages;
                if (!mbar_wait(&empty_bar[s], ((unsigned)(kb / q.stages) & 1u) ^ 1u, q.error_flag)) break;
                unsigned char* b_hi = smem + (size_t)s * stage_bytes + (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
                mbar_expect_tx(&full_bar[s], (unsigned)((q.three_pass ? 2 : 1) * B_TILE));
                tma_load_3d(b_hi, &map_w, &full_bar[s], kb * TC_BK, n0, 0);
                if (q.three_pass) tma_load_3d(b_hi + B_TILE, &map_wlo, &full_bar[s], kb * TC_BK, n0, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_tf32(TC_BM, BN, 0, 0);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % q.stages;
                if (!mbar_wait(&full_bar[s], (unsigned)(kb / q.stages) & 1u, q.error_flag)) break;
                tc_fence_after();
                const uint32_t st = smem_u32(smem + (size_t)s * stage_bytes);
                const uint32_t a_hi = st, a_lo = st + TC_TILE_BYTES;
                const uint32_t b_hi = st + (q.three_pass ? 2 : 1) * TC_TILE_BYTES, b_lo = b_hi + B_TILE;
#pragma unroll
                for (int j = 0; j < TC_BK / TC_UK; ++j) {
                    const uint32_t step = j * TC_UK * 4;
                    const uint64_t da = umma_desc(a_hi + step, 16, 1024), db = umma_desc(b_hi + step, 16, 1024);
                    umma_tf32(tmem_base, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    if (q.three_pass) {
                        umma_tf32(tmem_base, umma_desc(a_lo + step, 16, 1024), db, idesc, 1u);
                        umma_tf32(tmem_base, da, umma_desc(b_lo + step, 16, 1024), idesc, 1u);
                    }
                }
                umma_commit(&empty_bar[s]);
            }
            umma_commit(acc_bar);
        }
    } else {
        // ---- gather: thread t builds row t of every A tile ----
        const int t = threadIdx.x - 64;                     // 0..127
        const long long row = m0 + t;
        const bool live = row < q.M;
        int n = 0, oh = 0, ow = 0;
        if (live) {
            const int hw = q.Ho * q.Wo;
            n = (int)(row / hw);
            const int r = (int)(row - (long long)n * hw);
            oh = r / q.Wo; ow = r - oh * q.Wo;
        }
        const float* xrow = x + ((long long)n * q.C * q.H + (oh - q.pad)) * q.W + (ow - q.pad);
        // Which taps of the window fall inside the image for this output position: one bit
        // per (kh, kw) when the window has at most 32 taps, so that the per-element test
        // in the gather is a single AND with the tap's bit from the table.
        unsigned vm = 0;
        if (q.tap_mask && live) {
            for (int kh = 0; kh < q.KH; ++kh)
                for (int kw = 0; kw < q.KW; ++kw)
                    if ((unsigned)(oh + kh - q.pad) < (unsigned)q.H && (unsigned)(ow + kw - q.pad) < (unsigned)q.W)
                        vm |= 1u << (kh * q.KW + kw);
        }
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
            const int s = kb % q.stages;
            ok = mbar_wait(&empty_bar[s], ((unsigned)(kb / q.stages) & 1u) ^ 1u, q.error_flag);
            if (!ok) break;
            unsigned char* a_hi = smem + (size_t)s * stage_bytes + (size_t)t * 128;
            unsigned char* a_lo = a_hi + TC_TILE_BYTES;
            // all 32 loads of the row are issued before the first shared-memory store
            float v[32];
            const int2* kt = ktab + kb * TC_BK;
            if (q.tap_mask) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int2 e = kt[i];
                    v[i] = (vm & (unsigned)e.y) ? __ldg(xrow + e.x) : 0.0f;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int2 e = kt[i];
                    const int ih = oh + (e.y & 0xffff) - q.pad, iw = ow + (e.y >> 16) - q.pad;
                    const bool in = live && kb * TC_BK + i < q.K && (unsigned)ih < (unsigned)q.H && (unsigned)iw < (unsigned)q.W;
                    v[i] = in ? __ldg(xrow + e.x) : 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int chunk = (j ^ (t & 7)) * 16;        // 128-byte swizzle: 16-byte chunk index XOR row % 8
                const float v0 = v[4 * j], v1 = v[4 * j + 1], v2 = v[4 * j + 2], v3 = v[4 * j + 3];
                if (q.three_pass) {
                    const float h0 = tf32_hi(v0), h1 = tf32_hi(v1), h2 = tf32_hi(v2), h3 = tf32_hi(v3);
                    *reinterpret_cast<float4*>(a_hi + chunk) = make_float4(h0, h1, h2, h3);
                    *reinterpret_cast<float4*>(a_lo + chunk) = make_float4(v0 - h0, v1 - h1, v2 - h2, v3 - h3);
                } else {
                    *reinterpret_cast<float4*>(a_hi + chunk) = make_float4(v0, v1, v2, v3);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // make the tile visible to the tensor core
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full_bar[s])) : "memory");
        }
        // ---- epilogue: the same warps own tensor-memory lanes 32*(warp%4) .. +31 ----
        const int quarter = warp & 3;
        const bool acc_ok = ok && mbar_wait(acc_bar, 0, q.error_flag);
        tc_fence_after();
        const long long orow = m0 + quarter * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < (BN + 31) / 32; ++c) {
            float v[32];
            tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), v);
            const int col0 = n0 + c * 32;
            if (!acc_ok || orow >= q.M || col0 >= q.Co) continue;
            float* dst = out + orow * q.Co + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (q.has_bias && col0 + i < q.Co) v[i] += __ldg(bias + col0 + i);
                if (q.relu) v[i] = fmaxf(v[i], 0.0f);
            }
            if (col0 + 32 <= q.Co && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col0 + i < q.Co) dst[i] = v[i];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, BN < 32 ? 32 : BN);
}

// Weights [Co][K] -> [Co][Kpad] zero padded, as tf32 hi (and lo) parts.
__global__ void __launch_bounds__(256) conv_prep_weights_kernel(const float* __restrict__ w, float* __restrict__ hi,
                                                                float* __restrict__ lo, int Co, int K, int Kpad, int three) {
    const int total = Co * Kpad;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int co = e / Kpad, k = e - co * Kpad;
        const float v = k < K ? w[(long long)co * K + k] : 0.0f;
        if (three) {
            const float h = tf32_hi(v);
            hi[e] = h;
            lo[e] = v - h;
        } else {
            hi[e] = v;
        }
    }
}

// ---- host side --------------------------------------------------------------------------
bool conv2d_supported(const ConvShape& c) {
    const long long K = (long long)c.C * c.KH * c.KW;
    if (c.N < 1 || c.C < 1 || c.Co < 1 || c.KH < 1 || c.KW < 1 || c.pad < 0) return false;
    if (c.H + 2 * c.pad < c.KH || c.W + 2 * c.pad < c.KW) return false;
    if (K > CV_MAX_K || c.KH >= 32768 || c.KW >= 32768) return false;
    const long long M = (long long)c.N * (c.H + 2 * c.pad - c.KH + 1) * (c.W + 2 * c.pad - c.KW + 1);
    if ((M + TC_BM - 1) / TC_BM >= (1LL << 31)) return false;
    if ((long long)c.N * c.C * c.H * c.W >= (1LL << 31)) return false;     // 32-bit window offsets
    return true;
}

long long conv2d_scratch_floats(const ConvShape& c) {
    const long long kpad = ((long long)c.C * c.KH * c.KW + 31) / 32 * 32;
    return 2 * (long long)c.Co * kpad;
}

int launch_conv2d(Device* dev, const Plan& plan, const float* x, const float* w, const float* bias, float* out, void* scratch) {
    const ConvShape& c = plan.conv;
    EB_REQUIRE(scratch, EB200_ERR_INVALID, "conv2d launched without scratch");
    ConvParams q{};
    q.N = c.N; q.C = c.C; q.H = c.H; q.W = c.W; q.Co = c.Co; q.KH = c.KH; q.KW = c.KW; q.pad = c.pad;
    q.Ho = c.H + 2 * c.pad - c.KH + 1;
    q.Wo = c.W + 2 * c.pad - c.KW + 1;
    q.M = (long long)c.N * q.Ho * q.Wo;
    q.K = c.C * c.KH * c.KW;
    q.Kpad = (q.K + 31) / 32 * 32;
    q.relu = c.relu; q.has_bias = bias != nullptr; q.three_pass = c.mode == EB200_GEMM_3XTF32;
    q.error_flag = dev->error_flag_dev;
    if (q.M <= 0) return EB200_OK;
    float* whi = reinterpret_cast<float*>(scratch);
    float* wlo = whi + (long long)c.Co * q.Kpad;
    {
        const int total = c.Co * q.Kpad;
        const int blocks = std::min(dev->prop.multiProcessorCount * 4, (total + 255) / 256);
        conv_prep_weights_kernel<<<blocks, 256, 0, dev->stream>>>(w, whi, wlo, c.Co, q.K, q.Kpad, q.three_pass);
        count_launch();
    }
    const int bn = c.Co <= 32 ? 32 : (c.Co <= 64 ? 64 : 128);
    CUtensorMap mw, mwl;
    int st;
    if ((st = make_map(&mw, whi, q.Kpad, c.Co, 1, q.Kpad, 0, bn))) return st;
    if ((st = make_map(&mwl, wlo, q.Kpad, c.Co, 1, q.Kpad, 0, bn))) return st;
    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + bn * TC_BK * 4);
    q.tap_mask = c.KH * c.KW <= 32;
    // Three CTAs per SM (75 KB each) when two stages fit in that; the gather warps of one
    // CTA then run under the tensor-core and epilogue phases of the others.
    const size_t fixed = 1024 + 256 + (size_t)q.Kpad * sizeof(int2);
    q.stages = std::max(2, std::min(4, (int)((75 * 1024 - fixed) / stage_bytes)));
    const size_t smem = (size_t)q.stages * stage_bytes + fixed;
    if (!dev->conv_configured) {
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_igemm_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_igemm_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_igemm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        dev->conv_configured = true;
    }
    dim3 grid((unsigned)((q.M + TC_BM - 1) / TC_BM), (unsigned)((c.Co + bn - 1) / bn), 1);
    if (bn == 32) conv2d_igemm_kernel<32><<<grid, CV_THREADS, smem, dev->stream>>>(mw, mwl, q, x, bias, out);
    else if (bn == 64) conv2d_igemm_kernel<64><<<grid, CV_THREADS, smem, dev->stream>>>(mw, mwl, q, x, bias, out);
    else conv2d_igemm_kernel<128><<<grid, CV_THREADS, smem, dev->stream>>>(mw, mwl, q, x, bias, out);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

}  // namespace eb200
