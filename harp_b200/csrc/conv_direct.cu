// conv2d for layers whose reduction is tiny (C * KH * KW <= 32: the first layer of
// config 4 has K = 9).  A 128-row tensor-core tile would be seven eighths padding and
// the kernel ends up bound by per-tile handshakes; these layers are pure streaming
// (conv1: 12.8 MB in, 354 MB out), so plain FFMA code with coalesced accesses is the
// right tool: lanes are consecutive output positions, a thread keeps its K window
// values in registers, the weights sit in shared memory and are read warp-uniformly.
// Accumulation is f32 FMA in the reference's (c, kh, kw) order
// (crates/nn/src/functional/conv.rs:113-184 lowers to a sequential sum over k).
#include <stdlib.h>

#include <algorithm>

#include "common.h"

namespace eb200 {

struct DirectParams {
    int N, C, H, W, Co, KH, KW, pad;
    int Ho, Wo, P, K, K4;      // positions per image; K rounded up to a multiple of 4
    long long M;               // N * P
    int relu, has_bias, flip, nchw_out, g_nchw;
    int streams, chunks;       // weight gradient: position streams x channel chunks (8 or 4 channels per warp)
};

__device__ __forceinline__ void window_offsets(const DirectParams& q, int k, int& off, int& kh, int& kw) {
    const int taps = q.KH * q.KW;
    const int c = k / taps, r = k - c * taps;
    kh = r / q.KW; kw = r - kh * q.KW;
    off = (c * q.H + kh) * q.W + kw;
}

// ---- forward (and input gradient through the flipped weights) -------------------------------
template <int KT>
__global__ void __launch_bounds__(256) conv2d_direct_kernel(const __grid_constant__ DirectParams q, const float* __restrict__ x,
                                                            const float* __restrict__ w, const float* __restrict__ bias,
                                                            float* __restrict__ out) {
    extern __shared__ float ws[];                 // [Co][K4] weights, then [Co] bias
    float* bs = ws + (size_t)q.Co * q.K4;
    const int taps = q.KH * q.KW;
    for (int e = threadIdx.x; e < q.Co * q.K4; e += 256) {
        const int co = e / q.K4, k = e - co * q.K4;
        float v = 0.0f;
        if (k < q.K) {
            long long at = (long long)co * q.K + k;
            if (q.flip) {                          // w'[co][c][tap] = w[c][co][taps - 1 - tap]
                const int c = k / taps, tap = k - c * taps;
                at = ((long long)c * q.Co + co) * taps + (taps - 1 - tap);
            }
            v = w[at];
        }
        ws[e] = v;
    }
    for (int e = threadIdx.x; e < q.Co; e += 256) bs[e] = q.has_bias ? bias[e] : 0.0f;
    __shared__ int2 ktab[KT];                       // per k: {offset of the tap in the window, kh | kw << 16}
    if (threadIdx.x < KT) {
        int off = 0, kh = 0, kw = 0;
        if ((int)threadIdx.x < q.K) window_offsets(q, threadIdx.x, off, kh, kw);
        ktab[threadIdx.x] = make_int2(off, kh | (kw << 16));
    }
    __syncthreads();
    int koff[KT];
#pragma unroll
    for (int k = 0; k < KT; ++k) koff[k] = ktab[k].x;

    const unsigned stride = gridDim.x * 256u, M = (unsigned)q.M;
    for (unsigned m = blockIdx.x * 256u + threadIdx.x; m < M; m += stride) {
        const int n = (int)(m / (unsigned)q.P), pos = (int)(m - (unsigned)n * (unsigned)q.P);
        const int oh = pos / q.Wo, ow = pos - oh * q.Wo;
        const float* xb = x + ((long long)n * q.C * q.H + (oh - q.pad)) * q.W + (ow - q.pad);
        float xv[KT];
        if (q.pad == 0) {
#pragma unroll
            for (int k = 0; k < KT; ++k) xv[k] = k < q.K ? __ldg(xb + koff[k]) : 0.0f;
        } else {
#pragma unroll
            for (int k = 0; k < KT; ++k) {
                const int2 e = ktab[k];
                const bool in = k < q.K && (unsigned)(oh + (e.y & 0xffff) - q.pad) < (unsigned)q.H &&
                                (unsigned)(ow + (e.y >> 16) - q.pad) < (unsigned)q.W;
                xv[k] = in ? __ldg(xb + e.x) : 0.0f;
            }
        }
        float* o_nchw = out + (long long)n * q.Co * q.P + pos;
        float* o_rows = out + (long long)m * q.Co;
        const bool rows4 = !q.nchw_out && (q.Co & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        // four output channels at a time: in the rows layout they leave as one 128-bit store
        for (int co = 0; co < q.Co; co += 4) {
            float acc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = co + j < q.Co ? bs[co + j] : 0.0f;
#pragma unroll
            for (int k4 = 0; k4 < KT / 4; ++k4) {
                if (k4 * 4 < q.K) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (co + j < q.Co) {
                            const float4 t = reinterpret_cast<const float4*>(ws + (size_t)(co + j) * q.K4)[k4];   // warp-uniform address
                            acc[j] = fmaf(xv[4 * k4], t.x, acc[j]);
                            acc[j] = fmaf(xv[4 * k4 + 1], t.y, acc[j]);
                            acc[j] = fmaf(xv[4 * k4 + 2], t.z, acc[j]);
                            acc[j] = fmaf(xv[4 * k4 + 3], t.w, acc[j]);
                        }
                    }
                }
            }
            if (q.relu) {
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = fmaxf(acc[j], 0.0f);
            }
            if (rows4) {
                *reinterpret_cast<float4*>(o_rows + co) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (co + j < q.Co) {
                        if (q.nchw_out) o_nchw[(long long)(co + j) * q.P] = acc[j];     // a warp writes 32 consecutive positions of one plane
                        else o_rows[co + j] = acc[j];
                    }
                }
            }
        }
    }
}

// ---- weight gradient ------------------------------------------------------------------------
// dW[co][k] = sum_m g[m][co] * x_k[m].  A warp owns one chunk of 8 output channels and a stream
// of positions (lane = position); 8 x K accumulators per thread, folded over the lanes by
// shuffles at the end, one partial per stream summed in stream order afterwards.
template <int KT, int CHN, int UP>
__global__ void __launch_bounds__(256) conv2d_direct_wgrad_kernel(const __grid_constant__ DirectParams q, const float* __restrict__ x,
                                                                  const float* __restrict__ g, float* __restrict__ partials) {
    __shared__ int2 ktab[KT];                       // per k: {offset of the tap in the window, kh | kw << 16}
    if (threadIdx.x < KT) {
        int off = 0, kh = 0, kw = 0;
        if ((int)threadIdx.x < q.K) window_offsets(q, threadIdx.x, off, kh, kw);
        ktab[threadIdx.x] = make_int2(off, kh | (kw << 16));
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int wg = (int)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int chunk = wg % q.chunks, stream = wg / q.chunks;
    if (stream >= q.streams) return;
    const int co0 = chunk * CHN;
    const unsigned M = (unsigned)q.M, step = (unsigned)q.streams * 32u;
    int koff[KT];                                    // tap offsets, kept in registers
#pragma unroll
    for (int k = 0; k < KT; ++k) koff[k] = ktab[k].x;
    float acc[CHN][KT];
#pragma unroll
    for (int j = 0; j < CHN; ++j)
#pragma unroll
        for (int k = 0; k < KT; ++k) acc[j][k] = 0.0f;
    // UP positions per lane in flight: their loads are all issued before the first FMA
    for (unsigned m0 = (unsigned)stream * 32u + lane; m0 < M; m0 += (unsigned)UP * step) {
        float xv[UP][KT], gv[UP][CHN];
#pragma unroll
        for (int u = 0; u < UP; ++u) {
            const unsigned m = m0 + u * step;
            const bool live = m < M;
            const unsigned n = live ? m / (unsigned)q.P : 0u, pos = live ? m - n * (unsigned)q.P : 0u;
            const int oh = (int)(pos / (unsigned)q.Wo), ow = (int)(pos - (unsigned)oh * (unsigned)q.Wo);
            const float* xb = x + ((long long)n * q.C * q.H + (oh - q.pad)) * q.W + (ow - q.pad);
            if (q.pad == 0) {                                  // every tap of a live position is inside the image
#pragma unroll
                for (int k = 0; k < KT; ++k) xv[u][k] = (live && k < q.K) ? __ldg(xb + koff[k]) : 0.0f;
            } else {
#pragma unroll
                for (int k = 0; k < KT; ++k) {
                    const int2 e = ktab[k];
                    const bool in = live && k < q.K && (unsigned)(oh + (e.y & 0xffff) - q.pad) < (unsigned)q.H &&
                                    (unsigned)(ow + (e.y >> 16) - q.pad) < (unsigned)q.W;
                    xv[u][k] = in ? __ldg(xb + e.x) : 0.0f;
                }
            }
            const float* gp = q.g_nchw ? g + ((long long)n * q.Co + co0) * q.P + pos : g + (long long)m * q.Co + co0;
            const long long gs = q.g_nchw ? (long long)q.P : 1LL;
#pragma unroll
            for (int j = 0; j < CHN; ++j) gv[u][j] = (live && co0 + j < q.Co) ? __ldg(gp + j * gs) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < UP; ++u)
#pragma unroll
            for (int j = 0; j < CHN; ++j)
#pragma unroll
                for (int k = 0; k < KT; ++k) acc[j][k] = fmaf(gv[u][j], xv[u][k], acc[j][k]);
    }
#pragma unroll
    for (int j = 0; j < CHN; ++j)
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            float v = acc[j][k];
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
            if (lane == 0 && k < q.K && co0 + j < q.Co) partials[((long long)stream * q.Co + co0 + j) * q.K + k] = v;
        }
}

// ---- host side ------------------------------------------------------------------------------
static DirectParams direct_params(const ConvShape& c) {
    DirectParams q{};
    q.N = c.N; q.C = c.C; q.H = c.H; q.W = c.W; q.Co = c.Co; q.KH = c.KH; q.KW = c.KW; q.pad = c.pad;
    q.Ho = c.H + 2 * c.pad - c.KH + 1;
    q.Wo = c.W + 2 * c.pad - c.KW + 1;
    q.P = q.Ho * q.Wo;
    q.K = c.C * c.KH * c.KW;
    q.K4 = (q.K + 3) / 4 * 4;
    q.M = (long long)c.N * q.P;
    q.relu = c.relu; q.has_bias = c.has_bias; q.flip = c.flip; q.nchw_out = c.nchw; q.g_nchw = c.g_nchw;
    return q;
}

bool conv2d_direct_supported(const ConvShape& c) {
    const long long K = (long long)c.C * c.KH * c.KW;
    if (c.wgrad) return K <= 12;                    // 8 x K accumulators per thread
    return K <= 32 && (long long)c.Co * ((K + 3) / 4 * 4 + 1) * 4 <= 48 * 1024;
}

static int direct_variant() { return 2; }   // 8: 8 channels x 2 positions, 4: 4 x 4, 2: 4 x 2 (the fastest measured)
static int direct_chn() { return direct_variant() == 8 ? 8 : 4; }

static int direct_streams(const ConvShape& c, int sms) {
    const int chunks = (c.Co + direct_chn() - 1) / direct_chn();
    const int full = std::max(1, (sms * 32) / chunks);       // four CTAs of eight warps per SM
    // small batches: at least 16 steps of 2 x 32 positions per stream, so the per-stream fold (36 shuffle
    // trees, one partial row) and the sum over the streams stay small next to the streaming work
    const long long Ho = c.H + 2 * c.pad - c.KH + 1, Wo = c.W + 2 * c.pad - c.KW + 1;
    const long long by_work = ((long long)c.N * Ho * Wo + 1023) / 1024;
    return (int)std::max(1LL, std::min<long long>(full, by_work));
}

long long conv2d_direct_wgrad_scratch_floats(const ConvShape& c, int sms) {
    return (long long)direct_streams(c, sms) * c.Co * c.C * c.KH * c.KW;
}

int launch_conv2d_direct(Device* dev, const Plan& plan, const float* x, const float* w, const float* bias, float* out) {
    DirectParams q = direct_params(plan.conv);
    q.has_bias = bias != nullptr;
    if (q.M <= 0) return EB200_OK;
    const size_t smem = (size_t)q.Co * (q.K4 + 1) * sizeof(float);
    const long long blocks = std::min<long long>((q.M + 255) / 256, (long long)dev->prop.multiProcessorCount * 8);
    const unsigned grid = (unsigned)blocks;
    if (q.K <= 12) conv2d_direct_kernel<12><<<grid, 256, smem, dev->stream>>>(q, x, w, bias, out);
    else if (q.K <= 20) conv2d_direct_kernel<20><<<grid, 256, smem, dev->stream>>>(q, x, w, bias, out);
    else conv2d_direct_kernel<32><<<grid, 256, smem, dev->stream>>>(q, x, w, bias, out);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

int launch_conv2d_direct_wgrad(Device* dev, const Plan& plan, const float* x, const float* g, float* dw, void* scratch) {
    const ConvShape& c = plan.conv;
    EB_REQUIRE(scratch, EB200_ERR_INVALID, "conv2d weight gradient launched without scratch");
    DirectParams q = direct_params(c);
    q.chunks = (c.Co + direct_chn() - 1) / direct_chn();
    q.streams = direct_streams(c, dev->prop.multiProcessorCount);
    float* partials = reinterpret_cast<float*>(scratch);
    const unsigned grid = (unsigned)((q.streams * q.chunks + 7) / 8);
    EB_REQUIRE(q.K <= 12, EB200_ERR_UNSUPPORTED, "direct weight gradient serves K <= 12");
    // measured on conv1 of config 4 (batch 4096): 4 channels x 2 positions per lane (128 registers, two
    // CTAs per SM) 0.43 ms, 8 x 2 (191 registers) 0.52 ms, 4 x 4 (164 registers) 0.59 ms
    if (direct_variant() == 8) conv2d_direct_wgrad_kernel<12, 8, 2><<<grid, 256, 0, dev->stream>>>(q, x, g, partials);
    else if (direct_variant() == 2) conv2d_direct_wgrad_kernel<12, 4, 2><<<grid, 256, 0, dev->stream>>>(q, x, g, partials);
    else conv2d_direct_wgrad_kernel<12, 4, 4><<<grid, 256, 0, dev->stream>>>(q, x, g, partials);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    // dW[co][k] = sum over streams of partials[stream][co][k]
    GemmShape gs;
    gs.batch = 1; gs.m = c.Co; gs.n = q.K; gs.k = 0;
    gs.splits = q.streams;
    gs.c_off = 0; gs.c_sb = 0; gs.c_sm = q.K; gs.c_sn = 1;
    return launch_splitk_reduce(dev, gs, partials, dw);
}

}  // namespace eb200
