// conv2d_igemm: convolution as an implicit GEMM on the tensor cores.
//
// The reference spells conv2d as pad -> unfold -> permute -> contiguous -> broadcast
// multiply -> sum (crates/nn/src/functional/conv.rs:113-184): two materialised
// copies of the 9x-inflated window tensor and a scalar triple loop.  Here the
// window tensor never exists:  out[(n,oh,ow), co] = sum_k A[(n,oh,ow), k] * W[co, k].
//
// Persistent CTAs (one per SM, 512 threads) walk output tiles of up to 128 positions: whole
// output rows of one image, or 128 consecutive positions of the flattened (n, oh, ow) space
// when small images would otherwise leave rows of the tile empty.  Per tile:
//   loader    brings the input patch the tile's windows touch (32 channels, or all channels
//             when C is not a multiple of 32) into shared memory once: one bulk copy of the
//             raw channel planes for small images, one tiled TMA box with zero fill when
//             W % 4 == 0, else 4-byte asynchronous copies row by row; every input element
//             crosses L2 -> SM once per tile instead of once per window tap;
//   gather    eight warps in two groups (alternate k blocks) build the 128 x 32 A tile of
//             each k block from the patch, shared memory to shared memory, in the
//             128-byte-swizzled K-major layout the tensor core expects (what a TMA load would
//             have produced);
//   TMA       brings the matching weight tile;
//   MMA       the MMA warp runs a warp-uniform loop, one elected lane issues tcgen05.mma
//             kind::tf32 into a double-buffered accumulator in tensor memory;
//   epilogue  four warps drain the accumulator: bias, optional ReLU, then either 128-bit
//             stores of [M, Co] rows or, for the [N, Co, Ho, Wo] layout, one coalesced store
//             per channel plane (a warp's lanes are 32 consecutive positions), while the next
//             tile is already being gathered.
// 3xTF32 splits A into hi/lo on the fly in the gather; the weights are split (reordered,
// padded to a multiple of 32 in K, and for the input gradient transposed and flipped) by a
// small prep kernel.  Patches that do not fit shared memory fall back to gathering from
// global memory.  Stride 1, symmetric zero padding.  All mbarrier waits are bounded.
// The weight gradient is a second kernel further down; layers with C*KH*KW <= 32 run the
// streaming kernels of conv_direct.cu instead.
#include <stdlib.h>

#include <algorithm>

#include "tc_ptx.cuh"

namespace eb200 {

struct ConvParams {
    int N, C, H, W, Co, KH, KW, pad;
    int Ho, Wo;
    int K, Kpad;        // C * KH * KW, rounded up to 32
    int relu, has_bias, three_pass;
    int nchw;           // output as [N, Co, Ho, Wo] instead of [N*Ho*Wo, Co]
    int stages;         // A/B ring
    int mode;           // CV_CBLOCK / CV_TABLE
    int taps;           // KH * KW
    // tile geometry: a tile is Rt output rows x Wt output columns of one image
    int Rt, Wt, tiles_h, tiles_w;
    int m_tiles, n_tiles, tiles;
    // patch geometry: PR x PW input pixels x CB channels, channel stride CH floats
    int staged, pstages, PR, PW, CB, CH, patch_floats;
    int load_mode;      // CV_LOAD_ROWS / CV_LOAD_BULK / CV_LOAD_TMA
    int linear;         // CV_LOAD_BULK only: a tile is 128 consecutive positions of the flattened (n, oh, ow) space and may
                        // span images (whole-row tiles would waste rows: 13 x 13 outputs fill 169 of 256); its patch
                        // holds the planes of every image it touches
    int P, Mtot;        // positions per image, positions in all
    int pcol;           // column of the tile's first window inside a patch row
    int patches_per_tile, kb_per_patch;
    int* error_flag;
};

// How the reduction index k runs over (c, kh, kw):
//   CV_CBLOCK  C % 32 == 0: k = ((c / 32 * taps) + tap) * 32 + c % 32, so one 32-wide k
//              block is 32 channels of ONE tap: one base address per block, then 32
//              reads one channel stride apart;
//   CV_TABLE   k = (c, kh, kw) in the reference's order through a per-k offset table.
enum { CV_CBLOCK = 0, CV_TABLE = 1 };

// How a patch reaches shared memory:
//   CV_LOAD_BULK  small images: the patch is the CB whole channel planes of the tile's image exactly as
//                 they lie in global memory, one contiguous run moved by a single bulk copy; padding is
//                 not materialised, the gather tests one bit per window tap instead;
//   CV_LOAD_TMA   W % 4 == 0: one tiled TMA load of a {PW, PR, CB} box; rows and columns outside the
//                 image (zero padding, the bottom of the last tile) come back as zeros.  The box starts
//                 at a multiple of 4 columns (TMA wants 16-byte aligned starts), pcol columns left of
//                 the first window;
//   CV_LOAD_ROWS  anything else: two warps copy row by row with 4-byte asynchronous copies.
enum { CV_LOAD_ROWS = 0, CV_LOAD_BULK = 1, CV_LOAD_TMA = 2 };

// warp 0: TMA (weights), warp 1: MMA, warps 2-3: patch loaders, warps 4-11: gather, warps 12-15: epilogue
constexpr int CV_THREADS = 512;
constexpr int CV_LOADERS = 64;
constexpr int CV_GATHERERS = 256;     // two groups of 128 threads, alternate k blocks
constexpr int CV_MAX_K = 2048;
constexpr int CV_MAX_PATCH_BYTES = 48 * 1024;

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u); }

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* gmem_src, bool valid) {
    // 4-byte asynchronous copy; src-size 0 writes zeros without touching global memory
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(valid ? 4u : 0u) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    // the barrier gets this thread's arrival once all its earlier cp.async have landed
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct TileCoord { int n, oh0, ow0; };
__device__ __forceinline__ TileCoord tile_coord(const ConvParams& q, int mt) {
    const int per_img = q.tiles_h * q.tiles_w;
    TileCoord t;
    t.n = mt / per_img;
    const int r = mt - t.n * per_img;
    const int th = r / q.tiles_w;
    t.oh0 = th * q.Rt;
    t.ow0 = (r - th * q.tiles_w) * q.Wt;
    return t;
}

template <int BN>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv2d_igemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_wlo,
                    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ ConvParams q, const float* __restrict__ x,
                    const float* __restrict__ bias, float* __restrict__ out) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int B_TILE = BN * TC_BK * 4;
    constexpr unsigned TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + B_TILE);
    float* patch0 = reinterpret_cast<float*>(smem + (size_t)q.stages * stage_bytes);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(patch0 + (size_t)q.pstages * q.patch_floats);
    uint64_t* empty_bar = full_bar + q.stages;
    uint64_t* acc_full = empty_bar + q.stages;       // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;               // [2] epilogue -> MMA
    uint64_t* pfull = acc_empty + 2;                  // [pstages] loaders -> gather
    uint64_t* pempty = pfull + q.pstages;             // [pstages] gather -> loaders
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty + q.pstages);
    int2* ktab = reinterpret_cast<int2*>(tmem_slot + 2);

    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    const int num_kb = q.Kpad / TC_BK;
    const int tiles = q.tiles;

    // ---- offset table: where tap (kh, kw) [of channel c] sits relative to a row's base ----
    {
        const int entries = q.mode == CV_CBLOCK ? q.taps : q.Kpad;
        const int rs = q.staged ? q.PW : q.W;                   // row stride of what the gather reads
        const int cs = q.staged ? q.CH : q.H * q.W;             // channel stride
        for (int k = threadIdx.x; k < entries; k += CV_THREADS) {
            int2 e = make_int2(0, q.staged ? 0 : -1);
            if (q.mode == CV_CBLOCK || k < q.K) {
                const int c = q.mode == CV_CBLOCK ? 0 : k / q.taps;
                const int r = q.mode == CV_CBLOCK ? k : k - c * q.taps;
                const int kh = r / q.KW, kw = r - kh * q.KW;
                e.x = c * cs + kh * rs + kw;
                e.y = q.staged ? (q.load_mode == CV_LOAD_BULK ? (int)(1u << r) : 1) : (kh | (kw << 16));
            }
            ktab[k] = e;
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < q.stages; ++s) { mbar_init(&full_bar[s], 129); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        for (int p = 0; p < q.pstages; ++p) { mbar_init(&pfull[p], q.load_mode == CV_LOAD_ROWS ? CV_LOADERS : 1); mbar_init(&pempty[p], CV_GATHERERS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- weights: one TMA tile (two with the lo part) per k block ----
        if (lane == 0) {
            int s = 0;
            unsigned ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int n0 = (tile % q.n_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(&empty_bar[s], ph ^ 1u, q.error_flag);
                    if (!ok) break;
                    unsigned char* b_hi = smem + (size_t)s * stage_bytes + (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
                    mbar_expect_tx(&full_bar[s], (unsigned)((q.three_pass ? 2 : 1) * B_TILE));
                    tma_load_3d(b_hi, &map_w, &full_bar[s], kb * TC_BK, n0, 0);
                    if (q.three_pass) tma_load_3d(b_hi + B_TILE, &map_wlo, &full_bar[s], kb * TC_BK, n0, 0);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor core: the whole warp runs the loop (its state stays warp-uniform), lane 0 issues ----
        const uint32_t idesc = umma_idesc_tf32(TC_BM, BN, 0, 0);
        const uint32_t smem_base = smem_u32(smem);
        const uint32_t b_off = (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
        int s = 0;
        unsigned ph = 0, ti = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++ti) {
            const unsigned buf = ti & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], ((ti >> 1) & 1u) ^ 1u, q.error_flag));
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * BN;
            for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), ph ^= (s == 0)) {
                ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], ph, q.error_flag));
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_hi = smem_base + (uint32_t)s * (uint32_t)stage_bytes, a_lo = a_hi + TC_TILE_BYTES;
                const uint32_t b_hi = a_hi + b_off, b_lo = b_hi + B_TILE;
                const uint64_t da0 = umma_desc(a_hi, 16, 1024), db0 = umma_desc(b_hi, 16, 1024);
                const uint64_t dal0 = umma_desc(a_lo, 16, 1024), dbl0 = umma_desc(b_lo, 16, 1024);
                if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < TC_BK / TC_UK; ++j) {
                        const uint64_t step = (uint64_t)(j * TC_UK * 4) >> 4;     // the address field counts 16-byte units
                        umma_tf32(acc, da0 + step, db0 + step, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                        if (q.three_pass) {
                            umma_tf32(acc, dal0 + step, db0 + step, idesc, 1u);
                            umma_tf32(acc, da0 + step, dbl0 + step, idesc, 1u);
                        }
                    }
                    umma_commit(&empty_bar[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) umma_commit(&acc_full[buf]);
            __syncwarp();
        }
    } else if (warp < 4) {
        // ---- loaders: input patch -> shared memory, zero filled outside the image ----
        if (q.staged && q.load_mode != CV_LOAD_ROWS) {
            if (warp == 2 && lane == 0) {
                int p = 0;
                unsigned pph = 0;
                bool ok = true;
                const unsigned bytes = (unsigned)(q.CB * q.CH) * 4u;
                for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                    const TileCoord tc = tile_coord(q, tile / q.n_tiles);
                    for (int pp = 0; pp < q.patches_per_tile; ++pp, p = (p + 1 == q.pstages ? 0 : p + 1), pph ^= (p == 0)) {
                        ok = mbar_wait(&pempty[p], pph ^ 1u, q.error_flag);
                        if (!ok) break;
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the gather's reads of this slot precede the copy
                        float* dst = patch0 + (size_t)p * q.patch_floats;
                        if (q.linear) {
                            const int mt = tile / q.n_tiles;
                            const int n_lo = (mt * TC_BM) / q.P, n_hi = min(q.N - 1, (mt * TC_BM + TC_BM - 1) / q.P);
                            mbar_expect_tx(&pfull[p], bytes * (unsigned)(n_hi - n_lo + 1));
                            for (int n = n_lo; n <= n_hi; ++n)
                                bulk_load(dst + (size_t)(n - n_lo) * q.CB * q.CH, x + ((long long)n * q.C + (long long)pp * q.CB) * q.H * q.W, bytes, &pfull[p]);
                            continue;
                        }
                        mbar_expect_tx(&pfull[p], bytes);
                        const long long plane = (long long)tc.n * q.C + (long long)pp * q.CB;
                        if (q.load_mode == CV_LOAD_BULK) bulk_load(dst, x + plane * q.H * q.W, bytes, &pfull[p]);     // CH == H * W
                        else tma_load_3d(dst, &map_x, &pfull[p], tc.ow0 - q.pad - q.pcol, tc.oh0 - q.pad, (int)plane);
                    }
                }
            }
        } else if (q.staged) {
            const int lw = warp - 2;                            // 0..1
            int p = 0;
            unsigned pph = 0;
            bool ok = true;
            const bool flat = q.pad == 0 && q.tiles_w == 1;     // patch rows are whole input rows: a channel plane is one run
            const int G = q.PW <= 8 ? 4 : (q.PW <= 16 ? 2 : 1); // rows per warp pass when rows are short
            const int lpr = 32 / G, g = lane / lpr, pc0 = lane - g * lpr;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const TileCoord tc = tile_coord(q, tile / q.n_tiles);
                const int ih0 = tc.oh0 - q.pad, iw0 = tc.ow0 - q.pad;
                for (int pp = 0; pp < q.patches_per_tile; ++pp, p = (p + 1 == q.pstages ? 0 : p + 1), pph ^= (p == 0)) {
                    ok = mbar_wait(&pempty[p], pph ^ 1u, q.error_flag);
                    if (!ok) break;
                    float* dst = patch0 + (size_t)p * q.patch_floats;
                    const float* src = x + ((long long)tc.n * q.C + (long long)pp * q.CB) * q.H * q.W;
                    if (flat) {
                        const int n_valid = min(q.PR, q.H - ih0) * q.W;     // rows past the image bottom read as zero
                        for (int c = lw; c < q.CB; c += CV_LOADERS / 32) {
                            const float* s_c = src + ((long long)c * q.H + ih0) * q.W;
                            float* d_c = dst + c * q.CH;
                            for (int e = lane; e < q.CH; e += 32) cp_async_f32(d_c + e, e < n_valid ? s_c + e : x, e < n_valid);
                        }
                    } else {
                        const int step = (CV_LOADERS / 32) * G;
                        int pr = lw * G + g, c = 0;
                        while (pr >= q.PR) { pr -= q.PR; ++c; }
                        while (c < q.CB) {
                            const int ih = ih0 + pr;
                            const bool row_ok = (unsigned)ih < (unsigned)q.H;
                            const float* s_r = src + ((long long)c * q.H + ih) * q.W + iw0;
                            float* d_r = dst + c * q.CH + pr * q.PW;
                            for (int pc = pc0; pc < q.PW; pc += lpr) {
                                const bool v = row_ok && (unsigned)(iw0 + pc) < (unsigned)q.W;
                                cp_async_f32(d_r + pc, v ? s_r + pc : x, v);
                            }
                            pr += step;
                            while (pr >= q.PR) { pr -= q.PR; ++c; }
                        }
                    }
                    cp_async_arrive(&pfull[p]);
                }
            }
        }
    } else if (warp < 12) {
        // ---- gather: two groups of 128 threads take alternate k blocks; thread t builds row t of the A tile ----
        const int grp = (warp - 4) >> 2;
        const int t = (threadIdx.x - 128) & 127;            // 0..127
        const int r_oh = t / q.Wt, r_ow = t - r_oh * q.Wt;
        int s = 0, pst = 0;
        unsigned ph = 0, pph = 0, it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const TileCoord tc = tile_coord(q, tile / q.n_tiles);
            int oh = tc.oh0 + r_oh, ow = tc.ow0 + r_ow, slot = 0;
            bool live = r_oh < q.Rt && oh < q.Ho && ow < q.Wo;
            if (q.linear) {
                const int mt = tile / q.n_tiles, m = mt * TC_BM + t;
                live = m < q.Mtot;
                const int n = live ? m / q.P : 0, pos = live ? m - n * q.P : 0;
                oh = pos / q.Wo; ow = pos - oh * q.Wo;
                slot = n - (mt * TC_BM) / q.P;
            }
            // staged: offset of this row's window origin inside the patch; direct: pointer into x
            int base_r = live ? r_oh * q.PW + r_ow + q.pcol : 0;
            unsigned vm = live ? 0xffffffffu : 0u;            // staged: which taps of this row's window to read
            if (q.staged && q.load_mode == CV_LOAD_BULK && live) {
                // the patch is the raw image: the window origin may lie outside it, one bit per tap inside
                base_r = slot * q.CB * q.CH + (oh - q.pad) * q.W + (ow - q.pad);
                vm = 0;
                for (int kh = 0; kh < q.KH; ++kh)
                    for (int kw = 0; kw < q.KW; ++kw)
                        if ((unsigned)(oh + kh - q.pad) < (unsigned)q.H && (unsigned)(ow + kw - q.pad) < (unsigned)q.W)
                            vm |= 1u << (kh * q.KW + kw);
            }
            const float* xrow = x + ((long long)tc.n * q.C * q.H + (oh - q.pad)) * q.W + (ow - q.pad);
            for (int pp = 0; pp < q.patches_per_tile && ok; ++pp, pst = (pst + 1 == q.pstages ? 0 : pst + 1), pph ^= (pst == 0)) {
                if (q.staged) {
                    ok = mbar_wait(&pfull[pst], pph, q.error_flag);
                    if (!ok) break;
                }
                const float* pb = patch0 + (size_t)pst * q.patch_floats + base_r;
                for (int kk = 0; kk < q.kb_per_patch; ++kk, ++it, s = (s + 1 == q.stages ? 0 : s + 1), ph ^= (s == 0)) {
                    if ((int)(it & 1u) != grp) continue;         // the other group's k block
                    ok = mbar_wait(&empty_bar[s], ph ^ 1u, q.error_flag);
                    if (!ok) break;
                    unsigned char* a_hi = smem + (size_t)s * stage_bytes + (size_t)t * 128;
                    unsigned char* a_lo = a_hi + TC_TILE_BYTES;
                    float v[32];                                 // all 32 reads are issued before the first store
                    if (q.staged) {
                        if (q.mode == CV_CBLOCK) {
                            const float* p0 = pb + ktab[kk].x;
                            const bool in = (vm >> (q.load_mode == CV_LOAD_BULK ? kk : 0)) & 1u;
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = in ? p0[i * q.CH] : 0.0f;
                        } else {
                            const int2* kt = ktab + (pp * q.kb_per_patch + kk) * TC_BK;
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const int2 e = kt[i];
                                v[i] = (vm & (unsigned)e.y) ? pb[e.x] : 0.0f;
                            }
                        }
                    } else if (q.mode == CV_CBLOCK) {
                        const int2 e = ktab[kk];
                        const int ih = oh + (e.y & 0xffff) - q.pad, iw = ow + (e.y >> 16) - q.pad;
                        const bool in = live && (unsigned)ih < (unsigned)q.H && (unsigned)iw < (unsigned)q.W;
                        const long long hw_in = (long long)q.H * q.W;
                        const float* p0 = xrow + (long long)pp * 32 * hw_in + e.x;
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = in ? __ldg(p0 + i * hw_in) : 0.0f;
                    } else {
                        const int2* kt = ktab + (pp * q.kb_per_patch + kk) * TC_BK;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int2 e = kt[i];
                            const int ih = oh + (e.y & 0xffff) - q.pad, iw = ow + ((e.y >> 16) & 0x7fff) - q.pad;
                            const bool in = live && e.y >= 0 && (unsigned)ih < (unsigned)q.H && (unsigned)iw < (unsigned)q.W;
                            v[i] = in ? __ldg(xrow + e.x) : 0.0f;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int chunk = (j ^ (t & 7)) * 16;    // 128-byte swizzle: 16-byte chunk index XOR row % 8
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
                    mbar_arrive(&full_bar[s]);
                }
                if (q.staged && ok) mbar_arrive(&pempty[pst]);   // this thread is done reading the patch
            }
        }
    } else {
        // ---- epilogue: warp w owns tensor-memory lanes 32*(w%4) .. +31 ----
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int r_oh = r / q.Wt, r_ow = r - r_oh * q.Wt;
        unsigned ti = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++ti) {
            const unsigned buf = ti & 1u;
            const TileCoord tc = tile_coord(q, tile / q.n_tiles);
            int oh = tc.oh0 + r_oh, ow = tc.ow0 + r_ow, n_img = tc.n;
            bool live = r_oh < q.Rt && oh < q.Ho && ow < q.Wo;
            if (q.linear) {
                const int m = (tile / q.n_tiles) * TC_BM + r;
                live = m < q.Mtot;
                n_img = live ? m / q.P : 0;
                const int pos = live ? m - n_img * q.P : 0;
                oh = pos / q.Wo; ow = pos - oh * q.Wo;
            }
            const long long orow = ((long long)n_img * q.Ho + oh) * q.Wo + ow;
            const int n0 = (tile % q.n_tiles) * BN;
            ok = mbar_wait(&acc_full[buf], (ti >> 1) & 1u, q.error_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                float v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c * 32), v);
                if (c == BN / 32 - 1) {                      // accumulator drained: hand it back to the MMA warp
                    tc_fence_before();
                    mbar_arrive(&acc_empty[buf]);
                }
                const int col0 = n0 + c * 32;
                if (!live || col0 >= q.Co) continue;
                float* dst = out + orow * q.Co + col0;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (q.has_bias && col0 + i < q.Co) v[i] += __ldg(bias + col0 + i);
                    if (q.relu) v[i] = fmaxf(v[i], 0.0f);
                }
                if (q.nchw) {
                    // one plane per channel: the warp's 32 positions are consecutive in every plane
                    const long long plane = (long long)q.Ho * q.Wo;
                    float* d2 = out + (((long long)n_img * q.Co + col0) * q.Ho + oh) * q.Wo + ow;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < q.Co) d2[i * plane] = v[i];
                } else if (col0 + 32 <= q.Co && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < q.Co) dst[i] = v[i];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Weights [Co][K] -> [Co][Kpad] zero padded, in the kernel's k order, as tf32 hi (and lo) parts.
__global__ void __launch_bounds__(256) conv_prep_weights_kernel(const float* __restrict__ w, float* __restrict__ hi,
                                                                float* __restrict__ lo, int Co, int K, int Kpad, int three,
                                                                int cblock_taps, int taps, int flip) {
    const int total = Co * Kpad;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int co = e / Kpad, k = e - co * Kpad;
        int src = k;
        if (cblock_taps) {       // k = ((cb * taps) + tap) * 32 + ci  <-  (cb * 32 + ci) * taps + tap
            const int ci = k & 31, r = k >> 5, cb = r / cblock_taps, tap = r - cb * cblock_taps;
            src = (cb * 32 + ci) * cblock_taps + tap;
        }
        long long at = (long long)co * K + src;
        if (flip && k < K) {     // w'[co][c][tap] = w[c][co][taps - 1 - tap]
            const int c = src / taps, tap = src - c * taps;
            at = ((long long)c * Co + co) * taps + (taps - 1 - tap);
        }
        const float v = k < K ? w[at] : 0.0f;
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
    // the per-k offset table bounds K only when the channels are not blocked by 32
    if ((c.C % 32 != 0 && K > CV_MAX_K) || K > (1 << 20) || c.KH >= 32768 || c.KW >= 32768) return false;
    const long long M = (long long)c.N * (c.H + 2 * c.pad - c.KH + 1) * (c.W + 2 * c.pad - c.KW + 1);
    if (M >= (1LL << 31)) return false;
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
    q.K = c.C * c.KH * c.KW;
    q.Kpad = (q.K + 31) / 32 * 32;
    q.relu = c.relu; q.has_bias = bias != nullptr; q.three_pass = c.mode == EB200_GEMM_3XTF32;
    q.nchw = c.nchw;
    q.error_flag = dev->error_flag_dev;
    if ((long long)c.N * q.Ho * q.Wo <= 0) return EB200_OK;
    q.taps = c.KH * c.KW;
    q.mode = c.C % 32 == 0 ? CV_CBLOCK : CV_TABLE;
    float* whi = reinterpret_cast<float*>(scratch);
    float* wlo = whi + (long long)c.Co * q.Kpad;
    {
        const int total = c.Co * q.Kpad;
        const int blocks = std::min(dev->prop.multiProcessorCount * 4, (total + 255) / 256);
        conv_prep_weights_kernel<<<blocks, 256, 0, dev->stream>>>(w, whi, wlo, c.Co, q.K, q.Kpad, q.three_pass,
                                                                  q.mode == CV_CBLOCK ? q.taps : 0, q.taps, c.flip);
        count_launch();
    }
    const int bn = c.Co <= 32 ? 32 : (c.Co <= 64 ? 64 : 128);
    CUtensorMap mw, mwl;
    int st;
    if ((st = make_map(&mw, whi, q.Kpad, c.Co, 1, q.Kpad, 0, bn))) return st;
    if ((st = make_map(&mwl, wlo, q.Kpad, c.Co, 1, q.Kpad, 0, bn))) return st;

    // tile: whole output rows of one image, up to 128 positions (a 128-wide segment of a longer row)
    q.Wt = std::min(q.Wo, TC_BM);
    q.Rt = q.Wo <= TC_BM ? std::max(1, std::min(q.Ho, TC_BM / q.Wt)) : 1;
    q.tiles_w = (q.Wo + q.Wt - 1) / q.Wt;
    q.tiles_h = (q.Ho + q.Rt - 1) / q.Rt;
    long long m_tiles = (long long)c.N * q.tiles_h * q.tiles_w;
    int linear_imgs = 1;
    q.n_tiles = (c.Co + bn - 1) / bn;
    q.patches_per_tile = q.mode == CV_CBLOCK ? c.C / 32 : 1;
    q.kb_per_patch = q.mode == CV_CBLOCK ? q.taps : q.Kpad / TC_BK;
    // patch: the input pixels the tile's windows touch
    q.PR = q.Rt + c.KH - 1;
    q.PW = q.Wt + c.KW - 1;
    q.CB = q.mode == CV_CBLOCK ? 32 : c.C;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const int load_limit = 2;
    if (load_limit >= 1 && aligned && q.taps <= 32 && ((long long)q.CB * c.H * c.W) % 4 == 0 && ((long long)c.C * c.H * c.W) % 4 == 0 &&
        (long long)q.CB * c.H * c.W * 4 <= CV_MAX_PATCH_BYTES) {
        q.load_mode = CV_LOAD_BULK;          // whole channel planes, unpadded
        q.PR = c.H;
        q.PW = c.W;
        q.P = q.Ho * q.Wo;
        q.Mtot = c.N * q.P;
        // whole-row tiles leave rows empty when Ho * Wo is not close to a multiple of 128: tile the
        // flattened position space instead when that saves a fifth of the tiles and the patch still fits
        const int per_image = q.tiles_h * q.tiles_w, imgs = (TC_BM - 1) / q.P + 2;
        if ((long long)per_image * TC_BM * 5 >= (long long)q.P * 6 &&
            (long long)imgs * q.CB * c.H * c.W * 4 <= CV_MAX_PATCH_BYTES) {
            q.linear = 1;
            linear_imgs = imgs;
        }
    } else if (load_limit >= 2 && aligned && c.W % 4 == 0 && q.CB <= 256 && q.PR <= 256 && q.PW + 6 <= 256) {
        q.load_mode = CV_LOAD_TMA;
        q.pcol = (4 - c.pad % 4) % 4;
        q.PW = (q.PW + q.pcol + 3) / 4 * 4;
    } else {
        q.load_mode = CV_LOAD_ROWS;
    }
    q.CH = q.PR * q.PW;
    q.patch_floats = (linear_imgs * q.CB * q.CH + 31) / 32 * 32;

    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + bn * TC_BK * 4);
    const size_t ktab_bytes = (size_t)(q.mode == CV_CBLOCK ? q.taps : q.Kpad) * sizeof(int2);
    const size_t fixed = 1024 + 256 + ktab_bytes;
    const size_t smem_limit = 220 * 1024;
    const size_t patch_bytes = (size_t)q.patch_floats * 4;
    q.staged = patch_bytes <= (size_t)CV_MAX_PATCH_BYTES;
    if (q.staged) {
        q.pstages = patch_bytes * 3 + 2 * (size_t)stage_bytes + fixed <= smem_limit ? 3 : 2;
        if (patch_bytes * q.pstages + 2 * (size_t)stage_bytes + fixed > smem_limit) q.staged = 0;
    }
    if (!q.staged) { q.pstages = 1; q.patch_floats = 0; q.linear = 0; }
    if (q.linear) m_tiles = ((long long)q.Mtot + TC_BM - 1) / TC_BM;
    EB_REQUIRE(m_tiles * q.n_tiles < (1LL << 31) - (1 << 20), EB200_ERR_UNSUPPORTED, "conv2d has too many tiles");
    q.m_tiles = (int)m_tiles;
    q.tiles = q.m_tiles * q.n_tiles;
    q.stages = (int)std::min<size_t>(6, (smem_limit - fixed - (size_t)q.pstages * q.patch_floats * 4) / stage_bytes);
    EB_REQUIRE(q.stages >= 2, EB200_ERR_UNSUPPORTED, "conv2d tile does not fit shared memory");
    const size_t smem = (size_t)q.stages * stage_bytes + (size_t)q.pstages * q.patch_floats * 4 + fixed;
    if (!dev->conv_configured) {
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_igemm_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_igemm_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_igemm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        dev->conv_configured = true;
    }
    CUtensorMap mx = mw;
    if (q.staged && q.load_mode == CV_LOAD_TMA) {
        const cuuint64_t dims[3] = {(cuuint64_t)c.W, (cuuint64_t)c.H, (cuuint64_t)c.N * c.C};
        const cuuint64_t strides[2] = {(cuuint64_t)c.W * 4, (cuuint64_t)c.H * c.W * 4};
        const cuuint32_t box[3] = {(cuuint32_t)q.PW, (cuuint32_t)q.PR, (cuuint32_t)q.CB};
        if ((st = make_map_plain(&mx, x, dims, strides, box))) return st;
    }
    const unsigned grid = (unsigned)std::min(q.tiles, dev->prop.multiProcessorCount);
    if (bn == 32) conv2d_igemm_kernel<32><<<grid, CV_THREADS, smem, dev->stream>>>(mw, mwl, mx, q, x, bias, out);
    else if (bn == 64) conv2d_igemm_kernel<64><<<grid, CV_THREADS, smem, dev->stream>>>(mw, mwl, mx, q, x, bias, out);
    else conv2d_igemm_kernel<128><<<grid, CV_THREADS, smem, dev->stream>>>(mw, mwl, mx, q, x, bias, out);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}


// =========================================================================================
// Weight gradient of the same convolution, again without the window tensor:
//     dW[co][k] = sum_m G[m][co] * A[m][k],   m = (n, oh, ow),  k = (c, kh, kw),
// (the reference multiplies the output gradient with the materialised unfold and sums
// over the batch and positions: src/grad/rules.rs:196-222 applied to conv.rs:150-170).
// As an MMA: D[k][co], reduction over positions.  The grid is (row tiles of 128 k) x
// (image streams); a CTA walks its images, stages each image's raw channel planes with one
// bulk copy, and per block of 32 positions
//   * TMA brings the G tile [32 positions][BN channels] (co contiguous: the N-major layout),
//     split into hi/lo in place by the gather threads for 3xTF32;
//   * 256 gather threads (two per row) build the A^T tile [128 k][32 positions] from the
//     patch through a per-position table {window origin, valid taps};
//   * one thread issues the MMAs into a single accumulator that lives for the whole kernel.
// Per-CTA partials go to scratch and are summed in stream order (deterministic).
struct WgradParams {
    int N, C, H, W, Co, KH, KW, pad;
    int Ho, Wo, P;      // positions per image
    int K, taps;
    int nb;             // 32-position blocks per image
    int m_tiles, streams;
    int three_pass, stages, pstages;
    int patch_floats;   // C * H * W rounded up to 32
    int* error_flag;
};

constexpr int WG_MAX_POS = 2048;
constexpr int WG_MAX_PATCH_BYTES = 64 * 1024;

template <int BN>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv2d_wgrad_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ WgradParams q,
                    const float* __restrict__ x, float* __restrict__ partials) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int G_TILE = BN * TC_BK * 4;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + G_TILE);   // [A hi | A lo | G hi | G lo]
    float* patch0 = reinterpret_cast<float*>(smem + (size_t)q.stages * stage_bytes);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(patch0 + (size_t)q.pstages * q.patch_floats);
    uint64_t* empty_bar = full_bar + q.stages;
    uint64_t* gfull = empty_bar + q.stages;           // G tile landed
    uint64_t* pfull = gfull + q.stages;
    uint64_t* pempty = pfull + q.pstages;
    uint64_t* acc_full = pempty + q.pstages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    int2* pos = reinterpret_cast<int2*>(tmem_slot + 2);           // per position: {window origin in the plane, valid taps}

    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    const int tile = (int)blockIdx.x % q.m_tiles, stream = (int)blockIdx.x / q.m_tiles;
    const int n_images = stream < q.N ? (q.N - stream + q.streams - 1) / q.streams : 0;
    const int g_off = (q.three_pass ? 2 : 1) * TC_TILE_BYTES;

    for (int m = threadIdx.x; m < q.nb * TC_BK; m += CV_THREADS) {
        int2 e = make_int2(0, 0);
        if (m < q.P) {
            const int oh = m / q.Wo, ow = m - oh * q.Wo;
            e.x = (oh - q.pad) * q.W + (ow - q.pad);
            unsigned vm = 0;
            for (int kh = 0; kh < q.KH; ++kh)
                for (int kw = 0; kw < q.KW; ++kw)
                    if ((unsigned)(oh + kh - q.pad) < (unsigned)q.H && (unsigned)(ow + kw - q.pad) < (unsigned)q.W)
                        vm |= 1u << (kh * q.KW + kw);
            e.y = (int)vm;
        }
        pos[m] = e;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < q.stages; ++s) { mbar_init(&full_bar[s], CV_GATHERERS); mbar_init(&empty_bar[s], 1); mbar_init(&gfull[s], 1); }
        for (int p = 0; p < q.pstages; ++p) { mbar_init(&pfull[p], 1); mbar_init(&pempty[p], CV_GATHERERS); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- G tiles: BN / 32 boxes of [32 positions][32 channels] per block ----
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        for (int i = 0; i < n_images && ok; ++i) {
            const int n = stream + i * q.streams;
            for (int b = 0; b < q.nb; ++b, s = (s + 1 == q.stages ? 0 : s + 1), ph ^= (s == 0)) {
                ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ph ^ 1u, q.error_flag));
                if (!ok) break;
                if (elect_one()) {
                    unsigned char* gt = smem + (size_t)s * stage_bytes + g_off;
                    mbar_expect_tx(&gfull[s], (unsigned)G_TILE);
#pragma unroll
                    for (int j = 0; j < BN / 32; ++j) tma_load_3d(gt + j * 4096, &map_g, &gfull[s], j * 32, n * q.P + b * TC_BK, 0);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---- tensor core ----
        const uint32_t idesc = umma_idesc_tf32(TC_BM, BN, 0, 1);       // A K-major, B N-major
        const uint32_t smem_base = smem_u32(smem);
        int s = 0;
        unsigned ph = 0;
        bool ok = true, first = true;
        for (int i = 0; i < n_images && ok; ++i) {
            for (int b = 0; b < q.nb; ++b, s = (s + 1 == q.stages ? 0 : s + 1), ph ^= (s == 0)) {
                ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], ph, q.error_flag));
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_hi = smem_base + (uint32_t)s * (uint32_t)stage_bytes, a_lo = a_hi + TC_TILE_BYTES;
                const uint32_t g_hi = a_hi + g_off, g_lo = g_hi + G_TILE;
                const uint64_t da0 = umma_desc(a_hi, 16, 1024), dal0 = umma_desc(a_lo, 16, 1024);
                const uint64_t db0 = umma_desc(g_hi, 4096, 512, 1), dbl0 = umma_desc(g_lo, 4096, 512, 1);
                if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < TC_BK / TC_UK; ++j) {
                        const uint64_t as = (uint64_t)(j * TC_UK * 4) >> 4, bs = (uint64_t)(j * 1024) >> 4;
                        umma_tf32(tmem_base, da0 + as, db0 + bs, idesc, (first && j == 0) ? 0u : 1u);
                        if (q.three_pass) {
                            umma_tf32(tmem_base, dal0 + as, db0 + bs, idesc, 1u);
                            umma_tf32(tmem_base, da0 + as, dbl0 + bs, idesc, 1u);
                        }
                    }
                    umma_commit(&empty_bar[s]);
                }
                first = false;
                __syncwarp();
            }
        }
        if (elect_one()) umma_commit(acc_full);
        __syncwarp();
    } else if (warp == 2) {
        // ---- patches: the image's C channel planes, one bulk copy ----
        if (lane == 0) {
            int p = 0;
            unsigned pph = 0;
            const unsigned bytes = (unsigned)(q.C * q.H * q.W) * 4u;
            for (int i = 0; i < n_images; ++i, p = (p + 1 == q.pstages ? 0 : p + 1), pph ^= (p == 0)) {
                const int n = stream + i * q.streams;
                if (!mbar_wait(&pempty[p], pph ^ 1u, q.error_flag)) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(&pfull[p], bytes);
                bulk_load(patch0 + (size_t)p * q.patch_floats, x + (long long)n * q.C * q.H * q.W, bytes, &pfull[p]);
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ---- gather: two threads per k row, 16 positions each ----
        const int gt = threadIdx.x - 128;                   // 0..255
        const int r = gt & 127, half = gt >> 7;
        const int k = tile * TC_BM + r;
        const bool krow = k < q.K;
        int koff = 0;
        unsigned kbit = 0;
        if (krow) {
            const int c = k / q.taps, tap = k - c * q.taps;
            const int kh = tap / q.KW, kw = tap - kh * q.KW;
            koff = c * q.H * q.W + kh * q.W + kw;
            kbit = 1u << tap;
        }
        int s = 0, p = 0;
        unsigned ph = 0, pph = 0;
        bool ok = true;
        for (int i = 0; i < n_images && ok; ++i, p = (p + 1 == q.pstages ? 0 : p + 1), pph ^= (p == 0)) {
            ok = mbar_wait(&pfull[p], pph, q.error_flag);
            if (!ok) break;
            const float* pb = patch0 + (size_t)p * q.patch_floats + koff;
            for (int b = 0; b < q.nb; ++b, s = (s + 1 == q.stages ? 0 : s + 1), ph ^= (s == 0)) {
                ok = mbar_wait(&empty_bar[s], ph ^ 1u, q.error_flag);
                if (!ok) break;
                unsigned char* st = smem + (size_t)s * stage_bytes;
                float v[16];
                const int2* pt = pos + b * TC_BK + half * 16;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int2 e = pt[j];
                    v[j] = ((unsigned)e.y & kbit) ? pb[e.x] : 0.0f;
                }
                unsigned char* a_hi = st + (size_t)r * 128;
                unsigned char* a_lo = a_hi + TC_TILE_BYTES;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int chunk = ((half * 4 + j) ^ (r & 7)) * 16;
                    const float v0 = v[4 * j], v1 = v[4 * j + 1], v2 = v[4 * j + 2], v3 = v[4 * j + 3];
                    if (q.three_pass) {
                        const float h0 = tf32_hi(v0), h1 = tf32_hi(v1), h2 = tf32_hi(v2), h3 = tf32_hi(v3);
                        *reinterpret_cast<float4*>(a_hi + chunk) = make_float4(h0, h1, h2, h3);
                        *reinterpret_cast<float4*>(a_lo + chunk) = make_float4(v0 - h0, v1 - h1, v2 - h2, v3 - h3);
                    } else {
                        *reinterpret_cast<float4*>(a_hi + chunk) = make_float4(v0, v1, v2, v3);
                    }
                }
                if (q.three_pass) {
                    // split the G tile TMA delivered: hi in place, lo beside it (elementwise, so the swizzle does not matter)
                    ok = mbar_wait(&gfull[s], ph, q.error_flag);
                    if (!ok) break;
                    float4* gh = reinterpret_cast<float4*>(st + g_off);
                    float4* gl = reinterpret_cast<float4*>(st + g_off + G_TILE);
#pragma unroll
                    for (int j = 0; j < G_TILE / 16 / CV_GATHERERS; ++j) {
                        const float4 t = gh[gt + j * CV_GATHERERS];
                        const float4 h = make_float4(tf32_hi(t.x), tf32_hi(t.y), tf32_hi(t.z), tf32_hi(t.w));
                        gh[gt + j * CV_GATHERERS] = h;
                        gl[gt + j * CV_GATHERERS] = make_float4(t.x - h.x, t.y - h.y, t.z - h.z, t.w - h.w);
                    }
                } else if (gt == 0) {
                    ok = mbar_wait(&gfull[s], ph, q.error_flag);     // one thread vouches for the G tile
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&full_bar[s]);
            }
            if (ok) mbar_arrive(&pempty[p]);
        }
    } else if (warp >= 12) {
        // ---- epilogue, once: this CTA's partial D[k][co] -> partials[stream][k][co] ----
        const int quarter = warp & 3;
        const int k = tile * TC_BM + quarter * 32 + lane;
        const bool ok = n_images > 0 && mbar_wait(acc_full, 0, q.error_flag);
        tc_fence_after();
        float* dst = partials + ((long long)stream * q.K + k) * q.Co;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            float v[32];
            if (n_images > 0) tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), v);
            if (k >= q.K) continue;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (c * 32 + i < q.Co) dst[c * 32 + i] = ok ? v[i] : 0.0f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

bool conv2d_wgrad_supported(const ConvShape& c) {
    if (!conv2d_supported(c)) return false;
    const long long P = (long long)(c.H + 2 * c.pad - c.KH + 1) * (c.W + 2 * c.pad - c.KW + 1);
    const long long plane = (long long)c.C * c.H * c.W;
    return c.KH * c.KW <= 32 && (P + 31) / 32 * 32 <= WG_MAX_POS && plane * 4 <= WG_MAX_PATCH_BYTES && plane % 4 == 0 &&
           c.Co % 4 == 0 && c.Co <= 128;
}

static int wgrad_streams(const ConvShape& c, int sms) {
    const int m_tiles = (c.C * c.KH * c.KW + TC_BM - 1) / TC_BM;
    return std::max(1, std::min(c.N, sms / m_tiles));
}

long long conv2d_wgrad_scratch_floats(const ConvShape& c, int sms) {
    return (long long)wgrad_streams(c, sms) * c.C * c.KH * c.KW * c.Co;
}

int launch_conv2d_wgrad(Device* dev, const Plan& plan, const float* x, const float* g, float* dw, void* scratch) {
    const ConvShape& c = plan.conv;
    EB_REQUIRE(scratch, EB200_ERR_INVALID, "conv2d weight gradient launched without scratch");
    EB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0, EB200_ERR_UNSUPPORTED,
               "conv2d weight gradient needs 16-byte aligned operands");
    WgradParams q{};
    q.N = c.N; q.C = c.C; q.H = c.H; q.W = c.W; q.Co = c.Co; q.KH = c.KH; q.KW = c.KW; q.pad = c.pad;
    q.Ho = c.H + 2 * c.pad - c.KH + 1;
    q.Wo = c.W + 2 * c.pad - c.KW + 1;
    q.P = q.Ho * q.Wo;
    q.K = c.C * c.KH * c.KW;
    q.taps = c.KH * c.KW;
    q.nb = (q.P + TC_BK - 1) / TC_BK;
    q.m_tiles = (q.K + TC_BM - 1) / TC_BM;
    q.streams = wgrad_streams(c, dev->prop.multiProcessorCount);
    q.three_pass = c.mode == EB200_GEMM_3XTF32;
    q.error_flag = dev->error_flag_dev;
    q.patch_floats = (c.C * c.H * c.W + 31) / 32 * 32;
    const int bn = c.Co <= 32 ? 32 : (c.Co <= 64 ? 64 : 128);
    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + bn * TC_BK * 4);
    const size_t fixed = 1024 + 256 + (size_t)q.nb * TC_BK * sizeof(int2);
    const size_t smem_limit = 220 * 1024;
    q.pstages = 2;
    EB_REQUIRE(fixed + 2 * (size_t)q.patch_floats * 4 + 2 * (size_t)stage_bytes <= smem_limit, EB200_ERR_UNSUPPORTED,
               "conv2d weight gradient does not fit shared memory");
    q.stages = (int)std::min<size_t>(6, (smem_limit - fixed - 2 * (size_t)q.patch_floats * 4) / stage_bytes);
    const size_t smem = (size_t)q.stages * stage_bytes + 2 * (size_t)q.patch_floats * 4 + fixed;
    // the output gradient as [M][Co] rows: boxes of 32 positions x 32 channels, channels contiguous
    CUtensorMap mg;
    int st;
    if ((st = make_map(&mg, g, c.Co, (long long)c.N * q.P, 1, c.Co, 0, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))) return st;
    // function attributes are per device: one bit per device index
    static unsigned long long configured_devices = 0;
    const unsigned long long dev_bit = 1ULL << (dev->index & 63);
    if (!(configured_devices & dev_bit)) {
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_wgrad_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_wgrad_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        EB_CHECK_CUDA(cudaFuncSetAttribute(conv2d_wgrad_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        configured_devices |= dev_bit;
    }
    float* partials = reinterpret_cast<float*>(scratch);
    const unsigned grid = (unsigned)(q.m_tiles * q.streams);
    if (bn == 32) conv2d_wgrad_kernel<32><<<grid, CV_THREADS, smem, dev->stream>>>(mg, q, x, partials);
    else if (bn == 64) conv2d_wgrad_kernel<64><<<grid, CV_THREADS, smem, dev->stream>>>(mg, q, x, partials);
    else conv2d_wgrad_kernel<128><<<grid, CV_THREADS, smem, dev->stream>>>(mg, q, x, partials);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    // dW[co][k] = sum over streams of partials[stream][k][co]
    GemmShape gs;
    gs.batch = 1; gs.m = q.K; gs.n = c.Co; gs.k = 0;
    gs.splits = q.streams;
    gs.c_off = 0; gs.c_sb = 0; gs.c_sm = 1; gs.c_sn = q.K;
    return launch_splitk_reduce(dev, gs, partials, dw);
}

}  // namespace eb200
