// gemm_tc: dense contraction on the 5th-generation tensor cores (sm_100a).
//
// The reference has no f32 matmul op; `C = A.B` is an R_ kernel over a
// broadcast product (crates/nn/src/functional/linear.rs:27-56,
// examples/matmul_demo.rs:43-60) that its backends run as a scalar triple loop.
// The classifier (plan.cpp) recognises the pattern and this file serves it:
//
//   * operands stay f32 in HBM; TMA (cp.async.bulk.tensor, 128-byte swizzle)
//     stages 128 x 32 / 32 x 128 tiles into a shared-memory ring, completion on
//     mbarriers;
//   * one elected thread issues tcgen05.mma kind::tf32 (M=128, N=128, K=8) with
//     the accumulator in tensor memory (128 lanes x 128 columns of f32);
//   * tcgen05.commit hands ring slots back to the TMA warp and, after the last
//     k block, the accumulator to four epilogue warps, which read it with
//     tcgen05.ld and store C.
//
// Modes: TF32 feeds the raw f32 bits (the tensor core ignores the low 13
// mantissa bits); 3xTF32 first splits every operand into hi (exactly
// representable in tf32) and lo = x - hi and accumulates hi.hi + lo.hi + hi.lo,
// which restores f32-level accuracy at three times the MMA work.
//
// Layouts: A K-major or M-major, B K-major ([N][K], the `linear` form) or N-major ([K][N], the matmul_demo
// form); odd strides and unaligned offsets stay on the f32 SIMT kernel.
//
// Kernels: gemm_tc_kernel<BN> (one tile per CTA), gemm_tc1p_kernel<BN> (persistent, the hi / lo split done
// inside by dedicated warps, accumulator double buffered), gemm_tc2p_kernel (persistent CTA pairs,
// cta_group::2, 256 x 256 tiles, accumulator double buffered; also serves f16 / bf16 operands with
// tcgen05.mma kind::f16).
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel raises
// a flag in global memory, leaves its loops, frees its tensor memory and
// returns; eb200_device_sync reports the flag as EB200_ERR_TIMEOUT.
#include <stdlib.h>

#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tc_ptx.cuh"

namespace eb200 {


struct TcParams {
    long long m, n, k;
    long long c_sm, c_sn, c_sb, c_off;
    int b_nmajor;      // 1: B tiles are [k][n] with n contiguous
    int a_mmajor;      // 1: A tiles are [k][m] with m contiguous
    int splits;        // split-K factor (blockIdx.z = batch * splits + split)
    int kb_per_split;  // k blocks per split
    int three_pass;    // 1: 3xTF32
    int stages;
    int raster;        // tile rows per band
    int tiles_n;
    int convert;       // one-CTA kernel, 3xTF32: bit 0 / bit 1 = TMA brings the raw f32 tiles of A / of B and the epilogue warps
                       // split them into hi / lo in shared memory (an operand without its bit comes pre-split from scratch copies)
    int half;          // 0: f32 operands (kind::tf32); EB200_F16 / EB200_BF16: 16-bit operands (kind::f16), pair kernel only
    int bke;           // elements of k per 128-byte block: 32 (f32) or 64 (16-bit)
    int c_dtype;       // storage type of C
    int total_tiles;   // persistent pair kernel: pair tiles over all batches and splits, band padding included
    int tiles_per_z;   // ... per batch x split slot
    int* error_flag;
};


// ---- the kernel -------------------------------------------------------------------------
// Shared memory: [stages][A hi | (A lo) | B hi | (B lo)] tiles, 1024-byte aligned,
// then the mbarriers and the tensor-memory address slot.
template <int TC_BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_alo,
               const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_blo,
               const __grid_constant__ TcParams q, float* __restrict__ C, int a_zmul, int b_zmul) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int B_TILE_BYTES = TC_BN * TC_BK * 4;
    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + B_TILE_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)q.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + q.stages;
    uint64_t* conv_bar = empty_bar + q.stages;       // tiles split into hi / lo (convert mode)
    uint64_t* acc_bar = conv_bar + q.stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);

    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    // Tile order: bands of `raster` tile rows, walked column by column, so the
    // CTAs in flight share a squarish set of A and B panels that stays in L2.
    const int tiles_m = (int)((q.m + TC_BM - 1) / TC_BM);
    const int per_band = q.raster * q.tiles_n;
    const int band = (int)blockIdx.x / per_band, within = (int)blockIdx.x % per_band;
    const int band_rows = min(q.raster, tiles_m - band * q.raster);
    const int tile_m = band * q.raster + within % band_rows;
    const int tile_n = within / band_rows;
    const long long n0 = (long long)tile_n * TC_BN, m0 = (long long)tile_m * TC_BM;
    const int bz = (int)blockIdx.z / q.splits, split = (int)blockIdx.z % q.splits;
    if (tile_n >= q.tiles_n) return;   // padding of the last, shorter band
    const int total_kb = (int)((q.k + TC_BK - 1) / TC_BK);
    const int kb_begin = split * q.kb_per_split;
    const int num_kb = min(total_kb - kb_begin, q.kb_per_split);   // k blocks of this CTA (>= 1 by construction)

    if (threadIdx.x == 0) {
        for (int s = 0; s < q.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); mbar_init(&conv_bar[s], 128); }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TC_BN);   // BN columns of f32 accumulators
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // which lo tiles TMA brings from pre-split copies (the others are made here from the raw tile)
    const bool lo_a = q.three_pass && !(q.convert & 1), lo_b = q.three_pass && !(q.convert & 2);

    // The producer and the MMA warp run their loops as whole warps and elect one lane to
    // issue: TMA and tcgen05.mma take their descriptors and coordinates from uniform
    // registers, and only warp-uniform control flow lets the compiler keep them there
    // (issued from a divergent lane-0 branch every tcgen05.mma cost ~200 cycles to issue).
    if (warp == 0) {
        // ---- TMA producer ----
        int s = 0;
        unsigned phase = 0;
        for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
            if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], phase ^ 1u, q.error_flag))) break;
            if (elect_one()) {
                unsigned char* st = smem + (size_t)s * stage_bytes;
                mbar_expect_tx(&full_bar[s], (unsigned)((lo_a ? 2 : 1) * TC_TILE_BYTES + (lo_b ? 2 : 1) * B_TILE_BYTES));
                const int kx = (kb_begin + kb) * TC_BK;
                unsigned char* a_hi = st;
                unsigned char* b_hi = st + (q.three_pass ? 2 : 1) * TC_TILE_BYTES;   // [A hi | A lo | B hi | B lo]
                if (q.a_mmajor) {
                    // four [32 k][32 m] boxes side by side along m
#pragma unroll
                    for (int j = 0; j < TC_BM / 32; ++j) {
                        tma_load_3d(a_hi + j * 4096, &map_a, &full_bar[s], (int)m0 + j * 32, kx, bz * a_zmul);
                        if (lo_a) tma_load_3d(st + TC_TILE_BYTES + j * 4096, &map_alo, &full_bar[s], (int)m0 + j * 32, kx, bz * a_zmul);
                    }
                } else {
                    tma_load_3d(a_hi, &map_a, &full_bar[s], kx, (int)m0, bz * a_zmul);
                    if (lo_a) tma_load_3d(st + TC_TILE_BYTES, &map_alo, &full_bar[s], kx, (int)m0, bz * a_zmul);
                }
                if (q.b_nmajor) {
                    // four [32 k][32 n] boxes side by side along n
#pragma unroll
                    for (int j = 0; j < TC_BN / 32; ++j) {
                        tma_load_3d(b_hi + j * 4096, &map_b, &full_bar[s], (int)n0 + j * 32, kx, bz * b_zmul);
                        if (lo_b) tma_load_3d(b_hi + B_TILE_BYTES + j * 4096, &map_blo, &full_bar[s], (int)n0 + j * 32, kx, bz * b_zmul);
                    }
                } else {
                    tma_load_3d(b_hi, &map_b, &full_bar[s], kx, (int)n0, bz * b_zmul);
                    if (lo_b) tma_load_3d(b_hi + B_TILE_BYTES, &map_blo, &full_bar[s], kx, (int)n0, bz * b_zmul);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        const uint32_t idesc = umma_idesc_tf32(TC_BM, TC_BN, q.a_mmajor, q.b_nmajor);
        // K-major: step 32 bytes inside the 128-byte swizzled row.
        // M/N-major: step one 8-row group (1024 bytes); m/n atoms are 4096 bytes apart
        // (swizzle atom = 4 k rows = 512 bytes, so one K=8 MMA spans two atoms).
        const uint32_t a_lbo = q.a_mmajor ? 4096 : 16, a_sbo = q.a_mmajor ? 512 : 1024, a_layout = q.a_mmajor ? 1 : 2;
        const uint32_t b_lbo = q.b_nmajor ? 4096 : 16, b_sbo = q.b_nmajor ? 512 : 1024, b_layout = q.b_nmajor ? 1 : 2;
        const uint64_t a_jstep = (q.a_mmajor ? 1024u : (unsigned)(TC_UK * 4)) >> 4;    // descriptor address units of 16 bytes
        const uint64_t b_jstep = (q.b_nmajor ? 1024u : (unsigned)(TC_UK * 4)) >> 4;
        const uint32_t smem_base = smem_u32(smem);
        const uint32_t b_off = (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
        int s = 0;
        unsigned phase = 0;
        for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
            if (!__all_sync(0xffffffffu, mbar_wait(q.convert ? &conv_bar[s] : &full_bar[s], phase, q.error_flag))) break;
            tc_fence_after();
            const uint32_t st = smem_base + (uint32_t)s * (uint32_t)stage_bytes;
            const uint64_t da0 = umma_desc(st, a_lbo, a_sbo, a_layout), dal0 = umma_desc(st + TC_TILE_BYTES, a_lbo, a_sbo, a_layout);
            const uint64_t db0 = umma_desc(st + b_off, b_lbo, b_sbo, b_layout), dbl0 = umma_desc(st + b_off + B_TILE_BYTES, b_lbo, b_sbo, b_layout);
            if (elect_one()) {
#pragma unroll
                for (int j = 0; j < TC_BK / TC_UK; ++j) {
                    const uint64_t da = da0 + j * a_jstep, db = db0 + j * b_jstep;
                    umma_tf32(tmem_base, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    if (q.three_pass) {
                        umma_tf32(tmem_base, dal0 + j * a_jstep, db, idesc, 1u);
                        umma_tf32(tmem_base, da, dbl0 + j * b_jstep, idesc, 1u);
                    }
                }
                umma_commit(&empty_bar[s]);   // slot is free once these MMAs have read it
            }
            __syncwarp();
        }
        if (elect_one()) umma_commit(acc_bar);             // accumulator complete
        __syncwarp();
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32*(warp%4) .. +31 ----
        const int quarter = warp & 3;
        if (q.convert) {
            // 3xTF32 without the pre-split passes over HBM: the raw f32 tiles TMA delivered are split here,
            // hi (tf32-exact) in place, lo = x - hi beside it.  Elementwise, so the swizzle does not matter.
            const int ct = threadIdx.x - 64;                 // 0..127
            int s = 0;
            unsigned phase = 0;
            for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
                if (!mbar_wait(&full_bar[s], phase, q.error_flag)) break;
                unsigned char* st = smem + (size_t)s * stage_bytes;
                float4* ah = reinterpret_cast<float4*>(st);
                float4* al = reinterpret_cast<float4*>(st + TC_TILE_BYTES);
                float4* bh = reinterpret_cast<float4*>(st + 2 * TC_TILE_BYTES);
                float4* bl = reinterpret_cast<float4*>(st + 2 * TC_TILE_BYTES + B_TILE_BYTES);
                if (q.convert & 1)
#pragma unroll 4
                for (int i = ct; i < TC_TILE_BYTES / 16; i += 128) {
                    const float4 t = ah[i];
                    float4 h;
                    h.x = __uint_as_float((__float_as_uint(t.x) + 0x1000u) & 0xffffe000u);
                    h.y = __uint_as_float((__float_as_uint(t.y) + 0x1000u) & 0xffffe000u);
                    h.z = __uint_as_float((__float_as_uint(t.z) + 0x1000u) & 0xffffe000u);
                    h.w = __uint_as_float((__float_as_uint(t.w) + 0x1000u) & 0xffffe000u);
                    ah[i] = h;
                    al[i] = make_float4(t.x - h.x, t.y - h.y, t.z - h.z, t.w - h.w);
                }
                if (q.convert & 2)
#pragma unroll 4
                for (int i = ct; i < B_TILE_BYTES / 16; i += 128) {
                    const float4 t = bh[i];
                    float4 h;
                    h.x = __uint_as_float((__float_as_uint(t.x) + 0x1000u) & 0xffffe000u);
                    h.y = __uint_as_float((__float_as_uint(t.y) + 0x1000u) & 0xffffe000u);
                    h.z = __uint_as_float((__float_as_uint(t.z) + 0x1000u) & 0xffffe000u);
                    h.w = __uint_as_float((__float_as_uint(t.w) + 0x1000u) & 0xffffe000u);
                    bh[i] = h;
                    bl[i] = make_float4(t.x - h.x, t.y - h.y, t.z - h.z, t.w - h.w);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&conv_bar[s])) : "memory");
            }
        }
        const bool ok = mbar_wait(acc_bar, 0, q.error_flag);
        tc_fence_after();
        const long long row = m0 + quarter * 32 + lane;
        // split-K: C is the dense partial buffer [batch*splits][m][n] (strides set by the launcher)
        float* crow = C + q.c_off + (long long)(q.splits > 1 ? (int)blockIdx.z : bz) * q.c_sb + row * q.c_sm;
#pragma unroll 1
        for (int c = 0; c < TC_BN / 32; ++c) {
            float v[32];
            tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), v);
            const long long col0 = n0 + c * 32;
            if (!ok || row >= q.m || col0 >= q.n) continue;
            float* dst = crow + col0 * q.c_sn;
            if (q.c_sn == 1 && col0 + 32 <= q.n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col0 + i < q.n) dst[i * q.c_sn] = v[i];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TC_BN);
}

// ---- one-CTA form, persistent (the in-kernel hi / lo split lives here) --------------------------
// One CTA per SM walks tiles t, t + G, t + 2G, ... (G CTAs); the accumulator is double buffered in tensor
// memory (2 x BN columns), the operand ring runs on across tiles.  Ten warps: 0 TMA, 1 MMA, 2-5 epilogue
// (tensor-memory lanes 32 * (warp % 4) ..), 6-9 split the raw f32 tiles into hi / lo while the previous tile's
// accumulator is drained -- in the one-tile-per-CTA form the same four warps did both, one after the other,
// and every tile paid its own pipeline fill, tensor-memory allocation and epilogue (an MLP layer
// [65536, 256] x [256, 256]: 8 k blocks per tile, a third of the time outside the main loop).
//   full[s]      TMA -> split warps (or -> MMA when nothing is split in the kernel)
//   conv[s]      split warps -> MMA (128 arrivals)
//   empty[s]     MMA -> TMA (tcgen05.commit)
//   acc_full[a]  MMA -> epilogue (tcgen05.commit);  acc_empty[a]  epilogue -> MMA (4 arrivals)
constexpr int TC1P_THREADS = 320;

struct OneTile {
    bool idle;
    long long m0, n0;
    int bz, zslot, kb_begin, num_kb;
};

template <int TC_BN>
__device__ __forceinline__ OneTile decode_one_tile(const TcParams& q, int t) {
    OneTile p;
    const int z = t / q.tiles_per_z, r = t - z * q.tiles_per_z;
    const int tiles_m = (int)((q.m + TC_BM - 1) / TC_BM);
    const int per_band = q.raster * q.tiles_n;
    const int band = r / per_band, within = r - band * per_band;
    const int band_rows = min(q.raster, tiles_m - band * q.raster);
    const int tile_m = band * q.raster + within % band_rows;
    const int tile_n = within / band_rows;
    p.idle = tile_n >= q.tiles_n;
    p.n0 = (long long)tile_n * TC_BN;
    p.m0 = (long long)tile_m * TC_BM;
    p.bz = z / q.splits;
    p.zslot = z;
    const int split = z - p.bz * q.splits;
    const int total_kb = (int)((q.k + TC_BK - 1) / TC_BK);
    p.kb_begin = split * q.kb_per_split;
    p.num_kb = min(total_kb - p.kb_begin, q.kb_per_split);
    return p;
}

template <int TC_BN>
__global__ void __launch_bounds__(TC1P_THREADS, 1)
gemm_tc1p_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_alo,
                 const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_blo,
                 const __grid_constant__ TcParams q, float* __restrict__ C, int a_zmul, int b_zmul) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int B_TILE_BYTES = TC_BN * TC_BK * 4;
    const int stage_bytes = (q.three_pass ? 2 : 1) * (TC_TILE_BYTES + B_TILE_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)q.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + q.stages;
    uint64_t* conv_bar = empty_bar + q.stages;
    uint64_t* acc_full = conv_bar + q.stages;       // [2]
    uint64_t* acc_empty = acc_full + 2;             // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < q.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); mbar_init(&conv_bar[s], 128); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, 2 * TC_BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool lo_a = q.three_pass && !(q.convert & 1), lo_b = q.three_pass && !(q.convert & 2);
    const int first = (int)blockIdx.x, step = (int)gridDim.x;

    if (warp == 0) {
        // ---- TMA producer ----
        int s = 0;
        unsigned phase = 0;
        bool ok = true;
        for (int t = first; t < q.total_tiles && ok; t += step) {
            const OneTile p = decode_one_tile<TC_BN>(q, t);
            if (p.idle) continue;
            for (int kb = 0; kb < p.num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
                if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], phase ^ 1u, q.error_flag))) { ok = false; break; }
                if (elect_one()) {
                    unsigned char* st = smem + (size_t)s * stage_bytes;
                    mbar_expect_tx(&full_bar[s], (unsigned)((lo_a ? 2 : 1) * TC_TILE_BYTES + (lo_b ? 2 : 1) * B_TILE_BYTES));
                    const int kx = (p.kb_begin + kb) * TC_BK;
                    unsigned char* b_hi = st + (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
                    if (q.a_mmajor) {
#pragma unroll
                        for (int j = 0; j < TC_BM / 32; ++j) {
                            tma_load_3d(st + j * 4096, &map_a, &full_bar[s], (int)p.m0 + j * 32, kx, p.bz * a_zmul);
                            if (lo_a) tma_load_3d(st + TC_TILE_BYTES + j * 4096, &map_alo, &full_bar[s], (int)p.m0 + j * 32, kx, p.bz * a_zmul);
                        }
                    } else {
                        tma_load_3d(st, &map_a, &full_bar[s], kx, (int)p.m0, p.bz * a_zmul);
                        if (lo_a) tma_load_3d(st + TC_TILE_BYTES, &map_alo, &full_bar[s], kx, (int)p.m0, p.bz * a_zmul);
                    }
                    if (q.b_nmajor) {
#pragma unroll
                        for (int j = 0; j < TC_BN / 32; ++j) {
                            tma_load_3d(b_hi + j * 4096, &map_b, &full_bar[s], (int)p.n0 + j * 32, kx, p.bz * b_zmul);
                            if (lo_b) tma_load_3d(b_hi + B_TILE_BYTES + j * 4096, &map_blo, &full_bar[s], (int)p.n0 + j * 32, kx, p.bz * b_zmul);
                        }
                    } else {
                        tma_load_3d(b_hi, &map_b, &full_bar[s], kx, (int)p.n0, p.bz * b_zmul);
                        if (lo_b) tma_load_3d(b_hi + B_TILE_BYTES, &map_blo, &full_bar[s], kx, (int)p.n0, p.bz * b_zmul);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        const uint32_t idesc = umma_idesc_tf32(TC_BM, TC_BN, q.a_mmajor, q.b_nmajor);
        const uint32_t a_lbo = q.a_mmajor ? 4096 : 16, a_sbo = q.a_mmajor ? 512 : 1024, a_layout = q.a_mmajor ? 1 : 2;
        const uint32_t b_lbo = q.b_nmajor ? 4096 : 16, b_sbo = q.b_nmajor ? 512 : 1024, b_layout = q.b_nmajor ? 1 : 2;
        const uint64_t a_jstep = (q.a_mmajor ? 1024u : (unsigned)(TC_UK * 4)) >> 4;
        const uint64_t b_jstep = (q.b_nmajor ? 1024u : (unsigned)(TC_UK * 4)) >> 4;
        const uint32_t smem_base = smem_u32(smem);
        const uint32_t b_off = (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
        int s = 0, it = 0;
        unsigned phase = 0;
        bool ok = true;
        for (int t = first; t < q.total_tiles && ok; t += step) {
            const OneTile p = decode_one_tile<TC_BN>(q, t);
            if (p.idle) continue;
            const int a = it & 1;
            const unsigned aphase = (unsigned)(it >> 1) & 1u;
            // the epilogue of the tile that used this half two tiles ago must have drained it
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_empty[a], aphase ^ 1u, q.error_flag))) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + (uint32_t)(a * TC_BN);
            for (int kb = 0; kb < p.num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
                if (!__all_sync(0xffffffffu, mbar_wait(q.convert ? &conv_bar[s] : &full_bar[s], phase, q.error_flag))) { ok = false; break; }
                tc_fence_after();
                const uint32_t st = smem_base + (uint32_t)s * (uint32_t)stage_bytes;
                const uint64_t da0 = umma_desc(st, a_lbo, a_sbo, a_layout), dal0 = umma_desc(st + TC_TILE_BYTES, a_lbo, a_sbo, a_layout);
                const uint64_t db0 = umma_desc(st + b_off, b_lbo, b_sbo, b_layout), dbl0 = umma_desc(st + b_off + B_TILE_BYTES, b_lbo, b_sbo, b_layout);
                if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < TC_BK / TC_UK; ++j) {
                        const uint64_t da = da0 + j * a_jstep, db = db0 + j * b_jstep;
                        umma_tf32(acc, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                        if (q.three_pass) {
                            umma_tf32(acc, dal0 + j * a_jstep, db, idesc, 1u);
                            umma_tf32(acc, da, dbl0 + j * b_jstep, idesc, 1u);
                        }
                    }
                    umma_commit(&empty_bar[s]);
                }
                __syncwarp();
            }
            if (!ok) break;
            if (elect_one()) umma_commit(&acc_full[a]);
            __syncwarp();
            ++it;
        }
    } else if (warp >= 6) {
        // ---- hi / lo split of the raw f32 tiles (3xTF32 without pre-split copies) ----
        if (q.convert) {
            const int ct = threadIdx.x - 192;                // 0..127
            int s = 0;
            unsigned phase = 0;
            bool ok = true;
            for (int t = first; t < q.total_tiles && ok; t += step) {
                const OneTile p = decode_one_tile<TC_BN>(q, t);
                if (p.idle) continue;
                for (int kb = 0; kb < p.num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
                    if (!mbar_wait(&full_bar[s], phase, q.error_flag)) { ok = false; break; }
                    unsigned char* st = smem + (size_t)s * stage_bytes;
                    float4* ah = reinterpret_cast<float4*>(st);
                    float4* al = reinterpret_cast<float4*>(st + TC_TILE_BYTES);
                    float4* bh = reinterpret_cast<float4*>(st + 2 * TC_TILE_BYTES);
                    float4* bl = reinterpret_cast<float4*>(st + 2 * TC_TILE_BYTES + B_TILE_BYTES);
                    if (q.convert & 1)
#pragma unroll 4
                    for (int i = ct; i < TC_TILE_BYTES / 16; i += 128) {
                        const float4 v = ah[i];
                        float4 h;
                        h.x = __uint_as_float((__float_as_uint(v.x) + 0x1000u) & 0xffffe000u);
                        h.y = __uint_as_float((__float_as_uint(v.y) + 0x1000u) & 0xffffe000u);
                        h.z = __uint_as_float((__float_as_uint(v.z) + 0x1000u) & 0xffffe000u);
                        h.w = __uint_as_float((__float_as_uint(v.w) + 0x1000u) & 0xffffe000u);
                        ah[i] = h;
                        al[i] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
                    }
                    if (q.convert & 2)
#pragma unroll 4
                    for (int i = ct; i < B_TILE_BYTES / 16; i += 128) {
                        const float4 v = bh[i];
                        float4 h;
                        h.x = __uint_as_float((__float_as_uint(v.x) + 0x1000u) & 0xffffe000u);
                        h.y = __uint_as_float((__float_as_uint(v.y) + 0x1000u) & 0xffffe000u);
                        h.z = __uint_as_float((__float_as_uint(v.z) + 0x1000u) & 0xffffe000u);
                        h.w = __uint_as_float((__float_as_uint(v.w) + 0x1000u) & 0xffffe000u);
                        bh[i] = h;
                        bl[i] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&conv_bar[s])) : "memory");
                }
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32 * (warp % 4) .. + 31 ----
        const int quarter = warp & 3;
        int it = 0;
        for (int t = first; t < q.total_tiles; t += step) {
            const OneTile p = decode_one_tile<TC_BN>(q, t);
            if (p.idle) continue;
            const int a = it & 1;
            const unsigned aphase = (unsigned)(it >> 1) & 1u;
            if (!mbar_wait_warp(&acc_full[a], aphase, q.error_flag)) break;
            tc_fence_after();
            const long long row = p.m0 + quarter * 32 + lane;
            float* crow = C + q.c_off + (long long)(q.splits > 1 ? p.zslot : p.bz) * q.c_sb + row * q.c_sm;
#pragma unroll 1
            for (int c = 0; c < TC_BN / 32; ++c) {
                float v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * TC_BN + c * 32), v);
                const long long col0 = p.n0 + c * 32;
                if (row >= q.m || col0 >= q.n) continue;
                float* dst = crow + col0 * q.c_sn;
                if (q.c_sn == 1 && col0 + 32 <= q.n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < q.n) dst[i * q.c_sn] = v[i];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[a])) : "memory");
            ++it;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * TC_BN);
}

// ---- two-CTA form: the pair tile -------------------------------------------------------------
// A cluster of two CTAs computes a 256 x 256 tile with tcgen05.mma.cta_group::2:
// CTA r stages rows [r*128, r*128+128) of A and columns [r*128, r*128+128) of B, the
// tensor cores of both SMs read both halves of B, and each CTA's tensor memory holds
// its 128 rows x 256 columns of the accumulator.  Per SM that is 32 KB of operands
// per 128 x 256 x 32 block of MMA work, two thirds of the one-CTA kernel's traffic.
// The MMA is issued by the even CTA only; both CTAs' TMA loads complete on its
// mbarrier; tcgen05.commit multicasts slot-free and accumulator-ready to both.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the mbarrier at this offset in both CTAs of the pair once the MMAs so far are done
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// instruction descriptor for kind::f16: f32 accumulator, A and B both f16 (0) or both bf16 (1), K-major
__device__ __forceinline__ uint32_t umma_idesc_f16(int M, int N, bool bf16) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}

// ---- two-CTA form, persistent -------------------------------------------------------------
// The same pair tile as gemm_tc2_kernel, but one CTA pair per SM pair walks a list of tiles
// (tile t, t + P, t + 2P, ... for P pairs) and the accumulator is double buffered in tensor
// memory (2 x 256 columns = all 512): while the epilogue warps drain tile i (tcgen05.ld ->
// global stores), the MMA thread already accumulates tile i + 1 into the other half.  The
// operand ring keeps running across tile boundaries, so there is no pipeline fill / drain
// and no tensor-memory allocation per tile -- what cost the one-tile-per-CTA form a third of
// its time on short-K tiles (64 x [1024^2]: 32 k blocks per tile).
//   acc_full[a]   MMA -> epilogue, both CTAs (tcgen05.commit, multicast)
//   acc_empty[a]  epilogue warps of both CTAs -> the MMA thread (8 arrivals on the even CTA's barrier)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, unsigned parity, int* error_flag) {
    for (unsigned i = 0; i < TC_SPIN_LIMIT; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (i > 4096) __nanosleep(64);
    }
    atomicExch(error_flag, 1);
    return false;
}

struct PairTile {
    bool idle;
    long long m0, n0;     // first row of this CTA's half, first column of the pair tile
    int bz, zslot;        // batch index; batch * splits + split (slot of split-K partials)
    int kb_begin, num_kb;
};

__device__ __forceinline__ PairTile decode_pair_tile(const TcParams& q, int t, uint32_t rank) {
    PairTile p;
    const int z = t / q.tiles_per_z, r = t - z * q.tiles_per_z;
    const int tiles_m = (int)((q.m + 255) / 256);
    const int per_band = q.raster * q.tiles_n;
    const int band = r / per_band, within = r - band * per_band;
    const int band_rows = min(q.raster, tiles_m - band * q.raster);
    const int tile_m = band * q.raster + within % band_rows;
    const int tile_n = within / band_rows;
    p.idle = tile_n >= q.tiles_n;
    p.n0 = (long long)tile_n * 256;
    p.m0 = (long long)tile_m * 256 + rank * 128;
    p.bz = z / q.splits;
    p.zslot = z;
    const int split = z - p.bz * q.splits;
    const int total_kb = (int)((q.k + q.bke - 1) / q.bke);
    p.kb_begin = split * q.kb_per_split;
    p.num_kb = min(total_kb - p.kb_begin, q.kb_per_split);
    return p;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc2p_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_alo,
                 const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_blo,
                 const __grid_constant__ TcParams q, float* __restrict__ C, int a_zmul, int b_zmul) {
    constexpr int HALF = 128;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int stage_bytes = (q.three_pass ? 2 : 1) * 2 * TC_TILE_BYTES;     // [A hi | (A lo) | B hi | (B lo)], all 128 x 32
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)q.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + q.stages;
    uint64_t* acc_full = empty_bar + q.stages;      // [2]
    uint64_t* acc_empty = acc_full + 2;             // [2], used in the even CTA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    const uint32_t rank = __shfl_sync(0xffffffffu, cluster_ctarank(), 0);
    const int pair = (int)blockIdx.x >> 1, num_pairs = (int)gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < q.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer: the ring runs on across tiles ----
        int s = 0;
        unsigned phase = 0;
        bool ok = true;
        for (int t = pair; t < q.total_tiles && ok; t += num_pairs) {
            const PairTile p = decode_pair_tile(q, t, rank);
            if (p.idle) continue;
            const int nb = (int)p.n0 + (int)rank * HALF;
            for (int kb = 0; kb < p.num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
                if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], phase ^ 1u, q.error_flag))) { ok = false; break; }
                if (elect_one()) {
                    const uint32_t lead = map_to_cta(smem_u32(&full_bar[s]), 0);
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2u * (unsigned)stage_bytes);
                    unsigned char* st = smem + (size_t)s * stage_bytes;
                    const int kx = (p.kb_begin + kb) * q.bke;
                    unsigned char* b_hi = st + (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
                    if (q.a_mmajor) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            tma_load_3d_pair(st + j * 4096, &map_a, lead, (int)p.m0 + j * 32, kx, p.bz * a_zmul);
                            if (q.three_pass) tma_load_3d_pair(st + TC_TILE_BYTES + j * 4096, &map_alo, lead, (int)p.m0 + j * 32, kx, p.bz * a_zmul);
                        }
                    } else {
                        tma_load_3d_pair(st, &map_a, lead, kx, (int)p.m0, p.bz * a_zmul);
                        if (q.three_pass) tma_load_3d_pair(st + TC_TILE_BYTES, &map_alo, lead, kx, (int)p.m0, p.bz * a_zmul);
                    }
                    if (q.b_nmajor) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            tma_load_3d_pair(b_hi + j * 4096, &map_b, lead, nb + j * 32, kx, p.bz * b_zmul);
                            if (q.three_pass) tma_load_3d_pair(b_hi + TC_TILE_BYTES + j * 4096, &map_blo, lead, nb + j * 32, kx, p.bz * b_zmul);
                        }
                    } else {
                        tma_load_3d_pair(b_hi, &map_b, lead, kx, nb, p.bz * b_zmul);
                        if (q.three_pass) tma_load_3d_pair(b_hi + TC_TILE_BYTES, &map_blo, lead, kx, nb, p.bz * b_zmul);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            // ---- MMA issuer (even CTA) ----
            const uint32_t idesc = q.half ? umma_idesc_f16(256, 256, q.half == EB200_BF16) : umma_idesc_tf32(256, 256, q.a_mmajor, q.b_nmajor);
            const uint32_t a_lbo = q.a_mmajor ? 4096 : 16, a_sbo = q.a_mmajor ? 512 : 1024, a_layout = q.a_mmajor ? 1 : 2;
            const uint32_t b_lbo = q.b_nmajor ? 4096 : 16, b_sbo = q.b_nmajor ? 512 : 1024, b_layout = q.b_nmajor ? 1 : 2;
            const uint64_t a_jstep = (q.a_mmajor ? 1024u : (unsigned)(TC_UK * 4)) >> 4;
            const uint64_t b_jstep = (q.b_nmajor ? 1024u : (unsigned)(TC_UK * 4)) >> 4;
            const uint32_t smem_base = smem_u32(smem);
            const uint32_t b_off = (q.three_pass ? 2 : 1) * TC_TILE_BYTES;
            int s = 0, it = 0;
            unsigned phase = 0;
            bool ok = true;
            for (int t = pair; t < q.total_tiles && ok; t += num_pairs) {
                const PairTile p = decode_pair_tile(q, t, rank);
                if (p.idle) continue;
                const int a = it & 1;
                const unsigned aphase = (unsigned)(it >> 1) & 1u;
                // the epilogue of the tile that used this half two tiles ago must have drained it
                if (!__all_sync(0xffffffffu, mbar_wait_cluster(&acc_empty[a], aphase ^ 1u, q.error_flag))) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)a * 256u;
                for (int kb = 0; kb < p.num_kb; ++kb, s = (s + 1 == q.stages ? 0 : s + 1), phase ^= (s == 0)) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], phase, q.error_flag))) { ok = false; break; }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t st = smem_base + (uint32_t)s * (uint32_t)stage_bytes;
                        const uint64_t da0 = umma_desc(st, a_lbo, a_sbo, a_layout), dal0 = umma_desc(st + TC_TILE_BYTES, a_lbo, a_sbo, a_layout);
                        const uint64_t db0 = umma_desc(st + b_off, b_lbo, b_sbo, b_layout), dbl0 = umma_desc(st + b_off + TC_TILE_BYTES, b_lbo, b_sbo, b_layout);
#pragma unroll
                        for (int j = 0; j < TC_BK / TC_UK; ++j) {
                            const uint64_t da = da0 + j * a_jstep, db = db0 + j * b_jstep;
                            // (a 128-byte row holds four K = 8 steps of f32 or four K = 16 steps of f16 / bf16: same descriptors)
                            if (q.half) umma_f16_pair(acc, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                            else umma_tf32_pair(acc, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                            if (q.three_pass) {
                                umma_tf32_pair(acc, dal0 + j * a_jstep, db, idesc, 1u);
                                umma_tf32_pair(acc, da, dbl0 + j * b_jstep, idesc, 1u);
                            }
                        }
                        umma_commit_pair(&empty_bar[s]);
                    }
                    __syncwarp();
                }
                if (!ok) break;
                if (elect_one()) umma_commit_pair(&acc_full[a]);
                __syncwarp();
                ++it;
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32*(warp%4) .. +31 of this CTA ----
        const int quarter = warp & 3;
        int it = 0;
        for (int t = pair; t < q.total_tiles; t += num_pairs) {
            const PairTile p = decode_pair_tile(q, t, rank);
            if (p.idle) continue;
            const int a = it & 1;
            const unsigned aphase = (unsigned)(it >> 1) & 1u;
            if (!mbar_wait_warp(&acc_full[a], aphase, q.error_flag)) break;
            tc_fence_after();
            const long long row = p.m0 + quarter * 32 + lane;
            const long long crow_off = q.c_off + (long long)(q.splits > 1 ? p.zslot : p.bz) * q.c_sb + row * q.c_sm;
            float* crow = C + crow_off;
#pragma unroll 1
            for (int c = 0; c < 8; ++c) {
                float v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * 256 + c * 32), v);
                const long long col0 = p.n0 + c * 32;
                if (row >= q.m || col0 >= q.n) continue;
                if (q.c_dtype != EB200_F32) {
                    // C stored in the operands' 16-bit type: round to nearest even at the store
                    unsigned short* d16 = reinterpret_cast<unsigned short*>(C) + crow_off + col0 * q.c_sn;
                    if (q.c_sn == 1 && col0 + 32 <= q.n && (reinterpret_cast<uintptr_t>(d16) & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 w;
                            if (q.c_dtype == EB200_F16) {
                                *reinterpret_cast<__half2*>(&w.x) = __floats2half2_rn(v[i], v[i + 1]);
                                *reinterpret_cast<__half2*>(&w.y) = __floats2half2_rn(v[i + 2], v[i + 3]);
                                *reinterpret_cast<__half2*>(&w.z) = __floats2half2_rn(v[i + 4], v[i + 5]);
                                *reinterpret_cast<__half2*>(&w.w) = __floats2half2_rn(v[i + 6], v[i + 7]);
                            } else {
                                *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(v[i], v[i + 1]);
                                *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                                *reinterpret_cast<__nv_bfloat162*>(&w.z) = __floats2bfloat162_rn(v[i + 4], v[i + 5]);
                                *reinterpret_cast<__nv_bfloat162*>(&w.w) = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                            }
                            *reinterpret_cast<uint4*>(d16 + i) = w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < q.n)
                                d16[i * q.c_sn] = q.c_dtype == EB200_F16 ? __half_as_ushort(__float2half_rn(v[i]))
                                                                         : __bfloat16_as_ushort(__float2bfloat16_rn(v[i]));
                    }
                    continue;
                }
                float* dst = crow + col0 * q.c_sn;
                if (q.c_sn == 1 && col0 + 32 <= q.n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < q.n) dst[i * q.c_sn] = v[i];
                }
            }
            // this warp has read its lanes of the half: hand it back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&acc_empty[a]), 0));
            ++it;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}

// hi = x rounded to tf32 (low 13 mantissa bits zero), lo = x - hi (exact in f32).
__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ src, float* __restrict__ hi,
                                                         float* __restrict__ lo, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nvec = n >> 2;
    for (long long v = tid; v < nvec; v += stride) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(src) + v);
        float4 h, l;
        h.x = __uint_as_float((__float_as_uint(x.x) + 0x1000u) & 0xffffe000u); l.x = x.x - h.x;
        h.y = __uint_as_float((__float_as_uint(x.y) + 0x1000u) & 0xffffe000u); l.y = x.y - h.y;
        h.z = __uint_as_float((__float_as_uint(x.z) + 0x1000u) & 0xffffe000u); l.z = x.z - h.z;
        h.w = __uint_as_float((__float_as_uint(x.w) + 0x1000u) & 0xffffe000u); l.w = x.w - h.w;
        reinterpret_cast<float4*>(hi)[v] = h;
        reinterpret_cast<float4*>(lo)[v] = l;
    }
    for (long long i = (nvec << 2) + tid; i < n; i += stride) {
        const float x = src[i];
        const float h = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
        hi[i] = h;
        lo[i] = x - h;
    }
}


// Whether the tensor-core kernel can take this contraction (plan.cpp asks).
bool gemm_tc_supported(const GemmShape& g) {
    if (g.half) {
        // 16-bit operands: both contiguous along k; TMA wants 16-byte aligned rows (8 elements)
        auto mult8 = [](long long v) { return (v & 7) == 0; };
        if (g.a_sk != 1 || g.b_sk != 1 || g.a_sm <= 0 || g.b_sn <= 0) return false;
        if (!mult8(g.a_sm) || !mult8(g.a_sb) || !mult8(g.a_off) || !mult8(g.b_sn) || !mult8(g.b_sb) || !mult8(g.b_off)) return false;
        if (g.batch < 1 || g.batch > 65535 || (g.batch > 1 && (g.a_sb < 0 || g.b_sb < 0))) return false;
        if (g.m < 1 || g.n < 1 || g.k < 1 || g.m >= (1LL << 31) || g.n >= (1LL << 31) || g.k >= (1LL << 31)) return false;
        return true;
    }
    const bool a_kmajor = g.a_sk == 1, a_mmajor = g.a_sm == 1;
    if (!a_kmajor && !a_mmajor) return false;
    const bool b_kmajor = g.b_sk == 1, b_nmajor = g.b_sn == 1;
    if (!b_kmajor && !b_nmajor) return false;
    auto mult4 = [](long long v) { return (v & 3) == 0; };
    if (!mult4(a_kmajor ? g.a_sm : g.a_sk) || !mult4(g.a_sb) || !mult4(g.a_off)) return false;
    if (!mult4(b_kmajor ? g.b_sn : g.b_sk) || !mult4(g.b_sb) || !mult4(g.b_off)) return false;
    if ((a_kmajor ? g.a_sm : g.a_sk) <= 0 || (b_kmajor ? g.b_sn : g.b_sk) <= 0) return false;
    if (g.batch < 1 || g.batch > 65535) return false;
    if (g.m < 1 || g.n < 1 || g.k < 1) return false;
    if (g.m >= (1LL << 31) || g.n >= (1LL << 31) || g.k >= (1LL << 31)) return false;
    if ((g.m + TC_BM - 1) / TC_BM > 65535) return false;
    if (g.batch > 1 && (g.a_sb < 0 || g.b_sb < 0)) return false;
    return true;
}

// Elements of the memory span an operand covers (hi/lo copies mirror the span).
static long long span_of(long long batch, long long sb, long long rows, long long srow, long long inner) {
    return (batch - 1) * sb + (rows - 1) * srow + inner;
}

// 3xTF32 with the hi / lo split done inside the kernel (no scratch copies, no extra passes over the
// operands): for contractions that are short on arithmetic per operand byte, where the two pre-split
// passes cost more than the MMAs (an MLP layer [65536, 256] x [256, 256]: 64 flop per byte).
// Returns 0 (both operands pre-split), 3 (both split in the kernel) or 1 (A split in the kernel, B pre-split:
// when B is a small matrix every row tile re-reads -- a layer's weights -- one tiny pre-pass over it removes two
// thirds of the shared-memory traffic the in-kernel split costs per k block).
int gemm_tc_convert(const GemmShape& g, int flags) {
    if (g.mode != EB200_GEMM_3XTF32 || g.half) return 0;
    if (flags & 4096) return 0;          // descriptor flag bit 12: always split in a pre-pass
    if (flags & 8192) return 3;          // descriptor flag bit 13: always split inside the kernel
    const double flops = 2.0 * (double)g.batch * g.m * g.n * g.k;
    const double bytes = 4.0 * (double)g.batch * ((double)g.m * g.k + (double)g.k * g.n + (double)g.m * g.n);
    if (flops / bytes >= 200.0) return 0;
    long long a_span, b_span;
    gemm_tc_scratch(g, &a_span, &b_span);
    if (g.splits == 1 && b_span <= (1LL << 20) && b_span * 16 <= a_span) return 1;
    return 3;
}

void gemm_tc_scratch(const GemmShape& g, long long* a_span, long long* b_span) {
    const bool b_kmajor = g.b_sk == 1;
    long long a = g.a_sk == 1 ? span_of(g.batch, g.a_sb, g.m, g.a_sm, g.k) : span_of(g.batch, g.a_sb, g.k, g.a_sk, g.m);
    long long b = b_kmajor ? span_of(g.batch, g.b_sb, g.n, g.b_sn, g.k) : span_of(g.batch, g.b_sb, g.k, g.b_sk, g.n);
    *a_span = (a + 63) / 64 * 64;
    *b_span = (b + 63) / 64 * 64;
}

// Every tensor-core GEMM kernel needs more dynamic shared memory than the default limit (set once per device).
static int configure_tc(Device* dev) {
    if (dev->tc_configured) return EB200_OK;
    EB_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    EB_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    EB_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc2p_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    EB_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc1p_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    EB_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc1p_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    dev->tc_configured = true;
    return EB200_OK;
}

// 16-bit operands (f16 / bf16), both contiguous along k, f32 accumulation in tensor memory: the persistent pair
// kernel with tcgen05.mma.kind::f16.  A 128-byte swizzled row holds 64 elements of k, so a k block is 64 deep and
// every stage feeds four K = 16 MMAs; everything else (ring, double-buffered accumulator, epilogue) is shared
// with the f32 path.  C is f32 or the operands' type.
static int launch_gemm_tc_half(Device* dev, const GemmShape& g, const float* a, const float* b, float* c) {
    const unsigned short* a_src = reinterpret_cast<const unsigned short*>(a) + g.a_off;
    const unsigned short* b_src = reinterpret_cast<const unsigned short*>(b) + g.b_off;
    EB_REQUIRE((reinterpret_cast<uintptr_t>(a_src) & 15) == 0 && (reinterpret_cast<uintptr_t>(b_src) & 15) == 0,
               EB200_ERR_INVALID, "GEMM operands must be 16-byte aligned");
    const CUtensorMapDataType dt = g.half == EB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ma, mb;
    const long long a_b = g.a_sb > 0 ? g.batch : 1, b_b = g.b_sb > 0 ? g.batch : 1;
    int st;
    if ((st = make_map16(&ma, a_src, dt, g.k, g.m, a_b, g.a_sm, g.a_sb, 128))) return st;
    if ((st = make_map16(&mb, b_src, dt, g.k, g.n, b_b, g.b_sn, g.b_sb, 128))) return st;
    TcParams q{};
    q.m = g.m; q.n = g.n; q.k = g.k;
    q.c_sm = g.c_sm; q.c_sn = g.c_sn; q.c_sb = g.c_sb; q.c_off = g.c_off;
    q.splits = 1;
    q.half = g.half; q.bke = 64; q.c_dtype = g.c_dtype;
    q.kb_per_split = (int)((g.k + 63) / 64);
    q.error_flag = dev->error_flag_dev;
    q.raster = 8;
    { const int st_cfg = configure_tc(dev); if (st_cfg) return st_cfg; }
    const int stage_bytes = 2 * TC_TILE_BYTES;
    q.stages = std::min(8, (196 * 1024) / stage_bytes);
    const size_t smem = (size_t)q.stages * stage_bytes + 1024 + 256;
    const long long tm2 = (g.m + 255) / 256, tn2 = (g.n + 255) / 256;
    const long long bands = (tm2 + q.raster - 1) / q.raster;
    q.tiles_n = (int)tn2;
    const long long per_z = bands * q.raster * tn2, total = per_z * g.batch;
    EB_REQUIRE(total < (1LL << 31), EB200_ERR_UNSUPPORTED, "too many GEMM tiles");
    q.tiles_per_z = (int)per_z;
    q.total_tiles = (int)total;
    const long long pairs = std::min<long long>(total, dev->prop.multiProcessorCount / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(pairs * 2), 1, 1);
    cfg.blockDim = dim3(TC_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int az = g.a_sb > 0 ? 1 : 0, bzm = g.b_sb > 0 ? 1 : 0;
    EB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc2p_kernel, ma, ma, mb, mb, q, c, az, bzm));
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

int launch_gemm_tc(Device* dev, const Plan& plan, const float* a, const float* b, float* c, void* scratch) {
    const GemmShape& g = plan.gemm;
    if (g.half) return launch_gemm_tc_half(dev, g, a, b, c);
    const bool three = g.mode == EB200_GEMM_3XTF32;
    const bool b_nmajor = !(g.b_sk == 1);
    const bool a_mmajor = !(g.a_sk == 1);
    const float* a_src = a + g.a_off;
    const float* b_src = b + g.b_off;
    EB_REQUIRE((reinterpret_cast<uintptr_t>(a_src) & 15) == 0 && (reinterpret_cast<uintptr_t>(b_src) & 15) == 0,
               EB200_ERR_INVALID, "GEMM operands must be 16-byte aligned");
    const float *a_hi = a_src, *a_lo = a_src, *b_hi = b_src, *b_lo = b_src;
    const int convert = three ? g.convert : 0;       // bit 0 / 1: A / B split inside the kernel
    if (three && convert != 3) {
        EB_REQUIRE(scratch, EB200_ERR_INVALID, "3xTF32 launched without scratch");
        long long a_span, b_span;
        gemm_tc_scratch(g, &a_span, &b_span);
        float* s = reinterpret_cast<float*>(scratch);
        const long long cap = (long long)dev->prop.multiProcessorCount * 16;
        if (!(convert & 1)) {
            float *ah = s, *al = s + a_span;
            s += 2 * a_span;
            const long long blocks = std::min(cap, (a_span / 4 + 255) / 256 + 1);
            const long long as = a_mmajor ? span_of(g.batch, g.a_sb, g.k, g.a_sk, g.m) : span_of(g.batch, g.a_sb, g.m, g.a_sm, g.k);
            split_tf32_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(a_src, ah, al, as);
            count_launch();
            a_hi = ah; a_lo = al;
        }
        if (!(convert & 2)) {
            float *bh = s, *bl = s + b_span;
            const long long blocks = std::min(cap, (b_span / 4 + 255) / 256 + 1);
            const long long bs = b_nmajor ? span_of(g.batch, g.b_sb, g.k, g.b_sk, g.n) : span_of(g.batch, g.b_sb, g.n, g.b_sn, g.k);
            split_tf32_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(b_src, bh, bl, bs);
            count_launch();
            b_hi = bh; b_lo = bl;
        }
        EB_CHECK_CUDA(cudaGetLastError());
    }
    CUtensorMap ma, mal, mb, mbl;
    const long long a_b = g.a_sb > 0 ? g.batch : 1, b_b = g.b_sb > 0 ? g.batch : 1;
    int st;
    if (a_mmajor) {
        if ((st = make_map(&ma, a_hi, g.m, g.k, a_b, g.a_sk, g.a_sb, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))) return st;
        if ((st = make_map(&mal, a_lo, g.m, g.k, a_b, g.a_sk, g.a_sb, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))) return st;
    } else {
        if ((st = make_map(&ma, a_hi, g.k, g.m, a_b, g.a_sm, g.a_sb, TC_BM))) return st;
        if ((st = make_map(&mal, a_lo, g.k, g.m, a_b, g.a_sm, g.a_sb, TC_BM))) return st;
    }
    // 256-wide tiles halve the L2 traffic per flop; keep 128 when that would
    // leave SMs idle
    const long long tiles_m = (g.m + TC_BM - 1) / TC_BM;
    int bn = (tiles_m * ((g.n + 255) / 256) * g.batch * g.splits >= 2LL * dev->prop.multiProcessorCount) ? 256 : 128;
    if (b_nmajor) {
        if ((st = make_map(&mb, b_hi, g.n, g.k, b_b, g.b_sk, g.b_sb, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))) return st;
        if ((st = make_map(&mbl, b_lo, g.n, g.k, b_b, g.b_sk, g.b_sb, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))) return st;
    } else {
        if ((st = make_map(&mb, b_hi, g.k, g.n, b_b, g.b_sn, g.b_sb, bn))) return st;
        if ((st = make_map(&mbl, b_lo, g.k, g.n, b_b, g.b_sn, g.b_sb, bn))) return st;
    }
    TcParams q{};
    q.m = g.m; q.n = g.n; q.k = g.k;
    q.c_sm = g.c_sm; q.c_sn = g.c_sn; q.c_sb = g.c_sb; q.c_off = g.c_off;
    q.b_nmajor = b_nmajor ? 1 : 0;
    q.a_mmajor = a_mmajor ? 1 : 0;
    q.splits = g.splits;
    q.kb_per_split = g.splits > 1 ? (int)(g.k_chunk / TC_BK) : (int)((g.k + TC_BK - 1) / TC_BK);
    float* c_out = c;
    if (g.splits > 1) {
        EB_REQUIRE(scratch, EB200_ERR_INVALID, "split-K launched without scratch");
        c_out = reinterpret_cast<float*>(scratch) + g.partial_off;     // dense [batch*splits][m][n]
        q.c_off = 0; q.c_sm = g.n; q.c_sn = 1; q.c_sb = g.m * g.n;
    }
    q.three_pass = three ? 1 : 0;
    q.half = 0; q.bke = TC_BK; q.c_dtype = EB200_F32;
    q.convert = convert;
    // two-CTA pairs (256 x 256 per pair) when there are enough pair tiles to fill the machine
    const long long pair_tiles = ((g.m + 255) / 256) * ((g.n + 255) / 256) * g.batch * g.splits;
    bool two_cta = g.m > 128 && pair_tiles * 2 >= dev->prop.multiProcessorCount;
    if (convert) two_cta = false;      // the in-kernel split lives in the one-CTA kernel
    q.error_flag = dev->error_flag_dev;
    q.raster = 8;
    { const int st_cfg = configure_tc(dev); if (st_cfg) return st_cfg; }
    const int az = g.a_sb > 0 ? 1 : 0, bzm = g.b_sb > 0 ? 1 : 0;
    if (two_cta) {
        // B maps were built for `bn`-row boxes when B is K-major; each CTA stages 128 columns
        if (!b_nmajor && bn != 128) {
            if ((st = make_map(&mb, b_hi, g.k, g.n, b_b, g.b_sn, g.b_sb, 128))) return st;
            if ((st = make_map(&mbl, b_lo, g.k, g.n, b_b, g.b_sn, g.b_sb, 128))) return st;
        }
        const int stage_bytes = (three ? 2 : 1) * 2 * TC_TILE_BYTES;
        q.stages = std::min(8, (196 * 1024) / stage_bytes);
        EB_REQUIRE(q.stages >= 2, EB200_ERR_UNSUPPORTED, "GEMM stage does not fit shared memory twice");
        const size_t smem = (size_t)q.stages * stage_bytes + 1024 + 256;
        const long long tm2 = (g.m + 255) / 256, tn2 = (g.n + 255) / 256;
        const long long bands = (tm2 + q.raster - 1) / q.raster;
        q.tiles_n = (int)tn2;
        const long long per_z = bands * q.raster * tn2, total = per_z * g.batch * g.splits;
        EB_REQUIRE(total < (1LL << 31), EB200_ERR_UNSUPPORTED, "too many GEMM tiles");
        q.tiles_per_z = (int)per_z;
        q.total_tiles = (int)total;
        // one CTA pair per SM pair, each walking tiles pair, pair + P, ...
        const long long pairs = std::min<long long>(total, dev->prop.multiProcessorCount / 2);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(pairs * 2), 1, 1);
        cfg.blockDim = dim3(TC_THREADS, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = dev->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        EB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc2p_kernel, ma, mal, mb, mbl, q, c_out, az, bzm));
    } else {
        const int stage_bytes = (three ? 2 : 1) * (TC_TILE_BYTES + bn * TC_BK * 4);
        q.stages = std::min(8, (196 * 1024) / stage_bytes);
        const size_t smem = (size_t)q.stages * stage_bytes + 1024 /* alignment */ + 256 /* barriers */;
        const long long tiles_n = (g.n + bn - 1) / bn;
        const long long bands = (tiles_m + q.raster - 1) / q.raster;
        q.tiles_n = (int)tiles_n;
        // grid.x walks bands x (raster x tiles_n) slots; the last band may be padded
        const long long per_z = bands * q.raster * tiles_n, total = per_z * g.batch * g.splits;
        if (convert && total < (1LL << 31)) {
            // split inside the kernel: the persistent form (split warps work ahead while the epilogue drains)
            q.tiles_per_z = (int)per_z;
            q.total_tiles = (int)total;
            const unsigned ctas = (unsigned)std::min<long long>(total, dev->prop.multiProcessorCount);
            if (bn == 256) gemm_tc1p_kernel<256><<<ctas, TC1P_THREADS, smem, dev->stream>>>(ma, mal, mb, mbl, q, c_out, az, bzm);
            else gemm_tc1p_kernel<128><<<ctas, TC1P_THREADS, smem, dev->stream>>>(ma, mal, mb, mbl, q, c_out, az, bzm);
        } else {
            dim3 grid((unsigned)(bands * q.raster * tiles_n), 1, (unsigned)(g.batch * g.splits));
            if (bn == 256) gemm_tc_kernel<256><<<grid, TC_THREADS, smem, dev->stream>>>(ma, mal, mb, mbl, q, c_out, az, bzm);
            else gemm_tc_kernel<128><<<grid, TC_THREADS, smem, dev->stream>>>(ma, mal, mb, mbl, q, c_out, az, bzm);
        }
    }
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    if (g.splits > 1) return launch_splitk_reduce(dev, g, c_out, c);
    return EB200_OK;
}

}  // namespace eb200
