// PTX wrappers and host helpers shared by the tensor-core kernels (GEMM, implicit-GEMM
// convolution): mbarriers, TMA tile loads, tensor-memory allocation, tcgen05.mma /
// commit / ld, shared-memory matrix descriptors, tensor-map encoding.
#pragma once

#include <cuda.h>

#include "common.h"

namespace eb200 {

constexpr int TC_BM = 128, TC_BK = 32;   // tile rows; BK floats = one 128-byte swizzle row (tile columns BN = 128 or 256)
constexpr int TC_UK = 8;                               // K of one tf32 MMA
constexpr int TC_TILE_BYTES = TC_BM * TC_BK * 4;       // 16 KB per operand tile
constexpr int TC_THREADS = 192;                        // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr unsigned TC_SPIN_LIMIT = 1u << 24;

// ---- PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// One lane of a converged warp.  elect.sync (rather than lane == 0) lets the compiler keep
// warp-uniform operands of what the elected lane issues in uniform registers.
__device__ __forceinline__ bool elect_one() {
    unsigned pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
// Warp index the compiler can prove warp-uniform.
__device__ __forceinline__ int uniform_warp_idx() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }

// Bounded wait; false when the bound was hit (the caller must bail out).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, int* error_flag) {
    for (unsigned i = 0; i < TC_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 4096) __nanosleep(64);
    }
    atomicExch(error_flag, 1);
    return false;
}

// The same for a whole (converged) warp: lane 0 polls, the others wait at the warp
// barrier, so that a barrier word is polled by one thread per warp instead of 32.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, unsigned parity, int* error_flag) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, error_flag) ? 1 : 0;
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}

// Contiguous bulk copy global -> shared (16-byte aligned both sides, size a multiple of 16).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::tf32, issued by one thread.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// mbarrier arrives once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 columns of f32 from tensor memory: thread t of the warp gets lane t.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, version 1, 128-byte swizzle.
// layout 2 = 128-byte swizzle of 16-byte chunks; layout 1 = 128-byte swizzle of
// 32-byte chunks, the only layout the tensor core accepts for MN-major tf32.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout = 2) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version
    d |= (uint64_t)layout << 61;
    return d;
}

// Instruction descriptor for kind::tf32: f32 accumulate, tf32 A and B, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N, int a_mmajor, int b_nmajor) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a_mmajor ? 1 : 0) << 15) | ((uint32_t)(b_nmajor ? 1 : 0) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- host helpers -----------------------------------------------------------------------
// ---- host side --------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 3-D f32 tensor map: dims {inner, rows, batch}, byte strides of dims 1 and 2, box {32, box_rows, 1}.
static inline int make_map(CUtensorMap* map, const float* base, long long inner, long long rows, long long batch,
                    long long row_stride, long long batch_stride, int box_rows,
                    CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    EncodeTiledFn fn = encode_fn();
    EB_REQUIRE(fn, EB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)row_stride * 4, (cuuint64_t)(batch_stride > 0 ? batch_stride : row_stride * rows) * 4};
    cuuint32_t box[3] = {32, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    EB_REQUIRE(r == CUDA_SUCCESS, EB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (inner %lld rows %lld stride %lld)",
               (int)r, inner, rows, row_stride);
    return EB200_OK;
}

// 16-bit elements (f16 / bf16), K-major: boxes of 64 elements (one 128-byte swizzled row) x box_rows rows.
static inline int make_map16(CUtensorMap* map, const void* base, CUtensorMapDataType dt, long long inner, long long rows, long long batch,
                             long long row_stride, long long batch_stride, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    EB_REQUIRE(fn, EB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)(batch_stride > 0 ? batch_stride : row_stride * rows) * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    EB_REQUIRE(r == CUDA_SUCCESS, EB200_ERR_CUDA, "cuTensorMapEncodeTiled (16-bit) failed with %d (inner %lld rows %lld stride %lld)",
               (int)r, inner, rows, row_stride);
    return EB200_OK;
}

// General 3-D f32 tensor map without swizzle: dims/box innermost first, byte strides of dims 1 and 2.
static inline int make_map_plain(CUtensorMap* map, const float* base, const cuuint64_t dims[3], const cuuint64_t strides[2],
                                 const cuuint32_t box[3]) {
    EncodeTiledFn fn = encode_fn();
    EB_REQUIRE(fn, EB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    EB_REQUIRE(r == CUDA_SUCCESS, EB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (dims %llu %llu %llu box %u %u %u)", (int)r,
               (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2], box[0], box[1], box[2]);
    return EB200_OK;
}

void launch_split_tf32(Device* dev, const float* src, float* hi, float* lo, long long n);

}  // namespace eb200
