// Internal declarations shared by the translation units of libeb200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/eb200.h"

namespace eb200 {

// ---- error reporting --------------------------------------------------------
int set_error(int status, const char* fmt, ...);
void clear_error();

#define EB_CHECK_CUDA(expr)                                                        \
    do {                                                                           \
        cudaError_t _e = (expr);                                                   \
        if (_e != cudaSuccess) {                                                   \
            return ::eb200::set_error(                                             \
                _e == cudaErrorMemoryAllocation ? EB200_ERR_OOM : EB200_ERR_CUDA,  \
                "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__,  \
                __LINE__);                                                         \
        }                                                                          \
    } while (0)

#define EB_REQUIRE(cond, status, ...)                    \
    do {                                                 \
        if (!(cond)) return ::eb200::set_error(status, __VA_ARGS__); \
    } while (0)

extern std::atomic<int64_t> g_launch_count;
inline void count_launch(int n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }

// ---- device-side parameter block ---------------------------------------------
// What every generic kernel receives by value: the collapsed iteration space,
// operand addressing, bound conditions and the map program.
constexpr int KMAX_DIMS = EB200_MAX_DIMS;
constexpr int KMAX_IN = EB200_MAX_INPUTS;
constexpr int KMAX_BOUNDS = 8;   // total over all operands
constexpr int KMAX_INSNS = EB200_MAX_INSNS;
constexpr int KMAX_CONSTS = 32;
constexpr int KSTACK = 16;       // evaluation stack depth of the interpreter

struct KOperand {
    char* ptr;                 // set at launch
    long long offset;          // elements
    long long strides[KMAX_DIMS];
    int dtype;
    int bound_begin;
    int n_bounds;
    float pad;
    int flat;                  // f32, unmasked and laid out exactly like the iteration space: element e sits at offset + e
    long long delta[KMAX_DIMS]; // odometer steps: address change when dim d ticks and every dim after it wraps to 0
};

struct KBound {
    long long coef[KMAX_DIMS];
    long long c, lo, hi;
};

struct KInsn {
    short op;
    short arg;
    float imm;
};

struct KParams {
    int ndim;
    int n_in;
    int n_insns;
    int n_consts;
    long long shape[KMAX_DIMS];
    long long total;           // product of shape
    // reduce bookkeeping (collapsed coordinates)
    int raxis;                 // reduce dim, -1 if none
    int rop;
    long long rlen;            // shape[raxis]
    long long kept;            // total / rlen
    int splits;                // partial reductions over the reduce dim
    int vec;                   // 4 = 128-bit path legal, 1 = scalar
    long long chunk;           // reduce-dim elements per split
    KOperand in[KMAX_IN];
    KOperand out;
    KBound bounds[KMAX_BOUNDS];
    KInsn prog[KMAX_INSNS];
    float consts[KMAX_CONSTS];
    const float* cptr[KMAX_CONSTS];  // non-null: constant slot is read from a one-element tensor
    unsigned dmul[KMAX_DIMS];        // exact division of a 31-bit index by shape[d]: (n * dmul) >> dshr
    unsigned dshr[KMAX_DIMS];
    int tuning;                      // copy of the descriptor's flags
    int _pad1;
    int* error_flag;                 // host-mapped word a kernel raises when a bounded wait runs out (may be null)
};

// ---- host objects ------------------------------------------------------------
struct Device {
    int index = 0;
    cudaStream_t stream = nullptr;
    cudaMemPool_t pool = nullptr;
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
    cudaDeviceProp prop{};
    std::atomic<int64_t> in_use{0}, peak{0}, n_allocs{0};
    // raised by a kernel whose bounded device-side wait ran out (host-mapped, pinned)
    int* error_flag_host = nullptr;
    int* error_flag_dev = nullptr;
    bool tc_configured = false;
    bool conv_configured = false;
};

// Reference-counted device storage; several buffer handles may share one
// storage until one of them is written (copy-on-write clone).
struct Storage {
    Device* dev = nullptr;
    void* ptr = nullptr;
    size_t bytes = 0;
    ~Storage();
};

int storage_alloc(Device* dev, size_t bytes, bool zero, std::shared_ptr<Storage>* out);

}  // namespace eb200

struct eb200_device : eb200::Device {};

struct eb200_buffer {
    std::atomic<int> refs{1};
    eb200::Device* dev = nullptr;
    size_t bytes = 0;
    std::shared_ptr<eb200::Storage> storage;
};

namespace eb200 {

// Makes `buf` the only owner of its storage.  `keep_contents` copies the old
// bytes device-to-device; otherwise the new storage is left uninitialised.
int buffer_unshare(eb200_buffer* buf, bool keep_contents);

// ---- kernel plans -------------------------------------------------------------
enum Impl {
    IMPL_EW = 0,          // fused elementwise chain, 128-bit vectorised
    IMPL_REDUCE_INNER,    // reduce over the contiguous innermost dim (row reduce)
    IMPL_REDUCE_OUTER,    // reduce over a strided dim (column reduce) + generic fallback
    IMPL_TRANSPOSE,       // batched 2-D transpose through shared memory
    IMPL_SCATTER,         // zero fill + red.global.add
    IMPL_FOLD_GATHER,     // scatter-add of sliding windows (fold) as a gather over the output: deterministic, no atomics
    IMPL_SGD,             // p - lr*g
    IMPL_GEMM_SIMT,       // dense contraction, fp32 FFMA tiles (exact-f32 fallback)
    IMPL_GEMM_TC,         // dense contraction, tcgen05 TF32 / 3xTF32
    IMPL_CONV2D,          // convolution as implicit GEMM on the tensor cores
    IMPL_CONV2D_DIRECT,   // convolution with a tiny reduction (C*KH*KW <= 32): streaming FFMA kernel
    IMPL_CONV2D_DIRECT_WGRAD,
    IMPL_CONV2D_WGRAD,    // weight gradient of a convolution, positions contracted on the tensor cores
    IMPL_GEMM_TALL,       // one-tile output, reduction over millions of rows (small-layer weight gradients)
    IMPL_SCAN,            // cumulative op along an axis (P_ kernels)
    IMPL_SGD_MOMENTUM,    // v = momentum*v - lr*g; p += v
    IMPL_ADAM,            // Adam step with device-resident moments and step counter
    IMPL_SOFTMAX_XENT,    // log-softmax + cross-entropy, loss and logits gradient in one kernel
    IMPL_SIBLINGS,        // row reduce + column max + transposing copy of one [R, C] tensor in one pass
    IMPL_MAXPOOL,         // max_pool2d (stride = window) forward or gradient, optional fused ReLU
};

struct GemmShape {
    // C[b][m][n] = sum_k A[b][m][k] * B[b][k][n]; element strides
    long long batch = 1, m = 0, n = 0, k = 0;
    long long a_sb = 0, a_sm = 0, a_sk = 0, a_off = 0;
    long long b_sb = 0, b_sk = 0, b_sn = 0, b_off = 0;
    long long c_sb = 0, c_sm = 0, c_sn = 0, c_off = 0;
    int a_input = 0, b_input = 1;  // which kernel input is A / B
    int mode = EB200_GEMM_3XTF32;
    int splits = 1;            // split-K: partial products go to scratch and are summed by a second kernel
    long long k_chunk = 0;     // k extent per split (multiple of 32)
    long long partial_off = 0; // float offset of the partials inside the kernel's scratch
    int half = 0;              // 0: f32 operands; EB200_F16 / EB200_BF16: 16-bit operands (tcgen05 kind::f16, f32 accumulate)
    int c_dtype = EB200_F32;   // storage type of C (f32, or the operands' 16-bit type)
    int convert = 0;           // 3xTF32: bit 0 / bit 1 = A / B split into hi / lo inside the kernel; a clear bit = by a pre-pass into scratch copies; fixed at plan time
};

struct ConvShape {
    int N = 0, C = 0, H = 0, W = 0, Co = 0, KH = 0, KW = 0, pad = 0;
    int relu = 0, mode = EB200_GEMM_3XTF32, has_bias = 0, flip = 0, wgrad = 0, nchw = 0, g_nchw = 0, direct = 0;
};

struct TransposeShape {
    // out[b][r][c] (contiguous) = in[b*sb + c*sc + r]  (input contiguous along r)
    long long batch = 1, rows = 0, cols = 0;
    long long in_sb = 0, in_sc = 0, in_off = 0;
    long long out_sb = 0, out_off = 0;
    int esize = 4;
};

struct Plan {
    Impl impl = IMPL_EW;
    KParams p{};
    int chain = -1;           // index into the compiled-functor table, -1 = interpreter
    int threads_per_row = 0;  // REDUCE_INNER: 1, 32 or 256
    GemmShape gemm;
    ConvShape conv;
    bool narrow = false;          // outer reduce with few kept elements: column threads x row lanes
    long long sib_rows = 0, sib_cols = 0;   // IMPL_SIBLINGS: the shared [R, C] operand
    long long pool[4] = {0, 0, 0, 0};       // IMPL_MAXPOOL: planes, H, W, window
    // IMPL_FOLD_GATHER: the last four iteration dims are (Ho, Wo, KH, KW); output row pitch, window strides / dilations
    int scatter_plain = 0;                  // IMPL_SCATTER: the windows are disjoint, stores instead of atomic adds
    long long fold_pitch = 0;
    int fold_sh = 0, fold_sw = 0, fold_dh = 0, fold_dw = 0, fold_hout = 0, fold_wout = 0;
    int pool_flags = 0;                     // IMPL_MAXPOOL: 1 = ReLU on the taps, 2 = gradient
    TransposeShape tr;
    int64_t scratch_bytes = 0;
    bool scratch_zero = false;    // the scratch must start at zero (set once, at kernel creation)
    int64_t algo_bytes = 0, algo_flops = 0;
    int launches = 1;
    float scalar = 0.f;
    float hyper[7] = {0};     // optimizer hyper-parameters of the descriptor
    int n_inputs = 0;         // inputs of the descriptor
    int perm[KMAX_IN] = {0};  // kernel operand c is descriptor input perm[c]
    int dyn_input[KMAX_CONSTS];   // constant slot j is read from descriptor input dyn_input[j] (-1: literal)
    long long dyn_offset[KMAX_CONSTS] = {0};
    int in_dtype[KMAX_IN] = {0};
    int64_t in_numel[KMAX_IN] = {0};
    int out_dtype = 0;
    int64_t out_numel = 0;
    char name[64] = {0};
};

// plan.cpp: validate + normalise + classify.  Pure host logic, no CUDA calls.
int build_plan(const eb200_kernel_desc* d, int sm_count, Plan* plan);

// chains: compiled functors for known map programs (chains.cu)
int find_chain(const KInsn* prog, int n_insns);
int chain_count();
const char* chain_name(int chain);

// launchers (one per .cu)
int launch_ew(Device* dev, const Plan& plan, const KParams& p);
int launch_reduce(Device* dev, const Plan& plan, const KParams& p, void* scratch, bool finish = true);
int launch_transpose(Device* dev, const Plan& plan, const void* in, void* out);
int launch_scatter(Device* dev, const Plan& plan, const KParams& p);
int launch_fold_gather(Device* dev, const Plan& plan, const KParams& p);
int launch_sgd(Device* dev, const Plan& plan, const float* p, const float* g, float* out, long long n);
int launch_sgd_momentum(Device* dev, const Plan& plan, const float* p, const float* g, float* v, float* out, long long n);
int launch_adam(Device* dev, const Plan& plan, const float* p, const float* g, float* m, float* v, int* t, float* out,
                long long n, void* scratch);
int launch_softmax_xent(Device* dev, const Plan& plan, const float* logits, const float* onehot, float* out, void* scratch);
long long scan_scratch_floats(const KParams& p, int sms);
long long siblings_scratch_floats(long long R, long long C);
int launch_maxpool(Device* dev, const Plan& plan, const float* a, const float* b, const float* c, float* out);
int launch_siblings(Device* dev, const Plan& plan, const KParams& p, const float* x, float* out, void* scratch);
int launch_scan(Device* dev, const Plan& plan, const KParams& p, void* scratch);
int launch_gemm_simt(Device* dev, const Plan& plan, const float* a, const float* b, float* c, void* scratch);
int launch_splitk_reduce(Device* dev, const GemmShape& g, const float* partials, float* c);
bool gemm_tc_supported(const GemmShape& g);
void gemm_tc_scratch(const GemmShape& g, long long* a_span, long long* b_span);
int gemm_tc_convert(const GemmShape& g, int flags);
int launch_gemm_tc(Device* dev, const Plan& plan, const float* a, const float* b, float* c, void* scratch);
bool gemm_tall_supported(const GemmShape& g);
int launch_gemm_tall(Device* dev, const Plan& plan, const float* a, const float* b, float* c, void* scratch);
bool conv2d_supported(const ConvShape& c);
bool conv2d_wgrad_supported(const ConvShape& c);
bool conv2d_direct_supported(const ConvShape& c);
long long conv2d_direct_wgrad_scratch_floats(const ConvShape& c, int sms);
int launch_conv2d_direct(Device* dev, const Plan& plan, const float* x, const float* w, const float* bias, float* out);
int launch_conv2d_direct_wgrad(Device* dev, const Plan& plan, const float* x, const float* g, float* dw, void* scratch);
long long conv2d_wgrad_scratch_floats(const ConvShape& c, int sms);
int launch_conv2d_wgrad(Device* dev, const Plan& plan, const float* x, const float* g, float* dw, void* scratch);
long long conv2d_scratch_floats(const ConvShape& c);
int launch_conv2d(Device* dev, const Plan& plan, const float* x, const float* w, const float* bias, float* out, void* scratch);
// comm.cu: collectives used by kernels that carry an attached communicator
bool comm_can_fuse(eb200_comm* c, long long count);
int comm_reduce_finish_allreduce(eb200_comm* c, const float* partials, int splits, long long kept, int rop, float* out);
int comm_allreduce_buffer(eb200_comm* c, float* data, long long count, int rop);
// EB200_ERR_TIMEOUT if a kernel on this device reported a timed-out wait (clears the flag)
int check_device_flag(Device* dev);

}  // namespace eb200

struct eb200_kernel {
    std::atomic<int> refs{1};
    eb200::Device* dev = nullptr;
    eb200::Plan plan;
    std::shared_ptr<eb200::Storage> scratch;
    eb200_comm* comm = nullptr;   // set: the output is all-reduced over the ranks as part of the launch
};
