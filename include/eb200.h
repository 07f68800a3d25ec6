/*
 * eb200.h -- C ABI of the B200-native execution backend for eclat (uthree/harp).
 *
 * This is the drop-in boundary: what an eclat backend crate (a
 * `BackendRegistry` + `Device` + `Buffer` + `Kernel` implementation, the role
 * crates/backend-c and crates/backend-cuda play in the reference) binds over
 * FFI.  Everything is `extern "C"`, plain pointers and sizes; no torch, no C++
 * types.  Every call returns an `eb200_status` (0 = ok); the message of the
 * last failure on the calling thread is available from `eb200_last_error()`.
 *
 * The reference hands a backend one lowered `AstNode::Kernel` at a time
 * (src/backend/executor.rs:323-354).  Its information content -- a loop nest
 * over an iteration shape, affine loads with optional bounds masks, a `map`
 * expression, an optional reduce, one store -- is carried here by
 * `eb200_kernel_desc`.  `eb200_kernel_create` classifies the descriptor and
 * selects a pre-built, hand-written sm_100a kernel; there is no source
 * generation, no runtime compiler and no CPU fallback: a descriptor no kernel
 * class serves fails with EB200_ERR_UNSUPPORTED.
 */
#ifndef EB200_H
#define EB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EB200_ABI_VERSION 2

#define EB200_MAX_DIMS 8     /* iteration-space rank (reference tensors are D0..D8) */
#define EB200_MAX_INPUTS 8   /* the C backend caps a kernel at 6 pointers; fused chains may need more */
#define EB200_MAX_BOUNDS 4   /* affine bound conditions per operand (padded views) */
#define EB200_MAX_INSNS 96   /* postfix map program length */

typedef enum {
    EB200_OK = 0,
    EB200_ERR_INVALID = 1,      /* bad argument / malformed descriptor / size mismatch */
    EB200_ERR_UNSUPPORTED = 2,  /* no hand-written kernel class serves this descriptor */
    EB200_ERR_CUDA = 3,         /* a CUDA runtime call failed */
    EB200_ERR_OOM = 4,          /* device allocation failed */
    EB200_ERR_BOUNDS = 5,       /* descriptor would index outside a buffer */
    EB200_ERR_COMM = 6,         /* collective layer failure */
    EB200_ERR_TIMEOUT = 7,      /* a bounded device-side wait ran out */
    EB200_ERR_NO_DEVICE = 8     /* no usable sm_100 device */
} eb200_status;

/* Storage types.  Bool is stored as one byte, like the reference's
 * `unsigned char` (crates/backend-c/src/renderer.rs:117-121). */
typedef enum {
    EB200_F32 = 0,
    EB200_BOOL = 1,
    EB200_I32 = 2,
    EB200_I64 = 3,
    EB200_F16 = 4,    /* IEEE binary16, the reference's `_Float16` (crates/backend-c/src/renderer.rs:129) */
    EB200_BF16 = 5    /* bfloat16, the reference's `__bf16` (crates/backend-c/src/renderer.rs:130) */
} eb200_dtype;
/* 16-bit types are STORAGE types: elements are widened to f32 when loaded, all arithmetic and every
 * accumulator is f32, results are rounded to nearest even when stored. */

/* Kernel classes the lowerer emits (src/lowerer/lower.rs:335-388). */
typedef enum {
    EB200_K_ELEMENTWISE = 0, /* E_: lower_elementwise, lower.rs:504-522 */
    EB200_K_REDUCE = 1,      /* R_: lower_reduce, lower.rs:525-571 */
    EB200_K_COPY = 2,        /* C_: lower_view, lower.rs:448-501 */
    EB200_K_SCATTER = 3,     /* S_: lower_scatter, lower.rs:580-683 */
    EB200_K_SGD = 4,         /* p <- p - lr*g (crates/nn/src/optim/sgd.rs:73-103), device resident */
    EB200_K_CONV2D = 5,      /* functional::conv2d as one kernel (crates/nn/src/functional/conv.rs:113-184):
                              * shape = {N, C, H, W, Co, KH, KW, pad}; inputs x [N,C,H,W], w [Co,C,KH,KW] and
                              * optionally bias [Co], all contiguous; output [N*Ho*Wo, Co] row-major (the buffer
                              * the reference's GEMM step writes before its final permute view); stride 1;
                              * flags bit 6 = ReLU in the epilogue; flags bit 7 = the weight buffer is the FORWARD
                              * layer's [C, Co, KH, KW] and is read transposed and flipped, w'[co][c][kh][kw] =
                              * w[c][co][KH-1-kh][KW-1-kw]: with pad' = KH-1-pad this is the input gradient of the
                              * forward convolution (the VJP eclat derives through fold, src/grad/rules.rs:40-53);
                              * flags bit 10 = (weight gradient) the output gradient is given as [N, Co, Ho, Wo]; served for
                              * C*KH*KW <= 12 only; flags bit 11 = keep a layer with C*KH*KW <= 32 on the tensor-core kernel
                              * (such layers otherwise run a streaming f32 FFMA kernel);
                              * flags bit 9 = write the output as [N, Co, Ho, Wo] (the layout of the function's result)
                              * instead of [N*Ho*Wo, Co];
                              * flags bit 8 = weight gradient: inputs are x and the output gradient [N*Ho*Wo, Co],
                              * the output is dW [Co, C, KH, KW] (the contraction the reference spells as a broadcast
                              * multiply of the gradient with the materialised unfold, summed over batch and positions);
                              * gemm_mode picks TF32 / 3xTF32 */
    EB200_K_SCAN = 6,        /* P_: lower_scan, lower.rs:691-735; loops loop_gen.rs:237-327.  reduce_op / reduce_axis
                              * name the scan.  As in the reference's loop nest, ONE accumulator per index of the dims
                              * before the axis runs over the axis and every dim after it in row-major order (a plain
                              * cumulative op when the axis is innermost); the output has the iteration shape */
    EB200_K_SGD_MOMENTUM = 7,/* v <- momentum*v - lr*g; p <- p + v (crates/nn/src/optim/sgd.rs:84-89): inputs p, g, v;
                              * the output receives p, input 2 (v) is updated IN PLACE; scalar = lr, hyper[0] = momentum */
    EB200_K_SOFTMAX_XENT = 9,/* log_softmax (crates/nn/src/functional/activation.rs:174-187) + cross_entropy_loss
                              * (crates/nn/src/functional/loss.rs:32-65) forward AND backward as one kernel:
                              * shape = {N, C}; inputs logits [N, C] and the one-hot targets [N, C], contiguous;
                              * output [64 + N*C]: element 0 = scalar * sum(onehot * log_softmax(logits)), elements
                              * 64.. = its gradient with respect to the logits, scalar * (onehot - softmax *
                              * rowsum(onehot)); scalar = the loss scale (-1/N for the mean) */
    EB200_K_MAXPOOL2D = 10,  /* functional::max_pool2d with stride = window (crates/nn/src/functional/pool.rs:117-160: unfold,
                              * max over the window) as one kernel, and its VJP as one kernel: shape = {P, H, W, k} with
                              * P = N*C planes; forward: input x [P, H, W], output y [P, H/k, W/k] (floor: rows / columns
                              * no window covers are not read), the window folded as max(max(t0, t1), ...) in row-major
                              * tap order; flags bit 6 = the taps are max(x, 0) (a ReLU the function was applied to);
                              * flags bit 7 = gradient: inputs g [P, H/k, W/k], x [P, H, W], y [P, H/k, W/k] (the forward
                              * result), output gx [P, H, W] = (tap < y ? 0 : g) on covered elements (every element that
                              * equals its window's maximum receives the gradient, the mask-times-gradient of
                              * src/grad/rules.rs:379-399 folded back), 0 elsewhere; with bit 6 also the ReLU's own
                              * gradient mask, gx = x < 0 ? 0 : gx.  All operands contiguous f32 */
    EB200_K_ADAM = 8         /* Adam::step (crates/nn/src/optim/adam.rs:104-147): inputs p, g, m, v and a one-element
                              * I32 step counter t; the output receives p; m, v and t are updated IN PLACE (t <- t + 1
                              * on the device, so a captured step can be replayed); scalar = lr, hyper[0..2] = beta1,
                              * beta2, eps; bias corrections 1 - beta^t use the repeated-squaring powi of f32::powi */
} eb200_kclass;

/* ReduceOp (src/graph/node.rs:29-77). */
typedef enum {
    EB200_R_NONE = 0,
    EB200_R_SUM = 1,
    EB200_R_MAX = 2,
    EB200_R_MIN = 3,
    EB200_R_PROD = 4
} eb200_reduce_op;

/* Postfix opcodes = the AST primitive set a `map` may contain
 * (src/ast/mod.rs:107-385; rendering src/backend/renderer.rs:268-441).
 * Values are f32 on the evaluation stack; comparisons and logic produce
 * 1.0f / 0.0f; Select pops (cond, then, else). */
typedef enum {
    EB200_OP_LOAD = 0,   /* push inputs[arg] at the current index (Wildcard) */
    EB200_OP_CONST = 1,  /* push imm */
    EB200_OP_ADD = 2,
    EB200_OP_MUL = 3,
    EB200_OP_MAX = 4,
    EB200_OP_RECIP = 5,  /* 1.0f / x */
    EB200_OP_SQRT = 6,
    EB200_OP_LOG2 = 7,
    EB200_OP_EXP2 = 8,
    EB200_OP_SIN = 9,
    EB200_OP_FLOOR = 10,
    EB200_OP_LT = 11,
    EB200_OP_AND = 12,
    EB200_OP_NOT = 13,
    EB200_OP_SELECT = 14,
    EB200_OP_REM = 15,   /* C `%` on truncated integers */
    EB200_OP_IDIV = 16,  /* C `/` on truncated integers */
    EB200_OP_CAST = 17,  /* arg = target eb200_dtype */
    EB200_OP_FMA = 18    /* pops (a, b, c) -> a*b+c (AstNode::Fma) */
} eb200_opcode;

typedef struct {
    int32_t op;   /* eb200_opcode */
    int32_t arg;  /* input index for LOAD, dtype for CAST */
    float imm;    /* value for CONST */
    int32_t _pad;
} eb200_insn;

/* One affine condition of a padded view: lo <= c + sum_d coef[d]*idx[d] < hi.
 * The reference carries these as `ViewBounds` conditions AND-ed together and
 * wraps the load in Select(cond, load, pad) (src/lowerer/lower.rs:1145-1157). */
typedef struct {
    int64_t coef[EB200_MAX_DIMS];
    int64_t c;
    int64_t lo;
    int64_t hi;
} eb200_bound;

/* One kernel parameter as the loop nest addresses it: element index =
 * offset + sum_d strides[d]*idx[d]   (src/lowerer/index_gen.rs:45-63). */
typedef struct {
    int32_t dtype;      /* eb200_dtype */
    int32_t n_bounds;   /* 0 = unmasked */
    int64_t offset;
    int64_t strides[EB200_MAX_DIMS];
    int64_t numel;      /* elements in the underlying buffer (for validation) */
    float pad_value;    /* value when a bound fails */
    int32_t _pad;
    eb200_bound bounds[EB200_MAX_BOUNDS];
} eb200_operand;

/* GEMM arithmetic mode for descriptors the classifier recognises as a dense
 * contraction (sum over a product of two broadcast views). */
typedef enum {
    EB200_GEMM_DEFAULT = 0,  /* library default: 3xTF32 (f32-faithful) */
    EB200_GEMM_TF32 = 1,     /* single tcgen05 kind::tf32 pass, ~1e-3 relative */
    EB200_GEMM_3XTF32 = 2    /* hi*hi + hi*lo + lo*hi split, ~1e-6 relative */
} eb200_gemm_mode;

typedef struct {
    int32_t kclass;       /* eb200_kclass */
    int32_t ndim;         /* rank of the iteration space, 0..EB200_MAX_DIMS */
    int64_t shape[EB200_MAX_DIMS];
    int32_t n_inputs;
    int32_t reduce_op;    /* eb200_reduce_op; NONE unless kclass == REDUCE */
    int32_t reduce_axis;  /* iteration dim that is reduced */
    int32_t n_insns;      /* 0 = identity map of input 0 (COPY / SCATTER) */
    int32_t gemm_mode;    /* eb200_gemm_mode */
    int32_t flags;        /* tuning hints, 0 = automatic; bits 0-2 force the row-reduce group (1 thread, 2 warp, 3 CTA, 4 half CTA, 5 eight lanes per row); bit 3 keeps a contraction on the f32 FFMA kernel; bit 4 disables split-K (and keeps a narrow column reduce on the thread-per-vector kernel); bit 5 stages long reduce rows through shared memory with bulk async copies; bits 6-11: see EB200_K_CONV2D; 3xTF32 contractions split their operands into hi / lo either inside the kernel or by a pre-pass into scratch copies, chosen from the arithmetic intensity: bit 12 forces the pre-pass, bit 13 the in-kernel split (same results bit for bit); bit 14 (REDUCE, sum over axis 1 of [R, C], one full-size contiguous f32 operand x, R and C multiples of 64): sibling fusion -- the kernel reads x once and writes, into an output of R + C + R*C elements (y and z padded to multiples of 64), y = this reduce, z = max(x, axis 0) and t = x transposed, the three roots a graph like config 2 realizes together */
    float   scalar;       /* optimizer kernels: learning rate */
    float   hyper[7];     /* optimizer kernels: further hyper-parameters (see eb200_kclass) */
    eb200_operand inputs[EB200_MAX_INPUTS];
    eb200_operand output; /* store address; for REDUCE the reduce-axis stride is ignored (index := 0) */
    eb200_insn prog[EB200_MAX_INSNS];
} eb200_kernel_desc;

typedef struct eb200_device eb200_device;
typedef struct eb200_buffer eb200_buffer;
typedef struct eb200_kernel eb200_kernel;
typedef struct eb200_comm eb200_comm;

typedef struct {
    char name[128];
    int32_t cc_major, cc_minor;
    int32_t sm_count;
    int32_t _pad;
    int64_t total_mem_bytes;
    int64_t l2_bytes;
    int64_t smem_per_block_optin;
} eb200_device_props;

typedef struct {
    char impl[64];          /* name of the selected hand-written kernel */
    int32_t launches;       /* device launches one kernel_launch issues */
    int32_t specialised;    /* 1 = map runs as a compiled functor, 0 = bytecode interpreter */
    int64_t scratch_bytes;  /* device scratch the kernel object holds */
    int64_t algo_bytes;     /* algorithmic bytes moved per launch (each operand touched once) */
    int64_t algo_flops;     /* algorithmic flops per launch (2MNK for contractions, else 0) */
} eb200_kernel_info;

/* ---- library ------------------------------------------------------------ */
int eb200_abi_version(void);
/* Message of the last failed call on this thread ("" if none). */
const char* eb200_last_error(void);

/* sizeof() of the four ABI structs as this library was compiled, so a binding
 * can verify its own layout before the first call. */
int eb200_abi_sizes(size_t* kernel_desc, size_t* operand, size_t* device_props, size_t* kernel_info);

/* ---- device: BackendRegistry::{is_available,list_devices,create_device}
 *      (src/backend/device.rs:85-97) and Device (src/backend/traits.rs:273-306) */
int eb200_device_count(int* count);
int eb200_device_open(int index, eb200_device** dev);
int eb200_device_close(eb200_device* dev);
int eb200_device_sync(eb200_device* dev);
int eb200_device_get_props(eb200_device* dev, eb200_device_props* props);
/* The cudaStream_t all of this device's work is ordered on (for interop). */
int eb200_device_stream(eb200_device* dev, void** stream);
/* Device-side timing on that stream: begin/end bracket launches with CUDA
 * events; end synchronises and returns elapsed milliseconds. */
int eb200_timer_begin(eb200_device* dev);
int eb200_timer_end(eb200_device* dev, float* ms);
/* Any number of timing points on the device stream: record events between
 * launches, read the elapsed time between two of them (synchronises on `b`). */
typedef struct eb200_event eb200_event;
int eb200_event_create(eb200_device* dev, eb200_event** ev);
int eb200_event_record(eb200_event* ev);
int eb200_event_elapsed_ms(eb200_event* a, eb200_event* b, float* ms);
int eb200_event_destroy(eb200_event* ev);
/* Side streams for copies that overlap compute (PCIe is full duplex: the upload
 * of the next batch, the kernels of this one and the download of the previous
 * results can all be in flight).  A side stream only carries copies; ordering
 * against the device's compute stream is explicit through events:
 *   eb200_event_record_on(ev, s)   record on a side stream (NULL = compute stream)
 *   eb200_stream_wait(dev, s, ev)  make `s` (NULL = compute stream) wait for ev */
typedef struct eb200_stream eb200_stream;
int eb200_stream_create(eb200_device* dev, eb200_stream** s);
int eb200_stream_destroy(eb200_stream* s);
int eb200_stream_sync(eb200_stream* s);
int eb200_stream_wait(eb200_device* dev, eb200_stream* s, eb200_event* ev);
int eb200_event_record_on(eb200_event* ev, eb200_stream* s);
int eb200_buffer_write_on(eb200_buffer* buf, const void* pinned_host, size_t bytes, eb200_stream* s);
int eb200_buffer_read_on(eb200_buffer* buf, void* pinned_host, size_t bytes, eb200_stream* s);
/* A whole step as one CUDA graph: launches issued on this thread between
 * graph_begin and graph_end are recorded instead of run, then replayed by
 * graph_launch with a single submission (the reference synchronises after every
 * kernel, crates/backend-cuda/src/kernel.rs:213-225).  Allocate every buffer
 * the step touches before graph_begin; buffer reads/writes and device_sync are
 * not allowed while recording. */
typedef struct eb200_graph eb200_graph;
int eb200_graph_begin(eb200_device* dev);
int eb200_graph_end(eb200_device* dev, eb200_graph** graph);
int eb200_graph_launch(eb200_graph* graph);
int eb200_graph_release(eb200_graph* graph);
/* Pool statistics: bytes currently handed out, high-water mark, allocations. */
int eb200_device_mem_stats(eb200_device* dev, int64_t* in_use, int64_t* peak, int64_t* n_allocs);

/* ---- buffers: BackendRegistry::allocate_buffer (src/backend/device.rs:116-121)
 *      and Buffer (src/backend/traits.rs:455-482).  Allocation is zero-filled
 *      like CBuffer (crates/backend-c/src/buffer.rs:84-93). */
int eb200_buffer_alloc(eb200_device* dev, size_t bytes, eb200_buffer** buf);
/* Same without the zero fill, for callers that know the next kernel
 * overwrites every element. */
int eb200_buffer_alloc_uninit(eb200_device* dev, size_t bytes, eb200_buffer** buf);
int eb200_buffer_retain(eb200_buffer* buf);
int eb200_buffer_release(eb200_buffer* buf);
int eb200_buffer_bytes(eb200_buffer* buf, size_t* bytes);
/* write_from_host / read_to_host: `bytes` must equal the buffer size
 * (crates/backend-c/src/buffer.rs:151-160); read orders after prior launches. */
int eb200_buffer_write(eb200_buffer* buf, const void* host, size_t bytes);
int eb200_buffer_read(eb200_buffer* buf, void* host, size_t bytes);
/* Asynchronous forms for pinned host memory; complete at eb200_device_sync. */
int eb200_buffer_write_async(eb200_buffer* buf, const void* pinned_host, size_t bytes);
int eb200_buffer_read_async(eb200_buffer* buf, void* pinned_host, size_t bytes);
/* clone_buffer (traits.rs:475): a value copy; implemented as shared storage
 * with copy-on-write. */
int eb200_buffer_clone(eb200_buffer* buf, eb200_buffer** out);
/* Raw device address (un-shares copy-on-write storage first). */
int eb200_buffer_device_ptr(eb200_buffer* buf, void** ptr);
/* Pinned host staging memory for the async copies. */
int eb200_host_alloc(size_t bytes, void** ptr);
int eb200_host_free(void* ptr);

/* ---- kernels: BackendRegistry::compile_ast (src/backend/device.rs:136-141)
 *      and Kernel::execute (src/backend/traits.rs:545-550) */
int eb200_kernel_create(eb200_device* dev, const eb200_kernel_desc* desc, eb200_kernel** k);
int eb200_kernel_get_info(eb200_kernel* k, eb200_kernel_info* info);
/* Dry run of the classification kernel_create performs, without a device:
 * validates `desc` and reports the kernel that would serve it on a GPU with
 * `sm_count` SMs.  Lets a caller (e.g. the lowerer's dispatch,
 * src/lowerer/lower.rs:335-388) ask whether a loop nest is supported. */
int eb200_kernel_query(const eb200_kernel_desc* desc, int sm_count, eb200_kernel_info* info);
/* Inputs first, then outputs, in Kernel.params order
 * (src/lowerer/lower.rs:1047-1105).  Asynchronous on the device stream. */
int eb200_kernel_launch(eb200_kernel* k, eb200_buffer* const* inputs, int n_inputs,
                        eb200_buffer* const* outputs, int n_outputs);
int eb200_kernel_release(eb200_kernel* k);
/* Column reduce that allocates nothing (no counterpart in the reference; added
 * for callers that own device memory but may not allocate: cudaMalloc
 * synchronises the device, which a latency-critical loop cannot afford, and a
 * caller whose arena already holds all device memory has nothing left to ask
 * for).  out[c] = reduce over r of x[r*cols + c] for contiguous f32 x
 * [rows, cols]; `reduce_op` is an eb200_reduce_op, `stream` the cudaStream_t
 * to launch on (NULL = default stream); x and out are device pointers the
 * caller owns, 16-byte aligned.  Partial results go through a 2 MiB array
 * compiled into the library (every GPU that loads the library holds it until
 * exit): row-splits x cols may not exceed 524 288 partials, and a shape whose
 * split needs more fails with EB200_ERR_UNSUPPORTED before anything launches.
 * The first call on a device looks up that array's device address; make that
 * first call outside any stream capture.  All calls share the array: two calls
 * whose kernels overlap on the GPU (different streams) race on it.  The device
 * that owns x, out and `stream` must be the calling thread's current device
 * (cudaSetDevice): the scratch array is looked up, and the kernels are
 * launched, on the current device. */
int eb200_reduce_cols_static(const float* x, int64_t rows, int64_t cols, int reduce_op,
                             float* out, void* stream);
/* ---- collectives.  No counterpart in the reference (it has no distributed code: no collective
 *      call site, an Rc-based single-thread graph, src/graph/node.rs:222); they serve the
 *      data-parallel training step (batch shards, one gradient all-reduce per step: the update
 *      loop of crates/nn/src/optim/sgd.rs:73-103 once per rank) and row-sharded reductions.
 *      One process per GPU.  Rank 0 makes a unique id, the host passes it to the other ranks by
 *      any channel it has, every rank calls eb200_comm_init.  Messages of up to 524 288 floats go
 *      through a one-shot kernel over NVLink (each rank stores its part into an inbox in every
 *      peer's memory, then reduces from its own memory); larger ones, and all of them when the
 *      peers' memory cannot be mapped, through NCCL (loaded at run time).  All ranks must issue
 *      the same collectives in the same order.  A rank whose peers do not arrive gives up after
 *      about a second; eb200_device_sync then returns EB200_ERR_TIMEOUT. */
typedef struct { char bytes[128]; } eb200_comm_id;
int eb200_comm_unique_id(eb200_comm_id* id);
int eb200_comm_init(eb200_device* dev, int rank, int nranks, const eb200_comm_id* id, eb200_comm** comm);
/* rank, size, whether the one-shot transport is up, and how many collectives took each transport */
int eb200_comm_info(eb200_comm* comm, int* rank, int* nranks, int* one_shot, int64_t* calls_one_shot, int64_t* calls_nccl);
/* In-place all-reduce of f32 elements [offset, offset + count) of `buf` with an eb200_reduce_op,
 * ordered on the device's compute stream like a kernel launch. */
int eb200_comm_allreduce(eb200_comm* comm, eb200_buffer* buf, int64_t offset, int64_t count, int reduce_op);
/* The same on the communicator's own high-priority stream: it starts once the work queued on the
 * compute stream so far is done and runs beside what is queued afterwards; eb200_comm_join makes
 * the compute stream wait for it.  Both may be issued while a step is recorded by eb200_graph_begin
 * (join before eb200_graph_end). */
int eb200_comm_allreduce_async(eb200_comm* comm, eb200_buffer* buf, int64_t offset, int64_t count, int reduce_op);
int eb200_comm_join(eb200_comm* comm);
/* Gradient all-reduce fused with the SGD update, one kernel: params[i] -= lr * sum over ranks of
 * grads[i] for i in [offset, offset + count) (gradient mean: pass lr / nranks).  grads keeps this
 * rank's own values.  The _async form runs on the communicator's stream (see above). */
int eb200_comm_allreduce_sgd(eb200_comm* comm, eb200_buffer* params, eb200_buffer* grads, int64_t offset, int64_t count, float lr);
int eb200_comm_allreduce_sgd_async(eb200_comm* comm, eb200_buffer* params, eb200_buffer* grads, int64_t offset, int64_t count, float lr);
/* Makes a REDUCE kernel's output the all-reduce over the ranks of what it computes locally (a
 * row-sharded sum / max): for a split column reduce the pass that folds the split partials also
 * pushes them to the peers and reduces theirs (one kernel); other reduce kernels are followed by
 * an all-reduce of the output.  The output must be a contiguous f32 range.  NULL detaches. */
int eb200_kernel_set_allreduce(eb200_kernel* k, eb200_comm* comm);
int eb200_comm_destroy(eb200_comm* comm);
/* Number of device kernel launches issued through this library so far. */
int eb200_launch_count(int64_t* count);

#ifdef __cplusplus
}
#endif
#endif /* EB200_H */
