// Collectives of the C ABI: eb200_comm_* (include/eb200.h).
//
// The reference has no distributed code at all (no collective call site; its graph is
// an Rc-based single-thread object, src/graph/node.rs:222).  Data-parallel training
// and row-sharded reductions are new with this backend: one process per GPU, the
// gradients (or the partial results of a sharded reduce) all-reduced between the
// ranks of one NVSwitch box.
//
// Two transports sit behind eb200_comm_allreduce:
//
//   one-shot push  for messages up to EB_AR_CAP floats (gradient buffers of the
//                  benchmark models are 0.27 - 0.9 MB, reduce partials 32 KB: latency
//                  bound).  Every rank owns an inbox in its own memory, mapped into the
//                  peers through CUDA IPC.  ONE kernel per rank: each CTA stores its
//                  chunk of the rank's data into the slot [rank] of every peer's inbox
//                  (plain stores over NVLink), publishes a sequence number to the
//                  peer's flag word (fence + st.release.sys), waits until every
//                  peer's flag for the same chunk shows the same number
//                  (ld.acquire.sys, bounded), then reduces the nranks slots from ITS
//                  OWN memory in rank order (so all ranks get bit-identical results)
//                  and applies the epilogue: plain store, or the SGD update
//                  p -= lr * sum (gradient all-reduce fused with the optimizer), or,
//                  as the prologue, the fold of a split column reduce's partials
//                  (reduce fused with its collective).  No loads from peer memory,
//                  no TMA, no multicast.  Slots and flags alternate between two
//                  parities and the sequence number lives on the device, so calls can
//                  follow each other (and be replayed from a CUDA graph) without any
//                  reset in between.
//   NCCL           everything larger, and every call when the peers' inboxes could
//                  not be mapped.  The library is loaded with dlopen at
//                  eb200_comm_init, so libeb200 itself does not link against it.
//
// Waiting is bounded: a rank whose peers never arrive gives up after about a
// second, raises the device's error word and returns; eb200_device_sync then
// reports EB200_ERR_TIMEOUT.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <algorithm>

#include "common.h"

namespace eb200 {

constexpr int EB_AR_MAX_RANKS = 8;
constexpr int EB_AR_MAX_CTAS = 256;
constexpr long long EB_AR_CAP = 1LL << 19;          // floats per rank slot (2 MiB)
constexpr int EB_AR_CHANNELS = 2;                   // 0: the device's compute stream, 1: the communicator's side stream
constexpr unsigned EB_AR_SPIN_LIMIT = 1u << 23;     // x >= 100 ns of back-off: about a second

struct ArChannel {
    float* inbox[EB_AR_MAX_RANKS];        // rank r's inbox [2][nranks][cap] as mapped here ([rank] = own memory)
    unsigned* flags[EB_AR_MAX_RANKS];     // rank r's flags [2][nranks][EB_AR_MAX_CTAS]
    unsigned* counter;                    // own: number of finished calls on this channel
    unsigned* ticket;                     // own: CTAs of the running call that have finished
};

struct ArParams {
    ArChannel ch;
    int rank, nranks, rop;
    long long count, chunk;               // elements in the message; per CTA (multiple of 4)
    const float* src;                     // SRC_BUFFER: this rank's contribution
    float* dst;                           // DST_STORE: result; DST_SGD: the parameters
    float lr;
    const float* partials;                // SRC_PARTIALS: [splits][kept] partial results of a split reduce
    int splits;
    long long kept;
    int* error_flag;
};

enum { SRC_BUFFER = 0, SRC_PARTIALS = 1 };
enum { DST_STORE = 0, DST_SGD = 1 };

__device__ __forceinline__ float ar_identity(int rop) {
    return rop == EB200_R_MAX ? -INFINITY : (rop == EB200_R_MIN ? INFINITY : (rop == EB200_R_PROD ? 1.0f : 0.0f));
}
__device__ __forceinline__ float ar_combine(int rop, float a, float b) {
    switch (rop) {
        case EB200_R_MAX: return fmaxf(a, b);
        case EB200_R_MIN: return a < b ? a : b;
        case EB200_R_PROD: return a * b;
        default: return a + b;
    }
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <int SRC>
__device__ __forceinline__ float ar_value(const ArParams& q, long long i) {
    if (SRC == SRC_BUFFER) return q.src[i];
    float acc = ar_identity(q.rop);
    for (int s = 0; s < q.splits; ++s) acc = ar_combine(q.rop, acc, __ldcg(q.partials + (long long)s * q.kept + i));
    return acc;
}

template <int SRC, int DST>
__global__ void __launch_bounds__(256) allreduce_push_kernel(const __grid_constant__ ArParams q) {
    // every CTA reads the call number before the last CTA to finish advances it
    const unsigned seq = *reinterpret_cast<volatile unsigned*>(q.ch.counter) + 1u;
    const unsigned par = seq & 1u;
    const int b = blockIdx.x, tid = threadIdx.x;
    const long long lo = (long long)b * q.chunk, hi = min(q.count, lo + q.chunk);
    const long long slot = ((long long)par * q.nranks + q.rank) * EB_AR_CAP;     // where this rank's data goes in every inbox

    // 1. push this rank's chunk into every inbox (its own included)
    const bool vec = SRC == SRC_BUFFER && ((reinterpret_cast<uintptr_t>(q.src) & 15) == 0);
    if (vec) {
        for (long long i = lo + tid * 4LL; i < hi; i += 256 * 4) {
            if (i + 4 <= hi) {
                const float4 v = *reinterpret_cast<const float4*>(q.src + i);
#pragma unroll
                for (int r = 0; r < EB_AR_MAX_RANKS; ++r)
                    if (r < q.nranks) *reinterpret_cast<float4*>(q.ch.inbox[r] + slot + i) = v;
            } else {
                for (long long j = i; j < hi; ++j) {
                    const float v = q.src[j];
#pragma unroll
                    for (int r = 0; r < EB_AR_MAX_RANKS; ++r)
                        if (r < q.nranks) q.ch.inbox[r][slot + j] = v;
                }
            }
        }
    } else {
        for (long long i = lo + tid; i < hi; i += 256) {
            const float v = ar_value<SRC>(q, i);
#pragma unroll
            for (int r = 0; r < EB_AR_MAX_RANKS; ++r)
                if (r < q.nranks) q.ch.inbox[r][slot + i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();

    // 2. tell every peer that chunk b of this rank has landed; wait for theirs
    bool ok = true;
    if (tid < q.nranks && tid != q.rank) {
        const long long f = ((long long)par * q.nranks + q.rank) * EB_AR_MAX_CTAS + b;
        st_release_sys(q.ch.flags[tid] + f, seq);
        const unsigned* mine = q.ch.flags[q.rank] + ((long long)par * q.nranks + tid) * EB_AR_MAX_CTAS + b;
        unsigned spins = 0;
        while (ld_acquire_sys(mine) != seq) {
            if (++spins > EB_AR_SPIN_LIMIT) { ok = false; break; }
            __nanosleep(spins < 64 ? 20 : 200);
        }
    }
    ok = __syncthreads_and(ok ? 1 : 0) != 0;

    // 3. reduce the slots from this rank's own memory, in rank order
    if (ok) {
        const float* base = q.ch.inbox[q.rank] + (long long)par * q.nranks * EB_AR_CAP;
        for (long long i = lo + tid * 4LL; i < hi; i += 256 * 4) {
            if (i + 4 <= hi && ((reinterpret_cast<uintptr_t>(q.dst + i) & 15) == 0)) {
                float4 acc = __ldcg(reinterpret_cast<const float4*>(base + i));
                for (int r = 1; r < q.nranks; ++r) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (long long)r * EB_AR_CAP + i));
                    acc.x = ar_combine(q.rop, acc.x, v.x); acc.y = ar_combine(q.rop, acc.y, v.y);
                    acc.z = ar_combine(q.rop, acc.z, v.z); acc.w = ar_combine(q.rop, acc.w, v.w);
                }
                float4* d = reinterpret_cast<float4*>(q.dst + i);
                if (DST == DST_SGD) {
                    const float4 pv = *d;
                    acc = make_float4(__fsub_rn(pv.x, __fmul_rn(q.lr, acc.x)), __fsub_rn(pv.y, __fmul_rn(q.lr, acc.y)),
                                      __fsub_rn(pv.z, __fmul_rn(q.lr, acc.z)), __fsub_rn(pv.w, __fmul_rn(q.lr, acc.w)));
                }
                *d = acc;
            } else {
                for (long long j = i; j < min(i + 4, hi); ++j) {
                    float acc = __ldcg(base + j);
                    for (int r = 1; r < q.nranks; ++r) acc = ar_combine(q.rop, acc, __ldcg(base + (long long)r * EB_AR_CAP + j));
                    q.dst[j] = DST == DST_SGD ? __fsub_rn(q.dst[j], __fmul_rn(q.lr, acc)) : acc;
                }
            }
        }
    } else if (tid == 0 && q.error_flag) {
        atomicExch(q.error_flag, 1);
    }

    // 4. the last CTA to finish advances the call number
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(q.ch.ticket, 1u) == gridDim.x - 1) {
            *q.ch.counter = seq;
            *q.ch.ticket = 0u;
            __threadfence();
        }
    }
}

// ---- NCCL through dlopen ------------------------------------------------------------------
struct Nccl {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static Nccl* nccl_api() {
    static Nccl api;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (api.lib) return &api;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return nullptr;
#define SYM(field, name) *reinterpret_cast<void**>(&api.field) = dlsym(h, name)
    SYM(GetUniqueId, "ncclGetUniqueId");
    SYM(CommInitRank, "ncclCommInitRank");
    SYM(CommDestroy, "ncclCommDestroy");
    SYM(AllReduce, "ncclAllReduce");
    SYM(AllGather, "ncclAllGather");
    SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.AllGather || !api.GetErrorString) return nullptr;
    api.lib = h;
    return &api;
}

#define EB_CHECK_NCCL(api, expr)                                                                   \
    do {                                                                                           \
        ncclResult_t _r = (expr);                                                                  \
        if (_r != ncclSuccess)                                                                     \
            return ::eb200::set_error(EB200_ERR_COMM, "%s failed: %s", #expr, (api)->GetErrorString(_r)); \
    } while (0)

}  // namespace eb200

using namespace eb200;

struct eb200_comm {
    eb200::Device* dev = nullptr;
    int rank = 0, nranks = 1;
    eb200::Nccl* api = nullptr;
    ncclComm_t nccl = nullptr;
    // one-shot transport
    bool one_shot = false;
    void* own_block = nullptr;                          // cudaMalloc'ed: both channels' inboxes, flags, counters
    void* peer_block[eb200::EB_AR_MAX_RANKS] = {nullptr};
    eb200::ArChannel ch[eb200::EB_AR_CHANNELS];
    cudaStream_t side = nullptr;                        // high-priority stream for collectives that overlap compute
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    bool side_pending = false;
    int64_t n_one_shot = 0, n_nccl = 0;
};

namespace eb200 {

static size_t channel_bytes(int nranks) {
    return (size_t)2 * nranks * EB_AR_CAP * 4 + (size_t)2 * nranks * EB_AR_MAX_CTAS * 4 + 256;
}

static void fill_channel(ArChannel* ch, char* const* blocks, int nranks, int channel) {
    const size_t cb = channel_bytes(nranks);
    for (int r = 0; r < nranks; ++r) {
        char* base = blocks[r] + (size_t)channel * cb;
        ch->inbox[r] = reinterpret_cast<float*>(base);
        ch->flags[r] = reinterpret_cast<unsigned*>(base + (size_t)2 * nranks * EB_AR_CAP * 4);
    }
}

// Maps every peer's inbox block.  Any failure leaves the communicator on NCCL only.
static bool setup_one_shot(eb200_comm* c) {
    if (c->nranks > EB_AR_MAX_RANKS) return false;
    const size_t cb = channel_bytes(c->nranks), total = cb * EB_AR_CHANNELS;
    if (cudaMalloc(&c->own_block, total) != cudaSuccess) { cudaGetLastError(); c->own_block = nullptr; return false; }
    cudaMemset(c->own_block, 0, total);
    cudaIpcMemHandle_t mine;
    bool ok = cudaIpcGetMemHandle(&mine, c->own_block) == cudaSuccess;
    if (!ok) { cudaGetLastError(); memset(&mine, 0, sizeof(mine)); }
    // all-gather {ok, handle} through NCCL
    struct Rec { int ok; int pad; cudaIpcMemHandle_t h; };
    Rec rec{ok ? 1 : 0, 0, mine};
    Rec* dbuf = nullptr;
    if (cudaMalloc(&dbuf, sizeof(Rec) * c->nranks) != cudaSuccess) { cudaGetLastError(); return false; }
    std::vector<Rec> all(c->nranks);
    bool good = cudaMemcpy(dbuf + c->rank, &rec, sizeof(Rec), cudaMemcpyHostToDevice) == cudaSuccess &&
                c->api->AllGather(dbuf + c->rank, dbuf, sizeof(Rec), ncclChar, c->nccl, c->dev->stream) == ncclSuccess &&
                cudaStreamSynchronize(c->dev->stream) == cudaSuccess &&
                cudaMemcpy(all.data(), dbuf, sizeof(Rec) * c->nranks, cudaMemcpyDeviceToHost) == cudaSuccess;
    cudaFree(dbuf);
    if (!good) { cudaGetLastError(); return false; }
    for (int r = 0; r < c->nranks; ++r) good = good && all[r].ok;
    int mapped = good ? 1 : 0;
    if (good) {
        for (int r = 0; r < c->nranks && mapped; ++r) {
            if (r == c->rank) { c->peer_block[r] = c->own_block; continue; }
            if (cudaIpcOpenMemHandle(&c->peer_block[r], all[r].h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                c->peer_block[r] = nullptr;
                mapped = 0;
            }
        }
    }
    // every rank must take the same transport: agree on the minimum
    int* dflag = nullptr;
    if (cudaMalloc(&dflag, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return false; }
    int agreed = 0;
    bool ex = cudaMemcpy(dflag, &mapped, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess &&
              c->api->AllReduce(dflag, dflag, 1, ncclInt, ncclMin, c->nccl, c->dev->stream) == ncclSuccess &&
              cudaStreamSynchronize(c->dev->stream) == cudaSuccess &&
              cudaMemcpy(&agreed, dflag, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess;
    cudaFree(dflag);
    if (!ex || !agreed) { cudaGetLastError(); return false; }
    char* blocks[EB_AR_MAX_RANKS];
    for (int r = 0; r < c->nranks; ++r) blocks[r] = reinterpret_cast<char*>(c->peer_block[r]);
    for (int k = 0; k < EB_AR_CHANNELS; ++k) {
        fill_channel(&c->ch[k], blocks, c->nranks, k);
        char* own = blocks[c->rank] + (size_t)k * cb;
        unsigned* ctl = reinterpret_cast<unsigned*>(own + cb - 256);
        c->ch[k].counter = ctl;
        c->ch[k].ticket = ctl + 1;
    }
    return true;
}

static ncclRedOp_t nccl_op(int rop) {
    switch (rop) {
        case EB200_R_MAX: return ncclMax;
        case EB200_R_MIN: return ncclMin;
        case EB200_R_PROD: return ncclProd;
        default: return ncclSum;
    }
}

static void ar_grid(long long count, long long* chunk, unsigned* grid) {
    // 2048 floats (8 KB) per CTA, at most EB_AR_MAX_CTAS CTAs; chunks are multiples of 4 floats
    long long ctas = std::max(1LL, std::min<long long>(EB_AR_MAX_CTAS, (count + 2047) / 2048));
    long long ch = ((count + ctas - 1) / ctas + 3) / 4 * 4;
    *chunk = ch;
    *grid = (unsigned)((count + ch - 1) / ch);
}

// The message as this rank holds it (src), where the result goes (dst), on `stream` over channel `k`.
static int allreduce_impl(eb200_comm* c, int k, cudaStream_t stream, const float* src, float* dst, long long count, int rop,
                          int dst_kind, float lr, const float* partials, int splits, long long kept) {
    if (count <= 0) return EB200_OK;
    if (c->nranks == 1 && !partials && dst_kind == DST_STORE) {
        if (src != dst) EB_CHECK_CUDA(cudaMemcpyAsync(dst, src, (size_t)count * 4, cudaMemcpyDeviceToDevice, stream));
        return EB200_OK;
    }
    if (c->one_shot && count <= EB_AR_CAP) {
        ArParams q{};
        q.ch = c->ch[k];
        q.rank = c->rank; q.nranks = c->nranks; q.rop = rop;
        q.count = count;
        unsigned grid = 1;
        ar_grid(count, &q.chunk, &grid);
        q.src = src; q.dst = dst; q.lr = lr;
        q.partials = partials; q.splits = splits; q.kept = kept;
        q.error_flag = c->dev->error_flag_dev;
        if (partials) allreduce_push_kernel<SRC_PARTIALS, DST_STORE><<<grid, 256, 0, stream>>>(q);
        else if (dst_kind == DST_SGD) allreduce_push_kernel<SRC_BUFFER, DST_SGD><<<grid, 256, 0, stream>>>(q);
        else allreduce_push_kernel<SRC_BUFFER, DST_STORE><<<grid, 256, 0, stream>>>(q);
        count_launch();
        EB_CHECK_CUDA(cudaGetLastError());
        ++c->n_one_shot;
        return EB200_OK;
    }
    EB_REQUIRE(!partials && dst_kind == DST_STORE, EB200_ERR_UNSUPPORTED,
               "a fused all-reduce needs the one-shot transport (message of %lld floats, limit %lld)", count, (long long)EB_AR_CAP);
    EB_REQUIRE(c->nccl, EB200_ERR_COMM, "communicator has no NCCL transport");
    EB_CHECK_NCCL(c->api, c->api->AllReduce(src, dst, (size_t)count, ncclFloat, nccl_op(rop), c->nccl, stream));
    ++c->n_nccl;
    return EB200_OK;
}

int comm_reduce_finish_allreduce(eb200_comm* c, const float* partials, int splits, long long kept, int rop, float* out) {
    return allreduce_impl(c, 0, c->dev->stream, nullptr, out, kept, rop, DST_STORE, 0.f, partials, splits, kept);
}
bool comm_can_fuse(eb200_comm* c, long long count) { return c && c->one_shot && count <= EB_AR_CAP; }
int comm_allreduce_buffer(eb200_comm* c, float* data, long long count, int rop) {
    return allreduce_impl(c, 0, c->dev->stream, data, data, count, rop, DST_STORE, 0.f, nullptr, 0, 0);
}

}  // namespace eb200

extern "C" {

int eb200_comm_unique_id(eb200_comm_id* id) {
    EB_REQUIRE(id, EB200_ERR_INVALID, "id is null");
    static_assert(sizeof(eb200_comm_id) >= sizeof(ncclUniqueId), "eb200_comm_id must hold an NCCL unique id");
    Nccl* api = nccl_api();
    EB_REQUIRE(api, EB200_ERR_COMM, "libnccl.so.2 could not be loaded: %s", dlerror());
    ncclUniqueId nid;
    EB_CHECK_NCCL(api, api->GetUniqueId(&nid));
    memset(id, 0, sizeof(*id));
    memcpy(id, &nid, sizeof(nid));
    return EB200_OK;
}

int eb200_comm_init(eb200_device* dev, int rank, int nranks, const eb200_comm_id* id, eb200_comm** out) {
    EB_REQUIRE(dev && out, EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, EB200_ERR_INVALID, "rank %d of %d", rank, nranks);
    EB_REQUIRE(nranks == 1 || id, EB200_ERR_INVALID, "a communicator of %d ranks needs the unique id rank 0 made", nranks);
    EB_CHECK_CUDA(cudaSetDevice(dev->index));
    auto c = new eb200_comm();
    c->dev = dev; c->rank = rank; c->nranks = nranks;
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);     // hi = numerically lowest = greatest priority
    if (cudaStreamCreateWithPriority(&c->side, cudaStreamNonBlocking, hi) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return set_error(EB200_ERR_CUDA, "could not create the communicator's stream and events");
    }
    if (nranks == 1) {
        // a single rank keeps the same kernels: its inbox is local and nobody is waited for
        const size_t total = channel_bytes(1) * EB_AR_CHANNELS;
        if (cudaMalloc(&c->own_block, total) == cudaSuccess && cudaMemset(c->own_block, 0, total) == cudaSuccess) {
            char* blocks[EB_AR_MAX_RANKS] = {reinterpret_cast<char*>(c->own_block)};
            for (int k = 0; k < EB_AR_CHANNELS; ++k) {
                fill_channel(&c->ch[k], blocks, 1, k);
                unsigned* ctl = reinterpret_cast<unsigned*>(blocks[0] + (size_t)(k + 1) * channel_bytes(1) - 256);
                c->ch[k].counter = ctl;
                c->ch[k].ticket = ctl + 1;
            }
            c->one_shot = true;
        } else {
            cudaGetLastError();
            delete c;
            return set_error(EB200_ERR_OOM, "could not allocate the communicator's inbox");
        }
    }
    if (nranks > 1) {
        c->api = nccl_api();
        if (!c->api) { delete c; return set_error(EB200_ERR_COMM, "libnccl.so.2 could not be loaded: %s", dlerror()); }
        ncclUniqueId nid;
        memcpy(&nid, id, sizeof(nid));
        ncclResult_t r = c->api->CommInitRank(&c->nccl, nranks, nid, rank);
        if (r != ncclSuccess) {
            const char* msg = c->api->GetErrorString(r);
            delete c;
            return set_error(EB200_ERR_COMM, "ncclCommInitRank failed: %s", msg);
        }
        c->one_shot = setup_one_shot(c);
    }
    *out = c;
    return EB200_OK;
}

int eb200_comm_info(eb200_comm* c, int* rank, int* nranks, int* one_shot, int64_t* calls_one_shot, int64_t* calls_nccl) {
    EB_REQUIRE(c, EB200_ERR_INVALID, "comm is null");
    if (rank) *rank = c->rank;
    if (nranks) *nranks = c->nranks;
    if (one_shot) *one_shot = c->one_shot ? 1 : 0;
    if (calls_one_shot) *calls_one_shot = c->n_one_shot;
    if (calls_nccl) *calls_nccl = c->n_nccl;
    return EB200_OK;
}

static int check_range(eb200_comm* c, eb200_buffer* buf, int64_t offset, int64_t count, int reduce_op) {
    EB_REQUIRE(c && buf, EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(buf->dev == c->dev, EB200_ERR_INVALID, "buffer lives on another device than the communicator");
    EB_REQUIRE(offset >= 0 && count >= 0 && (size_t)(offset + count) * 4 <= buf->bytes, EB200_ERR_BOUNDS,
               "elements [%lld, %lld) of a buffer of %zu bytes", (long long)offset, (long long)(offset + count), buf->bytes);
    EB_REQUIRE(reduce_op >= EB200_R_SUM && reduce_op <= EB200_R_PROD, EB200_ERR_INVALID, "reduce op %d", reduce_op);
    return EB200_OK;
}

int eb200_comm_allreduce(eb200_comm* c, eb200_buffer* buf, int64_t offset, int64_t count, int reduce_op) {
    int st = check_range(c, buf, offset, count, reduce_op);
    if (st) return st;
    EB_CHECK_CUDA(cudaSetDevice(c->dev->index));
    if ((st = buffer_unshare(buf, true))) return st;
    float* data = reinterpret_cast<float*>(buf->storage->ptr) + offset;
    return allreduce_impl(c, 0, c->dev->stream, data, data, count, reduce_op, DST_STORE, 0.f, nullptr, 0, 0);
}

static int fork_side(eb200_comm* c) {
    EB_CHECK_CUDA(cudaEventRecord(c->ev_fork, c->dev->stream));
    EB_CHECK_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
    return EB200_OK;
}

int eb200_comm_allreduce_async(eb200_comm* c, eb200_buffer* buf, int64_t offset, int64_t count, int reduce_op) {
    int st = check_range(c, buf, offset, count, reduce_op);
    if (st) return st;
    EB_CHECK_CUDA(cudaSetDevice(c->dev->index));
    if ((st = buffer_unshare(buf, true))) return st;
    if ((st = fork_side(c))) return st;
    float* data = reinterpret_cast<float*>(buf->storage->ptr) + offset;
    st = allreduce_impl(c, 1, c->side, data, data, count, reduce_op, DST_STORE, 0.f, nullptr, 0, 0);
    c->side_pending = true;
    return st;
}

static int sgd_range(eb200_comm* c, eb200_buffer* params, eb200_buffer* grads, int64_t offset, int64_t count) {
    int st = check_range(c, params, offset, count, EB200_R_SUM);
    if (st) return st;
    if ((st = check_range(c, grads, offset, count, EB200_R_SUM))) return st;
    EB_REQUIRE(params->storage->ptr != grads->storage->ptr, EB200_ERR_INVALID, "parameters and gradients share storage");
    EB_CHECK_CUDA(cudaSetDevice(c->dev->index));
    if ((st = buffer_unshare(params, true))) return st;
    return EB200_OK;
}

static int allreduce_sgd_on(eb200_comm* c, int k, cudaStream_t s, eb200_buffer* params, eb200_buffer* grads, int64_t offset,
                            int64_t count, float lr) {
    float* p = reinterpret_cast<float*>(params->storage->ptr) + offset;
    float* g = reinterpret_cast<float*>(grads->storage->ptr) + offset;
    if (c->one_shot && count <= EB_AR_CAP)
        return allreduce_impl(c, k, s, g, p, count, EB200_R_SUM, DST_SGD, lr, nullptr, 0, 0);
    // message too large for the inboxes (or no peer mapping): NCCL, then the plain update kernel
    int st = allreduce_impl(c, k, s, g, g, count, EB200_R_SUM, DST_STORE, 0.f, nullptr, 0, 0);
    if (st) return st;
    Device tmp_dev;
    tmp_dev.index = c->dev->index;
    tmp_dev.stream = s;
    tmp_dev.prop.multiProcessorCount = c->dev->prop.multiProcessorCount;
    Plan pl;
    pl.scalar = lr;
    st = launch_sgd(&tmp_dev, pl, p, g, p, count);
    tmp_dev.stream = nullptr;
    return st;
}

int eb200_comm_allreduce_sgd(eb200_comm* c, eb200_buffer* params, eb200_buffer* grads, int64_t offset, int64_t count, float lr) {
    int st = sgd_range(c, params, grads, offset, count);
    if (st) return st;
    return allreduce_sgd_on(c, 0, c->dev->stream, params, grads, offset, count, lr);
}

int eb200_comm_allreduce_sgd_async(eb200_comm* c, eb200_buffer* params, eb200_buffer* grads, int64_t offset, int64_t count, float lr) {
    int st = sgd_range(c, params, grads, offset, count);
    if (st) return st;
    if ((st = fork_side(c))) return st;
    st = allreduce_sgd_on(c, 1, c->side, params, grads, offset, count, lr);
    c->side_pending = true;
    return st;
}

int eb200_comm_join(eb200_comm* c) {
    EB_REQUIRE(c, EB200_ERR_INVALID, "comm is null");
    if (!c->side_pending) return EB200_OK;
    EB_CHECK_CUDA(cudaEventRecord(c->ev_join, c->side));
    EB_CHECK_CUDA(cudaStreamWaitEvent(c->dev->stream, c->ev_join, 0));
    c->side_pending = false;
    return EB200_OK;
}

int eb200_comm_destroy(eb200_comm* c) {
    if (!c) return EB200_OK;
    cudaSetDevice(c->dev->index);
    cudaStreamSynchronize(c->dev->stream);
    if (c->side) cudaStreamSynchronize(c->side);
    for (int r = 0; r < c->nranks && r < EB_AR_MAX_RANKS; ++r)
        if (r != c->rank && c->peer_block[r]) cudaIpcCloseMemHandle(c->peer_block[r]);
    // this rank's last collective only finished after every peer's stores into its inbox had landed,
    // and peers write nowhere else: the inbox can go
    if (c->nccl && c->api) c->api->CommDestroy(c->nccl);
    if (c->own_block) cudaFree(c->own_block);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    if (c->ev_join) cudaEventDestroy(c->ev_join);
    if (c->side) cudaStreamDestroy(c->side);
    delete c;
    return EB200_OK;
}

}  // extern "C"
