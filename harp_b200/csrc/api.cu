// Library, device and buffer entry points of the C ABI (include/eb200.h).
//
// Device = one CUDA device with one stream that orders all of its work and one
// stream-ordered memory pool (cudaMallocAsync) whose release threshold is
// unbounded, so freed blocks are reused by later allocations instead of going
// back to the driver.  This replaces the per-realize Vec<u8> allocations of the
// reference's C backend (crates/backend-c/src/buffer.rs:84-93) and the
// cudarc alloc_zeros of its CUDA backend (crates/backend-cuda/src/buffer.rs).
#include <stdarg.h>
#include <string.h>

#include "common.h"

namespace eb200 {

static thread_local char t_error[512] = {0};
std::atomic<int64_t> g_launch_count{0};

int set_error(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return status;
}
void clear_error() { t_error[0] = 0; }

Storage::~Storage() {
    if (ptr && dev) {
        // stream-ordered free: safe with respect to launches already queued
        cudaFreeAsync(ptr, dev->stream);
        dev->in_use.fetch_sub((int64_t)bytes);
    }
}

int storage_alloc(Device* dev, size_t bytes, bool zero, std::shared_ptr<Storage>* out) {
    auto s = std::make_shared<Storage>();
    size_t n = bytes ? bytes : 1;
    void* p = nullptr;
    cudaError_t e = cudaMallocFromPoolAsync(&p, n, dev->pool, dev->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(e == cudaErrorMemoryAllocation ? EB200_ERR_OOM : EB200_ERR_CUDA,
                         "device allocation of %zu bytes failed: %s", n, cudaGetErrorString(e));
    }
    s->dev = dev;
    s->ptr = p;
    s->bytes = bytes;
    int64_t now = dev->in_use.fetch_add((int64_t)bytes) + (int64_t)bytes;
    int64_t pk = dev->peak.load();
    while (now > pk && !dev->peak.compare_exchange_weak(pk, now)) {}
    dev->n_allocs.fetch_add(1);
    if (zero && bytes) EB_CHECK_CUDA(cudaMemsetAsync(p, 0, bytes, dev->stream));
    *out = std::move(s);
    return EB200_OK;
}

int buffer_unshare(eb200_buffer* buf, bool keep_contents) {
    if (buf->storage.use_count() <= 1) return EB200_OK;
    std::shared_ptr<Storage> fresh;
    int st = storage_alloc(buf->dev, buf->bytes, false, &fresh);
    if (st) return st;
    if (keep_contents && buf->bytes)
        EB_CHECK_CUDA(cudaMemcpyAsync(fresh->ptr, buf->storage->ptr, buf->bytes,
                                      cudaMemcpyDeviceToDevice, buf->dev->stream));
    buf->storage = std::move(fresh);
    return EB200_OK;
}

int check_device_flag(Device* dev) {
    if (dev->error_flag_host && *reinterpret_cast<volatile int*>(dev->error_flag_host) != 0) {
        *reinterpret_cast<volatile int*>(dev->error_flag_host) = 0;
        return set_error(EB200_ERR_TIMEOUT, "a kernel gave up a bounded device-side wait; its output is not valid");
    }
    return EB200_OK;
}

}  // namespace eb200

using namespace eb200;

extern "C" {

int eb200_abi_version(void) { return EB200_ABI_VERSION; }
const char* eb200_last_error(void) { return t_error; }

int eb200_abi_sizes(size_t* kernel_desc, size_t* operand, size_t* device_props, size_t* kernel_info) {
    if (kernel_desc) *kernel_desc = sizeof(eb200_kernel_desc);
    if (operand) *operand = sizeof(eb200_operand);
    if (device_props) *device_props = sizeof(eb200_device_props);
    if (kernel_info) *kernel_info = sizeof(eb200_kernel_info);
    return EB200_OK;
}

int eb200_device_count(int* count) {
    EB_REQUIRE(count, EB200_ERR_INVALID, "count is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *count = 0;
        return set_error(EB200_ERR_NO_DEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    *count = n;
    return EB200_OK;
}

int eb200_device_open(int index, eb200_device** out) {
    EB_REQUIRE(out, EB200_ERR_INVALID, "dev is null");
    int n = 0;
    int st = eb200_device_count(&n);
    if (st) return st;
    EB_REQUIRE(index >= 0 && index < n, EB200_ERR_NO_DEVICE, "device index %d out of range (%d devices)", index, n);
    auto dev = new eb200_device();
    dev->index = index;
    cudaError_t e = cudaGetDeviceProperties(&dev->prop, index);
    if (e != cudaSuccess) { delete dev; return set_error(EB200_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e)); }
    if (dev->prop.major != 10) {
        int maj = dev->prop.major, mnr = dev->prop.minor;
        delete dev;
        return set_error(EB200_ERR_NO_DEVICE, "device %d is sm_%d%d; this library carries sm_100a code only", index, maj, mnr);
    }
#define OPEN_CHECK(x) do { cudaError_t _e = (x); if (_e != cudaSuccess) { delete dev; return set_error(EB200_ERR_CUDA, "%s: %s", #x, cudaGetErrorString(_e)); } } while (0)
    OPEN_CHECK(cudaSetDevice(index));
    OPEN_CHECK(cudaStreamCreateWithFlags(&dev->stream, cudaStreamNonBlocking));
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = index;
    OPEN_CHECK(cudaMemPoolCreate(&dev->pool, &props));
    uint64_t threshold = UINT64_MAX;
    OPEN_CHECK(cudaMemPoolSetAttribute(dev->pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    OPEN_CHECK(cudaEventCreate(&dev->ev_begin));
    OPEN_CHECK(cudaEventCreate(&dev->ev_end));
    OPEN_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&dev->error_flag_host), sizeof(int), cudaHostAllocMapped));
    *dev->error_flag_host = 0;
    OPEN_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev->error_flag_dev), dev->error_flag_host, 0));
#undef OPEN_CHECK
    *out = dev;
    return EB200_OK;
}

int eb200_device_close(eb200_device* dev) {
    if (!dev) return EB200_OK;
    cudaSetDevice(dev->index);
    cudaStreamSynchronize(dev->stream);
    if (dev->ev_begin) cudaEventDestroy(dev->ev_begin);
    if (dev->ev_end) cudaEventDestroy(dev->ev_end);
    if (dev->error_flag_host) cudaFreeHost(dev->error_flag_host);
    if (dev->pool) cudaMemPoolDestroy(dev->pool);
    if (dev->stream) cudaStreamDestroy(dev->stream);
    delete dev;
    return EB200_OK;
}

int eb200_device_sync(eb200_device* dev) {
    EB_REQUIRE(dev, EB200_ERR_INVALID, "dev is null");
    EB_CHECK_CUDA(cudaStreamSynchronize(dev->stream));
    return check_device_flag(dev);
}

int eb200_device_get_props(eb200_device* dev, eb200_device_props* props) {
    EB_REQUIRE(dev && props, EB200_ERR_INVALID, "null argument");
    memset(props, 0, sizeof(*props));
    strncpy(props->name, dev->prop.name, sizeof(props->name) - 1);
    props->cc_major = dev->prop.major;
    props->cc_minor = dev->prop.minor;
    props->sm_count = dev->prop.multiProcessorCount;
    props->total_mem_bytes = (int64_t)dev->prop.totalGlobalMem;
    props->l2_bytes = dev->prop.l2CacheSize;
    props->smem_per_block_optin = (int64_t)dev->prop.sharedMemPerBlockOptin;
    return EB200_OK;
}

int eb200_device_stream(eb200_device* dev, void** stream) {
    EB_REQUIRE(dev && stream, EB200_ERR_INVALID, "null argument");
    *stream = (void*)dev->stream;
    return EB200_OK;
}

int eb200_timer_begin(eb200_device* dev) {
    EB_REQUIRE(dev, EB200_ERR_INVALID, "dev is null");
    EB_CHECK_CUDA(cudaEventRecord(dev->ev_begin, dev->stream));
    return EB200_OK;
}

int eb200_timer_end(eb200_device* dev, float* ms) {
    EB_REQUIRE(dev && ms, EB200_ERR_INVALID, "null argument");
    EB_CHECK_CUDA(cudaEventRecord(dev->ev_end, dev->stream));
    EB_CHECK_CUDA(cudaEventSynchronize(dev->ev_end));
    EB_CHECK_CUDA(cudaEventElapsedTime(ms, dev->ev_begin, dev->ev_end));
    return EB200_OK;
}

struct eb200_graph {
    eb200::Device* dev;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
};

int eb200_graph_begin(eb200_device* dev) {
    EB_REQUIRE(dev, EB200_ERR_INVALID, "dev is null");
    EB_CHECK_CUDA(cudaSetDevice(dev->index));
    EB_CHECK_CUDA(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
    return EB200_OK;
}

int eb200_graph_end(eb200_device* dev, eb200_graph** out) {
    EB_REQUIRE(dev && out, EB200_ERR_INVALID, "null argument");
    cudaGraph_t g = nullptr;
    EB_CHECK_CUDA(cudaStreamEndCapture(dev->stream, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        return set_error(EB200_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    *out = new eb200_graph{dev, g, exec};
    return EB200_OK;
}

int eb200_graph_launch(eb200_graph* graph) {
    EB_REQUIRE(graph, EB200_ERR_INVALID, "graph is null");
    EB_CHECK_CUDA(cudaGraphLaunch(graph->exec, graph->dev->stream));
    return EB200_OK;
}

int eb200_graph_release(eb200_graph* graph) {
    if (!graph) return EB200_OK;
    cudaGraphExecDestroy(graph->exec);
    cudaGraphDestroy(graph->graph);
    delete graph;
    return EB200_OK;
}

struct eb200_event {
    eb200::Device* dev;
    cudaEvent_t ev;
};

int eb200_event_create(eb200_device* dev, eb200_event** out) {
    EB_REQUIRE(dev && out, EB200_ERR_INVALID, "null argument");
    EB_CHECK_CUDA(cudaSetDevice(dev->index));
    cudaEvent_t e;
    EB_CHECK_CUDA(cudaEventCreate(&e));
    *out = new eb200_event{dev, e};
    return EB200_OK;
}

int eb200_event_record(eb200_event* ev) {
    EB_REQUIRE(ev, EB200_ERR_INVALID, "ev is null");
    EB_CHECK_CUDA(cudaEventRecord(ev->ev, ev->dev->stream));
    return EB200_OK;
}

int eb200_event_elapsed_ms(eb200_event* a, eb200_event* b, float* ms) {
    EB_REQUIRE(a && b && ms, EB200_ERR_INVALID, "null argument");
    EB_CHECK_CUDA(cudaEventSynchronize(b->ev));
    EB_CHECK_CUDA(cudaEventElapsedTime(ms, a->ev, b->ev));
    return EB200_OK;
}

int eb200_event_destroy(eb200_event* ev) {
    if (!ev) return EB200_OK;
    cudaEventDestroy(ev->ev);
    delete ev;
    return EB200_OK;
}

struct eb200_stream {
    eb200::Device* dev;
    cudaStream_t s;
};

int eb200_stream_create(eb200_device* dev, eb200_stream** out) {
    EB_REQUIRE(dev && out, EB200_ERR_INVALID, "null argument");
    EB_CHECK_CUDA(cudaSetDevice(dev->index));
    cudaStream_t s;
    EB_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = new eb200_stream{dev, s};
    return EB200_OK;
}

int eb200_stream_destroy(eb200_stream* s) {
    if (!s) return EB200_OK;
    cudaStreamSynchronize(s->s);
    cudaStreamDestroy(s->s);
    delete s;
    return EB200_OK;
}

int eb200_stream_sync(eb200_stream* s) {
    EB_REQUIRE(s, EB200_ERR_INVALID, "stream is null");
    EB_CHECK_CUDA(cudaStreamSynchronize(s->s));
    return EB200_OK;
}

int eb200_stream_wait(eb200_device* dev, eb200_stream* s, eb200_event* ev) {
    EB_REQUIRE(dev && ev, EB200_ERR_INVALID, "null argument");
    EB_CHECK_CUDA(cudaStreamWaitEvent(s ? s->s : dev->stream, ev->ev, 0));
    return EB200_OK;
}

int eb200_event_record_on(eb200_event* ev, eb200_stream* s) {
    EB_REQUIRE(ev, EB200_ERR_INVALID, "ev is null");
    EB_CHECK_CUDA(cudaEventRecord(ev->ev, s ? s->s : ev->dev->stream));
    return EB200_OK;
}

int eb200_buffer_write_on(eb200_buffer* buf, const void* host, size_t bytes, eb200_stream* s) {
    EB_REQUIRE(buf && host && s, EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(bytes == buf->bytes, EB200_ERR_INVALID, "Buffer size mismatch: expected %zu, got %zu", buf->bytes, bytes);
    EB_REQUIRE(buf->storage.use_count() <= 1, EB200_ERR_INVALID, "buffer shares storage with a clone; write it on the compute stream");
    EB_CHECK_CUDA(cudaSetDevice(buf->dev->index));
    EB_CHECK_CUDA(cudaMemcpyAsync(buf->storage->ptr, host, bytes, cudaMemcpyHostToDevice, s->s));
    return EB200_OK;
}

int eb200_buffer_read_on(eb200_buffer* buf, void* host, size_t bytes, eb200_stream* s) {
    EB_REQUIRE(buf && host && s, EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(bytes == buf->bytes, EB200_ERR_INVALID, "Buffer size mismatch: expected %zu, got %zu", buf->bytes, bytes);
    EB_CHECK_CUDA(cudaSetDevice(buf->dev->index));
    EB_CHECK_CUDA(cudaMemcpyAsync(host, buf->storage->ptr, bytes, cudaMemcpyDeviceToHost, s->s));
    return EB200_OK;
}

int eb200_device_mem_stats(eb200_device* dev, int64_t* in_use, int64_t* peak, int64_t* n_allocs) {
    EB_REQUIRE(dev, EB200_ERR_INVALID, "dev is null");
    if (in_use) *in_use = dev->in_use.load();
    if (peak) *peak = dev->peak.load();
    if (n_allocs) *n_allocs = dev->n_allocs.load();
    return EB200_OK;
}

static int buffer_new(eb200_device* dev, size_t bytes, bool zero, eb200_buffer** out) {
    EB_REQUIRE(dev && out, EB200_ERR_INVALID, "null argument");
    EB_CHECK_CUDA(cudaSetDevice(dev->index));
    auto b = new eb200_buffer();
    b->dev = dev;
    b->bytes = bytes;
    int st = storage_alloc(dev, bytes, zero, &b->storage);
    if (st) { delete b; return st; }
    *out = b;
    return EB200_OK;
}

int eb200_buffer_alloc(eb200_device* dev, size_t bytes, eb200_buffer** buf) { return buffer_new(dev, bytes, true, buf); }
int eb200_buffer_alloc_uninit(eb200_device* dev, size_t bytes, eb200_buffer** buf) { return buffer_new(dev, bytes, false, buf); }

int eb200_buffer_retain(eb200_buffer* buf) {
    EB_REQUIRE(buf, EB200_ERR_INVALID, "buf is null");
    buf->refs.fetch_add(1);
    return EB200_OK;
}

int eb200_buffer_release(eb200_buffer* buf) {
    if (!buf) return EB200_OK;
    if (buf->refs.fetch_sub(1) == 1) {
        cudaSetDevice(buf->dev->index);
        delete buf;
    }
    return EB200_OK;
}

int eb200_buffer_bytes(eb200_buffer* buf, size_t* bytes) {
    EB_REQUIRE(buf && bytes, EB200_ERR_INVALID, "null argument");
    *bytes = buf->bytes;
    return EB200_OK;
}

static int buffer_write(eb200_buffer* buf, const void* host, size_t bytes, bool sync) {
    EB_REQUIRE(buf && (host || !bytes), EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(bytes == buf->bytes, EB200_ERR_INVALID, "Buffer size mismatch: expected %zu, got %zu", buf->bytes, bytes);
    EB_CHECK_CUDA(cudaSetDevice(buf->dev->index));
    int st = buffer_unshare(buf, false);
    if (st) return st;
    if (bytes) EB_CHECK_CUDA(cudaMemcpyAsync(buf->storage->ptr, host, bytes, cudaMemcpyHostToDevice, buf->dev->stream));
    if (sync) EB_CHECK_CUDA(cudaStreamSynchronize(buf->dev->stream));
    return EB200_OK;
}

static int buffer_read(eb200_buffer* buf, void* host, size_t bytes, bool sync) {
    EB_REQUIRE(buf && (host || !bytes), EB200_ERR_INVALID, "null argument");
    EB_REQUIRE(bytes == buf->bytes, EB200_ERR_INVALID, "Buffer size mismatch: expected %zu, got %zu", buf->bytes, bytes);
    EB_CHECK_CUDA(cudaSetDevice(buf->dev->index));
    if (bytes) EB_CHECK_CUDA(cudaMemcpyAsync(host, buf->storage->ptr, bytes, cudaMemcpyDeviceToHost, buf->dev->stream));
    if (sync) {
        EB_CHECK_CUDA(cudaStreamSynchronize(buf->dev->stream));
        return check_device_flag(buf->dev);
    }
    return EB200_OK;
}

int eb200_buffer_write(eb200_buffer* buf, const void* host, size_t bytes) { return buffer_write(buf, host, bytes, true); }
int eb200_buffer_read(eb200_buffer* buf, void* host, size_t bytes) { return buffer_read(buf, host, bytes, true); }
int eb200_buffer_write_async(eb200_buffer* buf, const void* host, size_t bytes) { return buffer_write(buf, host, bytes, false); }
int eb200_buffer_read_async(eb200_buffer* buf, void* host, size_t bytes) { return buffer_read(buf, host, bytes, false); }

int eb200_buffer_clone(eb200_buffer* buf, eb200_buffer** out) {
    EB_REQUIRE(buf && out, EB200_ERR_INVALID, "null argument");
    auto b = new eb200_buffer();
    b->dev = buf->dev;
    b->bytes = buf->bytes;
    b->storage = buf->storage;
    *out = b;
    return EB200_OK;
}

int eb200_buffer_device_ptr(eb200_buffer* buf, void** ptr) {
    EB_REQUIRE(buf && ptr, EB200_ERR_INVALID, "null argument");
    EB_CHECK_CUDA(cudaSetDevice(buf->dev->index));
    int st = buffer_unshare(buf, true);
    if (st) return st;
    *ptr = buf->storage->ptr;
    return EB200_OK;
}

int eb200_host_alloc(size_t bytes, void** ptr) {
    EB_REQUIRE(ptr, EB200_ERR_INVALID, "ptr is null");
    EB_CHECK_CUDA(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocDefault));
    return EB200_OK;
}

int eb200_host_free(void* ptr) {
    if (ptr) EB_CHECK_CUDA(cudaFreeHost(ptr));
    return EB200_OK;
}

int eb200_launch_count(int64_t* count) {
    EB_REQUIRE(count, EB200_ERR_INVALID, "count is null");
    *count = g_launch_count.load();
    return EB200_OK;
}

}  // extern "C"
