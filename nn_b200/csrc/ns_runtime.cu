// Runtime part of libns_b200: error text, device objects, memory, copies, CUDA graphs, tensor maps.
// The counterpart in the reference is the host half of its GPU backend
// (src/NeuralSharp/Backends/Cuda/CudaBackend.cs:48-301, CudaBackend.Decoding.cs:43-130).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ns_common.cuh"

// ------------------------------------------------------------------------------------------------
// errors
// ------------------------------------------------------------------------------------------------
static thread_local char g_last_error[512] = "";

int ns_fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char* ns_last_error(void) { return g_last_error; }

extern "C" const char* ns_error_name(int code)
{
    switch (code) {
        case NS_OK: return "NS_OK";
        case NS_ERR_CUDA: return "NS_ERR_CUDA";
        case NS_ERR_ARGUMENT: return "NS_ERR_ARGUMENT";
        case NS_ERR_MEMORY: return "NS_ERR_MEMORY";
        case NS_ERR_KERNEL: return "NS_ERR_KERNEL";
        case NS_ERR_COMM: return "NS_ERR_COMM";
        case NS_ERR_STATE: return "NS_ERR_STATE";
        default: return "NS_ERR_UNKNOWN";
    }
}

bool ns_pdl_enabled()
{
    static int state = -1;
    if (state < 0) {
        const char* e = getenv("NS_B200_PDL");
        state = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

extern "C" int ns_version(void) { return 100; }

// ------------------------------------------------------------------------------------------------
// devices
// ------------------------------------------------------------------------------------------------
extern "C" int ns_device_count(int* count)
{
    NS_REQUIRE(count != nullptr, NS_ERR_ARGUMENT, "ns_device_count: count is null");
    NS_CUDA(cudaGetDeviceCount(count));
    return NS_OK;
}

int ns_device_make_current(NsDevice* d)
{
    // The reference binds its context on every entry (CudaBackend.MakeCurrent, CudaBackend.cs:176-183).
    NS_REQUIRE(d != nullptr, NS_ERR_ARGUMENT, "device handle is null");
    NS_CUDA(cudaSetDevice(d->ordinal));
    return NS_OK;
}

static int open_device(int ordinal, bool own_stream, cudaStream_t stream, ns_device_t* out)
{
    NS_REQUIRE(out != nullptr, NS_ERR_ARGUMENT, "ns_device_open: out handle is null");
    int count = 0;
    NS_CUDA(cudaGetDeviceCount(&count));
    NS_REQUIRE(ordinal >= 0 && ordinal < count, NS_ERR_ARGUMENT, "ns_device_open: ordinal %d out of range (%d devices)", ordinal, count);
    NS_CUDA(cudaSetDevice(ordinal));
    cudaDeviceProp prop;
    NS_CUDA(cudaGetDeviceProperties(&prop, ordinal));
    NS_REQUIRE(prop.major == 10, NS_ERR_ARGUMENT,
               "ns_device_open: device %d is sm_%d%d; this library holds sm_100a code only", ordinal, prop.major, prop.minor);
    NsDevice* d = new NsDevice();
    d->ordinal = ordinal;
    d->sm_count = prop.multiProcessorCount;
    d->owns_stream = own_stream;
    if (own_stream) {
        cudaError_t e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) { delete d; return ns_fail(NS_ERR_CUDA, "cudaStreamCreate failed: %s (%d)", cudaGetErrorName(e), (int)e); }
    } else {
        d->stream = stream;
    }
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&d->status_host), NS_STATUS_WORDS * sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&d->status_dev), d->status_host, 0);
    if (e != cudaSuccess) {
        if (own_stream) cudaStreamDestroy(d->stream);
        delete d;
        return ns_fail(NS_ERR_CUDA, "status block allocation failed: %s (%d)", cudaGetErrorName(e), (int)e);
    }
    memset(d->status_host, 0, NS_STATUS_WORDS * sizeof(int));
    e = cudaMalloc(reinterpret_cast<void**>(&d->sync_words), NS_SYNC_WORDS * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(d->sync_words, 0, NS_SYNC_WORDS * sizeof(uint32_t));
    if (e != cudaSuccess) {
        if (d->sync_words) cudaFree(d->sync_words);
        cudaFreeHost(d->status_host);
        if (own_stream) cudaStreamDestroy(d->stream);
        delete d;
        return ns_fail(NS_ERR_MEMORY, "synchronisation words: %s (%d)", cudaGetErrorName(e), (int)e);
    }
    *out = reinterpret_cast<ns_device_t>(d);
    return NS_OK;
}

extern "C" int ns_device_open(int ordinal, ns_device_t* dev) { return open_device(ordinal, true, nullptr, dev); }

extern "C" int ns_device_open_on_stream(int ordinal, uint64_t stream, ns_device_t* dev)
{
    return open_device(ordinal, false, reinterpret_cast<cudaStream_t>(stream), dev);
}

extern "C" int ns_device_close(ns_device_t h)
{
    NsDevice* d = ns_dev(h);
    if (d == nullptr) return NS_OK;
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    cudaStreamSynchronize(d->stream);
    if (d->host_pipe && d->host_pipe_free) d->host_pipe_free(d->host_pipe);
    if (d->scratch) cudaFree(d->scratch);
    for (void* p : d->retired_scratch) cudaFree(p);
    if (d->sync_words) cudaFree(d->sync_words);
    if (d->status_host) cudaFreeHost(d->status_host);
    if (d->owns_stream && d->stream) cudaStreamDestroy(d->stream);
    delete d;
    return NS_OK;
}

extern "C" int ns_device_info(ns_device_t h, char* name, int* sm_count, uint64_t* total_bytes, uint64_t* free_bytes)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    cudaDeviceProp prop;
    NS_CUDA(cudaGetDeviceProperties(&prop, d->ordinal));
    if (name) { strncpy(name, prop.name, 127); name[127] = 0; }
    if (sm_count) *sm_count = prop.multiProcessorCount;
    size_t fr = 0, tot = 0;
    NS_CUDA(cudaMemGetInfo(&fr, &tot));
    if (total_bytes) *total_bytes = tot;
    if (free_bytes) *free_bytes = fr;
    return NS_OK;
}

extern "C" int ns_device_stream(ns_device_t h, uint64_t* stream)
{
    NsDevice* d = ns_dev(h);
    NS_REQUIRE(d && stream, NS_ERR_ARGUMENT, "ns_device_stream: null argument");
    *stream = reinterpret_cast<uint64_t>(d->stream);
    return NS_OK;
}

extern "C" int ns_device_status(ns_device_t h, int* status)
{
    NsDevice* d = ns_dev(h);
    NS_REQUIRE(d && status, NS_ERR_ARGUMENT, "ns_device_status: null argument");
    *status = d->status_host[0];
    d->status_host[0] = 0;
    return NS_OK;
}

extern "C" int ns_stream_sync(ns_device_t h)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaStreamSynchronize(d->stream));
    int st = d->status_host[0];
    if (st != 0) {
        d->status_host[0] = 0;
        // a kernel that gave up may have left the arrival counters of the one-launch products half-way: start clean
        if (d->sync_words != nullptr && cudaMemsetAsync(d->sync_words, 0, NS_SYNC_WORDS * sizeof(uint32_t), d->stream) == cudaSuccess)
            cudaStreamSynchronize(d->stream);
        return ns_fail(NS_ERR_KERNEL, "a kernel gave up a bounded wait (status %d: kernel %d, role %d)", st, st / 100, st % 100);
    }
    return NS_OK;
}

extern "C" int ns_device_tune(ns_device_t h, int tile_n, int k_splits)
{
    NsDevice* d = ns_dev(h);
    NS_REQUIRE(d != nullptr, NS_ERR_ARGUMENT, "ns_device_tune: device is null");
    NS_REQUIRE(tile_n == 0 || tile_n == NS_TUNE_NARROW || tile_n == 64 || tile_n == 128 || tile_n == 256 || tile_n == NS_TUNE_PAIR ||
                   tile_n == NS_TUNE_DROP_ROW, NS_ERR_ARGUMENT,
               "ns_device_tune: tile_n must be 0, 64, 128, 256, NS_TUNE_NARROW, NS_TUNE_PAIR or NS_TUNE_DROP_ROW");
    NS_REQUIRE(k_splits >= 0 && k_splits <= 64, NS_ERR_ARGUMENT, "ns_device_tune: k_splits must be in [0, 64]");
    d->rows_drop = -1;
    if (tile_n == NS_TUNE_DROP_ROW) {
        d->rows_drop = k_splits;
        return NS_OK;
    }
    d->force_bn = tile_n;
    d->force_splits = k_splits;
    return NS_OK;
}

extern "C" int ns_debug_tail_times(ns_device_t h, uint64_t buffer)
{
    NsDevice* d = ns_dev(h);
    NS_REQUIRE(d != nullptr, NS_ERR_ARGUMENT, "ns_debug_tail_times: device is null");
    d->tail_times = reinterpret_cast<unsigned long long*>(buffer);
    return NS_OK;
}

int ns_scratch_reserve(NsDevice* d, size_t bytes, void** out)
{
    if (bytes > d->scratch_bytes) {
        NS_REQUIRE(!d->capturing, NS_ERR_STATE,
                   "scratch memory must grow to %zu bytes but the stream is being captured; run the step once before capturing", bytes);
        NS_CUDA(cudaStreamSynchronize(d->stream));
        if (d->scratch) {
            // graphs recorded earlier still name the old block: keep it until the last of them is destroyed
            if (d->live_graphs > 0) d->retired_scratch.push_back(d->scratch);
            else NS_CUDA(cudaFree(d->scratch));
        }
        d->scratch = nullptr;
        d->scratch_bytes = 0;
        size_t want = bytes + (bytes >> 2);
        NS_CUDA(cudaMalloc(&d->scratch, want));
        d->scratch_bytes = want;
    }
    *out = d->scratch;
    return NS_OK;
}

// ------------------------------------------------------------------------------------------------
// memory
// ------------------------------------------------------------------------------------------------
extern "C" int ns_alloc(ns_device_t h, uint64_t bytes, int zeroed, uint64_t* ptr)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(ptr != nullptr, NS_ERR_ARGUMENT, "ns_alloc: out pointer is null");
    NS_REQUIRE(!d->capturing, NS_ERR_STATE, "ns_alloc: not allowed while the stream is being captured");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes == 0 ? 16 : bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return ns_fail(NS_ERR_MEMORY, "cudaMalloc of %llu bytes failed: %s (%d)", (unsigned long long)bytes, cudaGetErrorName(e), (int)e);
    }
    if (zeroed) NS_CUDA(cudaMemsetAsync(p, 0, bytes, d->stream));
    *ptr = reinterpret_cast<uint64_t>(p);
    return NS_OK;
}

extern "C" int ns_free(ns_device_t h, uint64_t ptr)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    if (ptr == 0) return NS_OK;
    NS_REQUIRE(!d->capturing, NS_ERR_STATE, "ns_free: not allowed while the stream is being captured");
    NS_CUDA(cudaFree(reinterpret_cast<void*>(ptr)));
    return NS_OK;
}

extern "C" int ns_h2d(ns_device_t h, uint64_t dst, const void* src, uint64_t bytes)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(dst), src, bytes, cudaMemcpyHostToDevice, d->stream));
    NS_CUDA(cudaStreamSynchronize(d->stream));
    return NS_OK;
}

extern "C" int ns_d2h(ns_device_t h, void* dst, uint64_t src, uint64_t bytes)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaMemcpyAsync(dst, reinterpret_cast<const void*>(src), bytes, cudaMemcpyDeviceToHost, d->stream));
    NS_CUDA(cudaStreamSynchronize(d->stream));
    return NS_OK;
}

extern "C" int ns_h2d_async(ns_device_t h, uint64_t dst, const void* src, uint64_t bytes)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(dst), src, bytes, cudaMemcpyHostToDevice, d->stream));
    return NS_OK;
}

extern "C" int ns_d2h_async(ns_device_t h, void* dst, uint64_t src, uint64_t bytes)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaMemcpyAsync(dst, reinterpret_cast<const void*>(src), bytes, cudaMemcpyDeviceToHost, d->stream));
    return NS_OK;
}

extern "C" int ns_d2d_async(ns_device_t h, uint64_t dst, uint64_t src, uint64_t bytes)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes, cudaMemcpyDeviceToDevice, d->stream));
    return NS_OK;
}

extern "C" int ns_d2d_2d_async(ns_device_t h, uint64_t dst, uint64_t dst_pitch, uint64_t src, uint64_t src_pitch, uint64_t width_bytes, uint64_t rows)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    if (rows == 0 || width_bytes == 0) return NS_OK;
    NS_CUDA(cudaMemcpy2DAsync(reinterpret_cast<void*>(dst), dst_pitch, reinterpret_cast<const void*>(src), src_pitch, width_bytes, rows,
                              cudaMemcpyDeviceToDevice, d->stream));
    return NS_OK;
}

__global__ void ns_fill32_kernel(uint32_t* dst, uint32_t value, uint64_t count)
{
    uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; i < count; i += stride) dst[i] = value;
}

extern "C" int ns_memset32_async(ns_device_t h, uint64_t dst, uint32_t value, uint64_t count)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    if (count == 0) return NS_OK;
    NS_REQUIRE((dst & 3) == 0, NS_ERR_ARGUMENT, "ns_memset32_async: destination not 4-byte aligned");
    uint64_t blocks = (count + 255) / 256;
    if (blocks > (uint64_t)d->sm_count * 16) blocks = (uint64_t)d->sm_count * 16;
    ns_fill32_kernel<<<(unsigned)blocks, 256, 0, d->stream>>>(reinterpret_cast<uint32_t*>(dst), value, count);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_host_alloc(uint64_t bytes, void** ptr)
{
    NS_REQUIRE(ptr != nullptr, NS_ERR_ARGUMENT, "ns_host_alloc: out pointer is null");
    NS_CUDA(cudaHostAlloc(ptr, bytes == 0 ? 16 : bytes, cudaHostAllocDefault));
    return NS_OK;
}

extern "C" int ns_host_free(void* ptr)
{
    if (ptr) NS_CUDA(cudaFreeHost(ptr));
    return NS_OK;
}

// ------------------------------------------------------------------------------------------------
// memory shared between the processes of one machine (one process per GPU)
// ------------------------------------------------------------------------------------------------
extern "C" int ns_ipc_handle(ns_device_t h, uint64_t ptr, void* handle64)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(ptr != 0 && handle64 != nullptr, NS_ERR_ARGUMENT, "ns_ipc_handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t ipc;
    NS_CUDA(cudaIpcGetMemHandle(&ipc, reinterpret_cast<void*>(ptr)));
    memcpy(handle64, &ipc, 64);
    return NS_OK;
}

extern "C" int ns_ipc_open(ns_device_t h, const void* handle64, uint64_t* ptr)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(handle64 != nullptr && ptr != nullptr, NS_ERR_ARGUMENT, "ns_ipc_open: null argument");
    cudaIpcMemHandle_t ipc;
    memcpy(&ipc, handle64, 64);
    void* p = nullptr;
    NS_CUDA(cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess));
    *ptr = reinterpret_cast<uint64_t>(p);
    return NS_OK;
}

extern "C" int ns_ipc_close(ns_device_t h, uint64_t ptr)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    if (ptr == 0) return NS_OK;
    NS_CUDA(cudaStreamSynchronize(d->stream));
    NS_CUDA(cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)));
    return NS_OK;
}

// ------------------------------------------------------------------------------------------------
// graphs
// ------------------------------------------------------------------------------------------------
struct NsGraph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int ordinal = 0;
    NsDevice* dev = nullptr;
};

extern "C" int ns_capture_begin(ns_device_t h)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(!d->capturing, NS_ERR_STATE, "ns_capture_begin: a capture is already open");
    NS_CUDA(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeRelaxed));
    d->capturing = 1;
    return NS_OK;
}

extern "C" int ns_capture_end(ns_device_t h, ns_graph_t* out)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(d->capturing, NS_ERR_STATE, "ns_capture_end: no capture is open");
    NS_REQUIRE(out != nullptr, NS_ERR_ARGUMENT, "ns_capture_end: out handle is null");
    d->capturing = 0;
    NsGraph* g = new NsGraph();
    g->ordinal = d->ordinal;
    g->dev = d;
    cudaError_t e = cudaStreamEndCapture(d->stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        if (g->graph) cudaGraphDestroy(g->graph);
        delete g;
        cudaGetLastError();
        return ns_fail(NS_ERR_CUDA, "graph capture failed: %s (%d)", cudaGetErrorName(e), (int)e);
    }
    {
        std::lock_guard<std::mutex> guard(d->lock);
        d->live_graphs++;
    }
    *out = reinterpret_cast<ns_graph_t>(g);
    return NS_OK;
}

extern "C" int ns_capture_abort(ns_device_t h)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    if (!d->capturing) return NS_OK;
    d->capturing = 0;
    cudaGraph_t g = nullptr;
    cudaStreamEndCapture(d->stream, &g);
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    return NS_OK;
}

extern "C" int ns_graph_launch(ns_device_t h, ns_graph_t gh)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsGraph* g = reinterpret_cast<NsGraph*>(gh);
    NS_REQUIRE(g && g->exec, NS_ERR_ARGUMENT, "ns_graph_launch: graph is null");
    NS_CUDA(cudaGraphLaunch(g->exec, d->stream));
    return NS_OK;
}

extern "C" int ns_graph_destroy(ns_graph_t gh)
{
    NsGraph* g = reinterpret_cast<NsGraph*>(gh);
    if (!g) return NS_OK;
    cudaSetDevice(g->ordinal);
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    // Must be called before ns_device_close of the graph's device.  With the last graph gone nothing names a retired
    // scratch block any more (a replay still in flight is waited for first).
    if (NsDevice* d = g->dev) {
        std::lock_guard<std::mutex> guard(d->lock);
        if (--d->live_graphs <= 0) {
            d->live_graphs = 0;
            if (!d->retired_scratch.empty()) {
                cudaStreamSynchronize(d->stream);
                for (void* p : d->retired_scratch) cudaFree(p);
                d->retired_scratch.clear();
            }
        }
    }
    delete g;
    return NS_OK;
}

// ------------------------------------------------------------------------------------------------
// events (device-side timing on the device object's stream)
// ------------------------------------------------------------------------------------------------
extern "C" int ns_event_create(ns_device_t h, uint64_t* event)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(event != nullptr, NS_ERR_ARGUMENT, "ns_event_create: out pointer is null");
    cudaEvent_t e;
    NS_CUDA(cudaEventCreate(&e));
    *event = reinterpret_cast<uint64_t>(e);
    return NS_OK;
}

extern "C" int ns_event_record(ns_device_t h, uint64_t event)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), d->stream));
    return NS_OK;
}

// Work queued on `dev`'s stream after this call waits for `event` (recorded on any stream of the same GPU, for instance
// another device object's): how two device objects of one GPU order a hand-over without a host synchronisation.
extern "C" int ns_stream_wait_event(ns_device_t h, uint64_t event)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(event != 0, NS_ERR_ARGUMENT, "ns_stream_wait_event: event is null");
    NS_CUDA(cudaStreamWaitEvent(d->stream, reinterpret_cast<cudaEvent_t>(event), 0));
    return NS_OK;
}

extern "C" int ns_event_elapsed_ms(ns_device_t h, uint64_t start, uint64_t stop, float* ms)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(ms != nullptr, NS_ERR_ARGUMENT, "ns_event_elapsed_ms: out pointer is null");
    NS_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(stop)));
    NS_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(stop)));
    return NS_OK;
}

extern "C" int ns_event_destroy(ns_device_t h, uint64_t event)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    if (event) NS_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
    return NS_OK;
}

// ------------------------------------------------------------------------------------------------
// tensor maps
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int ns_make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle)
{
    static EncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        NS_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        NS_REQUIRE(fn != nullptr && q == cudaDriverEntryPointSuccess, NS_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    NS_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, NS_ERR_ARGUMENT, "tensor base address %p is not 16-byte aligned", base);
    cuuint64_t gdim[5];
    cuuint64_t gstride[5];
    cuuint32_t bdim[5];
    cuuint32_t estride[5];
    for (int i = 0; i < rank; i++) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estride[i] = 1;
        if (i > 0) {
            gstride[i - 1] = strides_bytes[i - 1];
            NS_REQUIRE((strides_bytes[i - 1] & 15) == 0, NS_ERR_ARGUMENT, "tensor stride %llu bytes is not a multiple of 16",
                       (unsigned long long)strides_bytes[i - 1]);
        }
    }
    CUresult r = encode(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NS_REQUIRE(r == CUDA_SUCCESS, NS_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return NS_OK;
}
