// Host-to-host Linear: float32 activations in host memory in, float32 result in host memory out.
//
// In the reference a caller holding host data pays three serial steps: Tensor.From -> Backend.Upload
// (src/NeuralSharp/Tensor.cs:87, Backends/Cuda/CudaBackend.cs:283-290), the layer's kernels, Tensor.ToArray ->
// Backend.Download (Tensor.cs:204, CudaBackend.cs:292-301), each waiting for the previous one.  The product itself takes
// ~0.1 ms for 8192 x 4096 x 4096 while each copy takes milliseconds, so end-to-end speed is the speed of the copies.
// Here the rows are cut into chunks that flow through three streams -- upload, quantise + product on the device's
// stream, download -- so the two copy directions run at the same time (they use separate copy engines and separate
// halves of the full-duplex host link) and the compute hides under them.  Steady state: max(upload, download) per
// chunk instead of upload + compute + download.
//
// Ordering: x_host is read from the moment of the call (it is host memory: the caller has it ready, as for any
// upload); the device's stream waits for the call's last download, so an event recorded after the call, or
// ns_stream_sync, covers the result.  Back-to-back calls overlap: the next call's first uploads run under the previous
// call's last products and downloads.
#include "ns_gemm.cuh"

struct NsLinear;   // ns_linear.cu
int ns_linear_forward_on(NsDevice* d, NsLinear* L, const void* x, const float* x_scale, int M, int epilogue, void* y);
int ns_linear_shape(NsLinear* L, int* K, int* N, int* mode, int* split_ranks);

namespace {

constexpr int SLOTS = 3;

struct NsHostPipe {
    cudaStream_t up = nullptr, down = nullptr;
    cudaEvent_t uploaded[SLOTS] = {}, x_free[SLOTS] = {}, computed[SLOTS] = {}, downloaded[SLOTS] = {};
    float* xf[SLOTS] = {};     // chunk of float activations
    int8_t* xq[SLOTS] = {};    // quantised (int8 layer) or bf16-converted (bf16 layer) chunk
    float* xs[SLOTS] = {};     // row scales
    float* y[SLOTS] = {};      // chunk of results
    size_t xf_bytes = 0, xq_bytes = 0, xs_bytes = 0, y_bytes = 0;
    unsigned long long next_slot = 0;
};

void pipe_free(void* p)
{
    NsHostPipe* h = static_cast<NsHostPipe*>(p);
    for (int s = 0; s < SLOTS; s++) {
        if (h->xf[s]) cudaFree(h->xf[s]);
        if (h->xq[s]) cudaFree(h->xq[s]);
        if (h->xs[s]) cudaFree(h->xs[s]);
        if (h->y[s]) cudaFree(h->y[s]);
        if (h->uploaded[s]) cudaEventDestroy(h->uploaded[s]);
        if (h->x_free[s]) cudaEventDestroy(h->x_free[s]);
        if (h->computed[s]) cudaEventDestroy(h->computed[s]);
        if (h->downloaded[s]) cudaEventDestroy(h->downloaded[s]);
    }
    if (h->up) cudaStreamDestroy(h->up);
    if (h->down) cudaStreamDestroy(h->down);
    delete h;
}

int pipe_get(NsDevice* d, NsHostPipe** out)
{
    if (!d->host_pipe) {
        NsHostPipe* h = new NsHostPipe();
        d->host_pipe = h;
        d->host_pipe_free = pipe_free;
        NS_CUDA(cudaStreamCreateWithFlags(&h->up, cudaStreamNonBlocking));
        NS_CUDA(cudaStreamCreateWithFlags(&h->down, cudaStreamNonBlocking));
        for (int s = 0; s < SLOTS; s++) {
            NS_CUDA(cudaEventCreateWithFlags(&h->uploaded[s], cudaEventDisableTiming));
            NS_CUDA(cudaEventCreateWithFlags(&h->x_free[s], cudaEventDisableTiming));
            NS_CUDA(cudaEventCreateWithFlags(&h->computed[s], cudaEventDisableTiming));
            NS_CUDA(cudaEventCreateWithFlags(&h->downloaded[s], cudaEventDisableTiming));
        }
    }
    *out = static_cast<NsHostPipe*>(d->host_pipe);
    return NS_OK;
}

template <typename T>
int grow(NsDevice* d, T** slot, size_t* have, size_t want)
{
    // called for all slots with the same `want`; *have is updated by the caller after the last slot
    if (*slot && *have >= want) return NS_OK;
    if (*slot) { NS_CUDA(cudaDeviceSynchronize()); NS_CUDA(cudaFree(*slot)); *slot = nullptr; }
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(slot), want);
    if (e != cudaSuccess) { cudaGetLastError(); return ns_fail(NS_ERR_MEMORY, "ns_linear_forward_host: %s for %zu staging bytes", cudaGetErrorName(e), want); }
    return NS_OK;
}

}  // namespace

extern "C" int ns_linear_forward_host(ns_device_t hd, ns_linear_t lh, const float* x_host, int M, int epilogue, float* y_host, int chunk_rows)
{
    NsDevice* d = ns_dev(hd);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsLinear* L = reinterpret_cast<NsLinear*>(lh);
    NS_REQUIRE(L && x_host && y_host, NS_ERR_ARGUMENT, "ns_linear_forward_host: null argument");
    NS_REQUIRE(M >= 0 && chunk_rows >= 0, NS_ERR_ARGUMENT, "ns_linear_forward_host: bad row count");
    NS_REQUIRE(epilogue == NS_EPI_NONE || epilogue == NS_EPI_BIAS || epilogue == NS_EPI_BIAS_GELU, NS_ERR_ARGUMENT,
               "ns_linear_forward_host: epilogue must be NS_EPI_NONE, NS_EPI_BIAS or NS_EPI_BIAS_GELU");
    NS_REQUIRE(!d->capturing, NS_ERR_STATE, "ns_linear_forward_host: uses several streams and cannot be captured");
    int K = 0, N = 0, mode = 0, ranks = 1;
    rc = ns_linear_shape(L, &K, &N, &mode, &ranks);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(ranks == 1, NS_ERR_ARGUMENT, "ns_linear_forward_host: the layer is a tensor-parallel shard");
    if (M == 0) return NS_OK;
    const bool ramp = chunk_rows == 0;
    if (chunk_rows == 0) {
        // chunks of about 32 MiB of the larger side: the host issues about ten calls per chunk, which costs as much
        // as a 2 MiB copy, so steady-state chunks must be much longer than that (measured at 8192 x 4096 x 4096:
        // 4 MiB chunks 36.8 GB/s each way, 16 MiB 44.2, 32 MiB 45.2, 64 MiB 44.9)
        const size_t row_bytes = sizeof(float) * (size_t)(K > N ? K : N);
        chunk_rows = (int)((32u << 20) / row_bytes);
        chunk_rows = chunk_rows < 128 ? 128 : (chunk_rows / 128) * 128;
    }
    if (chunk_rows > M) chunk_rows = M;

    NsHostPipe* p = nullptr;
    rc = pipe_get(d, &p);
    if (rc != NS_OK) return rc;
    const size_t el = mode == NS_I8 ? 1 : 2;
    const size_t want_xf = (size_t)chunk_rows * K * sizeof(float), want_xq = (size_t)chunk_rows * K * el;
    const size_t want_xs = (size_t)chunk_rows * sizeof(float), want_y = (size_t)chunk_rows * N * sizeof(float);
    for (int s = 0; s < SLOTS; s++) {
        if ((rc = grow(d, &p->xf[s], &p->xf_bytes, want_xf)) != NS_OK) return rc;
        if ((rc = grow(d, &p->xq[s], &p->xq_bytes, want_xq)) != NS_OK) return rc;
        if ((rc = grow(d, &p->xs[s], &p->xs_bytes, want_xs)) != NS_OK) return rc;
        if ((rc = grow(d, &p->y[s], &p->y_bytes, want_y)) != NS_OK) return rc;
    }
    if (p->xf_bytes < want_xf) p->xf_bytes = want_xf;
    if (p->xq_bytes < want_xq) p->xq_bytes = want_xq;
    if (p->xs_bytes < want_xs) p->xs_bytes = want_xs;
    if (p->y_bytes < want_y) p->y_bytes = want_y;

    // Chunk schedule.  With the automatic size the first and the last chunks are short (256, 512, 1024, ... rows): nothing
    // overlaps the first upload and the last download, so they should be brief.
    std::vector<int> sizes;
    if (ramp) {
        std::vector<int> tail;
        int left = M;
        for (int r = 256; r < chunk_rows && left >= 2 * r + chunk_rows; r *= 2) { sizes.push_back(r); tail.push_back(r); left -= 2 * r; }
        while (left > 0) { const int r = left < chunk_rows ? left : chunk_rows; sizes.push_back(r); left -= r; }
        for (size_t i = tail.size(); i-- > 0;) sizes.push_back(tail[i]);
    } else {
        for (int left = M; left > 0; left -= chunk_rows) sizes.push_back(left < chunk_rows ? left : chunk_rows);
    }

    // Slots are handed out round-robin across calls and their events persist, so a call's first uploads may run while
    // the previous call's last chunks are still being multiplied and downloaded: back-to-back calls form one pipeline.
    // (Waiting on an event that was never recorded returns at once.)
    int r0 = 0, last = 0;
    for (size_t c = 0; c < sizes.size(); c++) {
        const int s = (int)(p->next_slot++ % SLOTS);
        const int rows = sizes[c];
        // upload: the slot's float buffer is free once the chunk that used it was quantised
        NS_CUDA(cudaStreamWaitEvent(p->up, p->x_free[s], 0));
        NS_CUDA(cudaMemcpyAsync(p->xf[s], x_host + (size_t)r0 * K, (size_t)rows * K * sizeof(float), cudaMemcpyHostToDevice, p->up));
        NS_CUDA(cudaEventRecord(p->uploaded[s], p->up));
        // compute: the slot's result buffer is free once its previous chunk was downloaded
        NS_CUDA(cudaStreamWaitEvent(d->stream, p->uploaded[s], 0));
        NS_CUDA(cudaStreamWaitEvent(d->stream, p->downloaded[s], 0));
        if (mode == NS_I8)
            rc = ns_quantize_rows_i8(hd, reinterpret_cast<uint64_t>(p->xf[s]), NS_F32, rows, K, reinterpret_cast<uint64_t>(p->xq[s]),
                                     reinterpret_cast<uint64_t>(p->xs[s]));
        else
            rc = ns_convert(hd, reinterpret_cast<uint64_t>(p->xf[s]), NS_F32, reinterpret_cast<uint64_t>(p->xq[s]), NS_BF16, (int64_t)rows * K);
        if (rc != NS_OK) return rc;
        NS_CUDA(cudaEventRecord(p->x_free[s], d->stream));
        rc = ns_linear_forward_on(d, L, p->xq[s], mode == NS_I8 ? p->xs[s] : nullptr, rows, epilogue, p->y[s]);
        if (rc != NS_OK) return rc;
        NS_CUDA(cudaEventRecord(p->computed[s], d->stream));
        // download
        NS_CUDA(cudaStreamWaitEvent(p->down, p->computed[s], 0));
        NS_CUDA(cudaMemcpyAsync(y_host + (size_t)r0 * N, p->y[s], (size_t)rows * N * sizeof(float), cudaMemcpyDeviceToHost, p->down));
        NS_CUDA(cudaEventRecord(p->downloaded[s], p->down));
        r0 += rows;
        last = s;
    }
    // the download stream runs in order: its last event covers every chunk
    NS_CUDA(cudaStreamWaitEvent(d->stream, p->downloaded[last], 0));
    return NS_OK;
}
