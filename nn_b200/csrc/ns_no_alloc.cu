// ns_qmatmul_i8_static: the int8 product for callers that must not cause a device allocation.
//
// The regular entry point (ns_qmatmul_i8) keeps the partial sums of a K-split product in the device object's
// scratch block, which it grows with cudaMalloc the first time a shape needs more room.  Two kinds of host cannot
// live with that: one that records its decode step into a CUDA graph without a warm-up run (memory cannot be
// allocated while a stream is being captured, so the growth request is refused), and one that budgets device memory
// itself -- NeuralSharp accounts every block against ComputeResources.GpuMemoryLimit, and a library that allocates
// behind its back breaks that accounting.  For them the partial sums live in the fixed array below.
//
// What that costs and what the caller must know:
//   - the array is part of the library image: every GPU whose context loads the library holds
//     NS_STATIC_SCRATCH_BYTES of device memory until the process ends;
//   - a shape whose partial sums (k_splits * M * N * 4 bytes) exceed it is rejected with NS_ERR_MEMORY, nothing runs;
//   - the first call on a device looks up the array's device address (cudaGetSymbolAddress) -- make that first call
//     outside any stream capture; later calls do no set-up;
//   - all calls on a device share the array and it keeps whatever the last call left there.  Nothing has to start
//     at zero (every split overwrites its own [M, N] slab before the finishing kernel reads it), but two calls that
//     overlap on the GPU (different streams, or graph branches that run side by side) would overwrite each other's
//     partial sums: keep them on one stream or otherwise ordered;
//   - no cudaMalloc, cudaFree or other allocating call is made, on any path.
#include "ns_gemm.cuh"

#define NS_STATIC_SCRATCH_BYTES (8u << 20)

// In host code this name is only a handle for the runtime's symbol table, not an address a kernel could use; the
// device address is fetched once per device below.
static __device__ __align__(256) unsigned char ns_static_scratch[NS_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_lock;
void* g_static_addr[64] = {nullptr};

int static_scratch_address(NsDevice* d, void** out)
{
    NS_REQUIRE(d->ordinal >= 0 && d->ordinal < 64, NS_ERR_ARGUMENT, "device ordinal %d out of range", d->ordinal);
    std::lock_guard<std::mutex> guard(g_static_lock);
    if (g_static_addr[d->ordinal] == nullptr) {
        void* p = nullptr;
        // the device was made current by the caller (ns_device_make_current)
        cudaError_t e = cudaGetSymbolAddress(&p, ns_static_scratch);
        NS_REQUIRE(e == cudaSuccess && p != nullptr, NS_ERR_CUDA, "cudaGetSymbolAddress(ns_static_scratch) failed: %s (%d)",
                   cudaGetErrorName(e), (int)e);
        g_static_addr[d->ordinal] = p;
    }
    *out = g_static_addr[d->ordinal];
    return NS_OK;
}
}  // namespace

extern "C" int ns_qmatmul_i8_static(ns_device_t h, uint64_t aq, uint64_t a_scale, uint64_t wq, uint64_t w_scale, uint64_t bias,
                                    uint64_t residual, int residual_dtype, int M, int N, int K, int epilogue, int out_dtype, uint64_t y)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(aq && wq && a_scale && w_scale && y, NS_ERR_ARGUMENT, "ns_qmatmul_i8_static: null operand");
    NS_REQUIRE(epilogue >= NS_EPI_NONE && epilogue <= NS_EPI_BIAS_RESIDUAL, NS_ERR_ARGUMENT, "ns_qmatmul_i8_static: unknown epilogue %d", epilogue);
    NS_REQUIRE(epilogue == NS_EPI_NONE || bias != 0, NS_ERR_ARGUMENT, "ns_qmatmul_i8_static: epilogue %d needs a bias vector", epilogue);
    NS_REQUIRE(epilogue != NS_EPI_BIAS_RESIDUAL || residual != 0, NS_ERR_ARGUMENT, "ns_qmatmul_i8_static: NS_EPI_BIAS_RESIDUAL needs a residual");
    NS_REQUIRE(out_dtype == NS_F32 || out_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_qmatmul_i8_static: output must be NS_F32 or NS_BF16");
    NS_REQUIRE(residual_dtype == NS_F32 || residual_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_qmatmul_i8_static: residual dtype must be NS_F32 or NS_BF16");
    NS_REQUIRE(M > 0 && N > 0 && K > 0, NS_ERR_ARGUMENT, "ns_qmatmul_i8_static: empty dimension");
    // size check first, so that an oversized request fails before anything is queued
    // (the split count the launcher ends up with: the requested count shrinks when the k-blocks do not divide evenly;
    // one to eight rows take the row-streaming kernel and nine to sixteen the streaming kernel, which have no partial sums)
    int tile_n = 0, splits = 1;
    const int k_blocks = (K + 127) / 128;
    ns_gemm_choose_tiling(d, M, N, k_blocks, &tile_n, &splits);
    const int kb_per_split = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + kb_per_split - 1) / kb_per_split;
    const bool streams_rows = d->force_bn == 0 && d->force_splits == 0 && (ns_gemv_i8_fits(M, K) || ns_stream_i8_fits(M, K)) && ((aq | wq) & 15) == 0;
    const size_t need = (splits > 1 && !streams_rows) ? (size_t)splits * M * N * 4 : 0;
    NS_REQUIRE(need <= NS_STATIC_SCRATCH_BYTES, NS_ERR_MEMORY,
               "ns_qmatmul_i8_static: M=%d N=%d K=%d splits K %d ways and needs %zu bytes of partial sums; the fixed scratch array holds %u",
               M, N, K, splits, need, (unsigned)NS_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    rc = static_scratch_address(d, &scratch);
    if (rc != NS_OK) return rc;
    NsGemmParams p = {};
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.residual_dtype = residual_dtype;
    p.out = reinterpret_cast<void*>(y);
    p.a_scale = reinterpret_cast<const float*>(a_scale);
    p.w_scale = reinterpret_cast<const float*>(w_scale);
    p.bias = reinterpret_cast<const float*>(bias);
    p.residual = reinterpret_cast<const void*>(residual);
    return ns_gemm_run(d, NS_KIND_I8, reinterpret_cast<const void*>(aq), reinterpret_cast<const void*>(wq), false, M, N, K, p, scratch,
                       NS_STATIC_SCRATCH_BYTES);
}
