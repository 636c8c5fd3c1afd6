// The exchange step of the tensor-parallel decoder as ONE kernel over peer memory: the sum over ranks of a
// row-parallel Linear's partial outputs, fused with bias + residual + LayerNorm + int8 row quantisation (the input of
// the next product).  It replaces, per half-layer, an NCCL all-reduce, the bias + residual kernel and the LayerNorm ->
// int8 kernel.  The reference has no multi-GPU code (its only cross-device move is Tensor.To through a host array,
// src/NeuralSharp/Tensor.cs:244-253); the arithmetic is that of x + Linear(...) followed by LayerNorm
// (src/NeuralSharp/Layers/Attention.cs:201-205; layernorm_fused_f32, Backends/Cuda/PtxKernels.Decoding.cs:61-90).
//
// One process per GPU.  Every rank allocates one block (flags + two slots of float partial sums), exports it as an IPC
// handle, and maps the blocks of its peers.  A half-layer: the product writes this rank's dequantised partial rows
// (float, no bias) into its own slot; the fused kernel then
//   1. tells every peer "my slot holds epoch e" by storing e into word [my rank] of the PEER's flag array
//      (st.release.sys after a system fence; the product finished before this kernel started: stream order),
//   2. waits until its own flag array shows epoch e for every rank (ld.acquire.sys, bounded: a peer that never arrives
//      costs about a second, then the kernel reports through the status word and returns),
//   3. per row: adds the ranks' partial rows in rank order (plain peer loads that bypass L1: the same addresses are
//      re-read every layer), so every rank computes bit-identical sums; adds bias and residual, rounds to bf16, writes
//      the residual stream, normalises and quantises the row in registers,
//   4. the last CTA to finish advances the slot's epoch (device-side state, so a captured graph replays correctly).
// Two slots alternate (attention output projection / second feed-forward product): a rank overwrites slot A for layer
// l+1 only after its own wait on slot B of layer l, and a peer signals slot B only after it has read slot A of layer
// l, so no partial sum is overwritten while a peer still reads it.  No multicast, no NVLS objects: plain loads and
// stores over NVLink.
#include <string.h>

#include "ns_rows.cuh"
#include "ns_tail.cuh"

namespace {

constexpr int PEER_MAX = 8;
constexpr int PEER_SLOTS = 2;
constexpr size_t PEER_HEADER = 1024;      // flags [PEER_SLOTS][PEER_MAX] uint32 at the start of the block

struct NsPeerGroup {
    NsDevice* dev = nullptr;
    int rank = 0, world = 1;
    size_t slot_bytes = 0;
    uint8_t* local = nullptr;                    // this rank's block
    uint8_t* peers[PEER_MAX] = {nullptr};        // every rank's block as mapped here (peers[rank] == local)
    uint32_t* state = nullptr;                   // local only: epoch[PEER_SLOTS], ticket[PEER_SLOTS]
    bool connected = false;
    bool loopback = false;                       // peers are stand-ins mapped to the local block
};

struct PeerReduceParams {
    const float* part[PEER_MAX];      // slot data of every rank
    uint32_t* remote_flag[PEER_MAX];  // word [my rank] of every rank's flag array for this slot
    const uint32_t* local_flags;      // this rank's flag array for this slot
    uint32_t* epoch;
    uint32_t* ticket;
    int rank, world;
    const float* bias;
    const uint16_t* residual;
    int64_t rows;
    int cols;
    uint16_t* x_out;
    const float* gamma;
    const float* beta;
    float eps;
    int8_t* q;
    float* q_scale;
    int* status;
};

__device__ __forceinline__ float4 peer_load4(const float* ptr)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr) : "memory");
    return v;
}

template <int VPT>
__global__ void ns_tp_reduce_norm_quant_kernel(const PeerReduceParams p)
{
    __shared__ ns_rows::RowShared sh;
    __shared__ int give_up;
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.epoch) + 1u;
    if (threadIdx.x == 0) give_up = 0;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.remote_flag[threadIdx.x]), "r"(e) : "memory");
    }
    __syncthreads();
    if (threadIdx.x < p.world) {
        // bounded wait for rank threadIdx.x: about a second, then report and leave
        const long long t0 = clock64();
        uint32_t seen = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.local_flags + threadIdx.x) : "memory");
            if ((int32_t)(seen - e) >= 0) break;
            if (clock64() - t0 > NS_WAIT_LIMIT_CYCLES) {
                *reinterpret_cast<volatile int*>(p.status) = 400 + (int)threadIdx.x;
                give_up = 1;
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    if (give_up == 0) {
        for (int64_t r = blockIdx.x; r < p.rows; r += gridDim.x) {
            float v[VPT * 8];
#pragma unroll
            for (int j = 0; j < VPT; j++) {
                const int col = ns_rows::vec_col(j);
                const size_t idx = (size_t)r * p.cols + col;
                // every rank's vectors are requested before the first is used: one NVLink round trip, not one per rank
                float4 va[PEER_MAX], vb[PEER_MAX];
#pragma unroll
                for (int k = 0; k < PEER_MAX; k++) {
                    if (k < p.world) {
                        va[k] = peer_load4(p.part[k] + idx);
                        vb[k] = peer_load4(p.part[k] + idx + 4);
                    }
                }
                float t[8] = {va[0].x, va[0].y, va[0].z, va[0].w, vb[0].x, vb[0].y, vb[0].z, vb[0].w};
#pragma unroll
                for (int k = 1; k < PEER_MAX; k++) {
                    if (k < p.world) {
                        t[0] = __fadd_rn(t[0], va[k].x); t[1] = __fadd_rn(t[1], va[k].y); t[2] = __fadd_rn(t[2], va[k].z); t[3] = __fadd_rn(t[3], va[k].w);
                        t[4] = __fadd_rn(t[4], vb[k].x); t[5] = __fadd_rn(t[5], vb[k].y); t[6] = __fadd_rn(t[6], vb[k].z); t[7] = __fadd_rn(t[7], vb[k].w);
                    }
                }
                if (p.bias != nullptr) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + col)), b1 = __ldg(reinterpret_cast<const float4*>(p.bias + col + 4));
                    const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                    for (int i = 0; i < 8; i++) t[i] = __fadd_rn(t[i], bs[i]);
                }
                if (p.residual != nullptr) {
                    float rs[8];
                    ns_rows::widen8(*reinterpret_cast<const uint4*>(p.residual + idx), rs);
#pragma unroll
                    for (int i = 0; i < 8; i++) t[i] = __fadd_rn(t[i], rs[i]);
                }
                const uint4 packed = make_uint4(ns_pack_bf16x2(t[0], t[1]), ns_pack_bf16x2(t[2], t[3]), ns_pack_bf16x2(t[4], t[5]), ns_pack_bf16x2(t[6], t[7]));
                *reinterpret_cast<uint4*>(p.x_out + idx) = packed;
                float xr[8];
                ns_rows::widen8(packed, xr);
#pragma unroll
                for (int i = 0; i < 8; i++) v[j * 8 + i] = xr[i];
            }
            if (p.gamma != nullptr) ns_rows::layernorm_quantize_row<VPT>(v, p.gamma, p.beta, p.eps, p.cols, p.q + (size_t)r * p.cols, p.q_scale + r, sh);
            __syncthreads();
        }
    }
    // the epoch advances whether or not the wait succeeded, so that the ranks stay in step
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(p.ticket, 1u);
        if (t == gridDim.x - 1) {
            *p.ticket = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(p.epoch) = e;
        }
    }
}

NsPeerGroup* as_group(ns_peer_group_t h) { return reinterpret_cast<NsPeerGroup*>(h); }

}  // namespace

extern "C" int ns_peer_group_create(ns_device_t h, int rank, int world, uint64_t slot_bytes, ns_peer_group_t* out)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(out != nullptr && world >= 1 && world <= PEER_MAX && rank >= 0 && rank < world, NS_ERR_ARGUMENT,
               "ns_peer_group_create: rank %d of %d (at most %d ranks)", rank, world, PEER_MAX);
    NS_REQUIRE(slot_bytes > 0 && slot_bytes % 256 == 0, NS_ERR_ARGUMENT, "ns_peer_group_create: slot size must be a multiple of 256 bytes");
    NsPeerGroup* g = new NsPeerGroup();
    g->dev = d; g->rank = rank; g->world = world; g->slot_bytes = slot_bytes;
    const size_t total = PEER_HEADER + PEER_SLOTS * slot_bytes;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&g->local), total);
    if (e == cudaSuccess) e = cudaMemset(g->local, 0, total);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&g->state), 256);
    if (e == cudaSuccess) e = cudaMemset(g->state, 0, 256);
    if (e != cudaSuccess) {
        if (g->local) cudaFree(g->local);
        if (g->state) cudaFree(g->state);
        delete g;
        return ns_fail(NS_ERR_MEMORY, "ns_peer_group_create: %s", cudaGetErrorString(e));
    }
    g->peers[rank] = g->local;
    g->connected = world == 1;
    *out = reinterpret_cast<ns_peer_group_t>(g);
    return NS_OK;
}

extern "C" int ns_peer_group_handle(ns_peer_group_t h, void* handle64)
{
    NsPeerGroup* g = as_group(h);
    NS_REQUIRE(g != nullptr && handle64 != nullptr, NS_ERR_ARGUMENT, "ns_peer_group_handle: null argument");
    int rc = ns_device_make_current(g->dev);
    if (rc != NS_OK) return rc;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t ipc;
    NS_CUDA(cudaIpcGetMemHandle(&ipc, g->local));
    memcpy(handle64, &ipc, 64);
    return NS_OK;
}

extern "C" int ns_peer_group_connect(ns_peer_group_t h, const void* handles)
{
    NsPeerGroup* g = as_group(h);
    NS_REQUIRE(g != nullptr, NS_ERR_ARGUMENT, "ns_peer_group_connect: null argument");
    int rc = ns_device_make_current(g->dev);
    if (rc != NS_OK) return rc;
    for (int r = 0; r < g->world; r++) {
        if (r == g->rank || g->peers[r] != nullptr) continue;
        if (handles == nullptr) {
            // no handles: the other ranks are stand-ins that never arrive (their flag words are never written); this is
            // how the bounded wait is exercised on one GPU
            g->peers[r] = g->local;
            g->loopback = true;
            continue;
        }
        cudaIpcMemHandle_t ipc;
        memcpy(&ipc, reinterpret_cast<const uint8_t*>(handles) + 64 * r, 64);
        void* ptr = nullptr;
        NS_CUDA(cudaIpcOpenMemHandle(&ptr, ipc, cudaIpcMemLazyEnablePeerAccess));
        g->peers[r] = reinterpret_cast<uint8_t*>(ptr);
    }
    g->connected = true;
    return NS_OK;
}

extern "C" int ns_peer_group_slot(ns_peer_group_t h, int slot, uint64_t* ptr)
{
    NsPeerGroup* g = as_group(h);
    NS_REQUIRE(g != nullptr && ptr != nullptr && slot >= 0 && slot < PEER_SLOTS, NS_ERR_ARGUMENT, "ns_peer_group_slot: bad argument");
    *ptr = reinterpret_cast<uint64_t>(g->local + PEER_HEADER + (size_t)slot * g->slot_bytes);
    return NS_OK;
}

extern "C" int ns_tp_reduce_norm_quant(ns_device_t dh, ns_peer_group_t h, int slot, uint64_t bias, uint64_t residual, int64_t rows, int cols,
                                       uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q, uint64_t q_scale)
{
    NsDevice* d = ns_dev(dh);
    NsPeerGroup* g = as_group(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(g != nullptr && g->dev == d && g->connected, NS_ERR_ARGUMENT, "ns_tp_reduce_norm_quant: the peer group is not connected on this device");
    NS_REQUIRE(slot >= 0 && slot < PEER_SLOTS && rows > 0 && x_out != 0, NS_ERR_ARGUMENT, "ns_tp_reduce_norm_quant: bad argument");
    NS_REQUIRE((size_t)rows * cols * 4 <= g->slot_bytes, NS_ERR_ARGUMENT, "ns_tp_reduce_norm_quant: %lld x %d floats exceed the slot", (long long)rows, cols);
    NS_REQUIRE(gamma == 0 || (beta != 0 && q != 0 && q_scale != 0), NS_ERR_ARGUMENT, "ns_tp_reduce_norm_quant: LayerNorm needs beta, q and q_scale");
    unsigned threads;
    int vpt;
    NS_REQUIRE(ns_rows::row_shape(cols, &threads, &vpt), NS_ERR_ARGUMENT, "ns_tp_reduce_norm_quant: cols = %d must be a multiple of 256 up to 8192", cols);
    // every CTA must be resident while it waits for the peers: at most one per SM
    NS_REQUIRE(rows <= (int64_t)d->sm_count * 64, NS_ERR_ARGUMENT, "ns_tp_reduce_norm_quant: too many rows");
    PeerReduceParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < g->world; r++) {
        p.part[r] = reinterpret_cast<const float*>(g->peers[r] + PEER_HEADER + (size_t)slot * g->slot_bytes);
        p.remote_flag[r] = reinterpret_cast<uint32_t*>(g->peers[r]) + slot * PEER_MAX + g->rank;
    }
    p.local_flags = reinterpret_cast<const uint32_t*>(g->local) + slot * PEER_MAX;
    p.epoch = g->state + slot;
    p.ticket = g->state + PEER_SLOTS + slot;
    p.rank = g->rank; p.world = g->world;
    p.bias = reinterpret_cast<const float*>(bias);
    p.residual = reinterpret_cast<const uint16_t*>(residual);
    p.rows = rows; p.cols = cols;
    p.x_out = reinterpret_cast<uint16_t*>(x_out);
    p.gamma = reinterpret_cast<const float*>(gamma);
    p.beta = reinterpret_cast<const float*>(beta);
    p.eps = eps;
    p.q = reinterpret_cast<int8_t*>(q);
    p.q_scale = reinterpret_cast<float*>(q_scale);
    p.status = d->status_dev;
    const dim3 grid((unsigned)(rows < d->sm_count ? rows : d->sm_count)), block(threads);
    switch (vpt) {
        case 1: NS_CUDA(ns_launch_plain(ns_tp_reduce_norm_quant_kernel<1>, grid, block, 0, d->stream, p)); break;
        case 2: NS_CUDA(ns_launch_plain(ns_tp_reduce_norm_quant_kernel<2>, grid, block, 0, d->stream, p)); break;
        default: NS_CUDA(ns_launch_plain(ns_tp_reduce_norm_quant_kernel<4>, grid, block, 0, d->stream, p)); break;
    }
    return NS_OK;
}

// The exchange of `slot` as the second phase of a product launch (ns_tail.cuh, NS_TAIL_PEER): fills the peer fields of
// `t` and returns the address the product must write this rank's float partial rows to.
int ns_peer_fill_tail(ns_peer_group_t h, NsDevice* d, int slot, int64_t rows, int cols, NsTail* t, void** slot_ptr)
{
    NsPeerGroup* g = as_group(h);
    NS_REQUIRE(g != nullptr && g->dev == d && g->connected, NS_ERR_ARGUMENT, "the peer group is not connected on this device");
    NS_REQUIRE(slot >= 0 && slot < PEER_SLOTS && rows > 0, NS_ERR_ARGUMENT, "bad exchange slot or row count");
    NS_REQUIRE((size_t)rows * cols * 4 <= g->slot_bytes, NS_ERR_ARGUMENT, "%lld x %d floats exceed the exchange slot", (long long)rows, cols);
    static_assert(PEER_MAX == NS_TAIL_PEER_MAX, "peer limits");
    for (int r = 0; r < PEER_MAX; r++) { t->part[r] = nullptr; t->remote_flag[r] = nullptr; }
    for (int r = 0; r < g->world; r++) {
        t->part[r] = reinterpret_cast<const float*>(g->peers[r] + PEER_HEADER + (size_t)slot * g->slot_bytes);
        t->remote_flag[r] = reinterpret_cast<uint32_t*>(g->peers[r]) + slot * PEER_MAX + g->rank;
    }
    t->local_flags = reinterpret_cast<const uint32_t*>(g->local) + slot * PEER_MAX;
    t->epoch = g->state + slot;
    t->rank = g->rank;
    t->world = g->world;
    *slot_ptr = g->local + PEER_HEADER + (size_t)slot * g->slot_bytes;
    return NS_OK;
}

extern "C" int ns_peer_group_destroy(ns_peer_group_t h)
{
    NsPeerGroup* g = as_group(h);
    if (g == nullptr) return NS_OK;
    ns_device_make_current(g->dev);
    cudaStreamSynchronize(g->dev->stream);
    for (int r = 0; r < g->world; r++)
        if (r != g->rank && g->peers[r] != nullptr && !g->loopback) cudaIpcCloseMemHandle(g->peers[r]);
    if (g->local) cudaFree(g->local);
    if (g->state) cudaFree(g->state);
    delete g;
    return NS_OK;
}
