// Shared declarations of libns_b200: error convention, the per-device object, PTX wrappers for the
// sm_100a features the kernels use (mbarrier, TMA tiled loads, tcgen05 MMA / TMEM).
//
// Error convention (mirrors the reference's CudaDriver.Check, src/NeuralSharp/Backends/Cuda/
// CudaDriver.cs:63-77): every exported function returns int, 0 = success; the text of the last
// failure of the calling thread is kept for ns_last_error().
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ns_b200.h"

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
int ns_fail(int code, const char* fmt, ...);  // records the message, returns code

#define NS_CUDA(call)                                                                          \
    do {                                                                                       \
        cudaError_t _e = (call);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return ns_fail(NS_ERR_CUDA, "%s failed: %s (%d)", #call, cudaGetErrorName(_e), (int)_e); \
    } while (0)

#define NS_REQUIRE(cond, code, ...)              \
    do {                                         \
        if (!(cond)) return ns_fail(code, __VA_ARGS__); \
    } while (0)

// Slots of the device status block kernels write to when a bounded wait gives up.
enum { NS_STATUS_WORDS = 16 };
// Device words for grid-wide phases: [0] arrivals, [1] departures of the product kernels' second phase;
// [NS_SYNC_ROW_TICKETS, +NS_SYNC_MAX_ROWS) one ticket per activation row for the decode attention's row quantisation.
enum { NS_SYNC_WORDS = 4096, NS_SYNC_ROW_TICKETS = 64, NS_SYNC_MAX_ROWS = 4000 };

struct NsDevice {
    int ordinal = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = true;
    int* status_host = nullptr;  // pinned, mapped; kernels write through status_dev
    int* status_dev = nullptr;
    // scratch memory for split-K partial sums and split-KV attention partials; grown on demand
    // outside stream capture, reused by every call on the device's stream.
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // A recorded graph keeps the scratch address it was captured with in its kernel arguments and tensor maps.  While
    // graphs of this device exist, a block that has to grow is retired (kept allocated) instead of freed, so those
    // graphs keep replaying on valid memory; retired blocks are freed when the last graph is destroyed.
    int live_graphs = 0;
    std::vector<void*> retired_scratch;
    // words for grid-wide phases inside one kernel (arrival counters, per-row tickets); zero between kernels
    uint32_t* sync_words = nullptr;
    unsigned long long* tail_times = nullptr;   // test hook (ns_debug_tail_times)
    // tuning overrides (0 = heuristic)
    int force_bn = 0;
    int force_splits = 0;
    int rows_drop = -1;     // test hook: the many-row kernels leave out the copy of this row (its group's wait then runs out)
    int capturing = 0;
    // streams, events and staging buffers of the host-to-host pipeline (ns_linear_forward_host); made on first use
    void* host_pipe = nullptr;
    void (*host_pipe_free)(void*) = nullptr;
    std::mutex lock;
};

int ns_device_make_current(NsDevice* d);
int ns_scratch_reserve(NsDevice* d, size_t bytes, void** out);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
// dims/strides innermost first; strides in bytes for dims 1..rank-1.
int ns_make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                       CUtensorMapSwizzle swizzle);

static inline NsDevice* ns_dev(ns_device_t h) { return reinterpret_cast<NsDevice*>(h); }

// Programmatic dependent launch: the kernel may start (set up barriers, allocate tensor memory, prefetch
// weights) while the previous kernel on the stream is still running; it must execute ns_pdl_wait() before it
// touches anything the previous kernel wrote or still reads.  NS_B200_PDL=0 in the environment turns it off.
bool ns_pdl_enabled();
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t ns_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ns_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Same call shape without the attribute, for kernels that have nothing to do before their inputs are ready (a
// programmatic edge costs about a microsecond per launch inside a graph and buys them nothing).  They still
// execute ns_pdl_trigger() so that a product launched after them can start early.
template <typename... KArgs, typename... Args>
inline cudaError_t ns_launch_plain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---------------------------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

#define NS_DEVINL __device__ __forceinline__

// About one second at 2 GHz: a wait that lasts this long records an error code and gives up.
constexpr long long NS_WAIT_LIMIT_CYCLES = 2000000000LL;

// Waits until the kernel this one depends on has completed and its writes are visible (no-op otherwise).
NS_DEVINL void ns_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// griddepcontrol.wait orders memory for the hardware; for the compiler it is an asm statement that clobbers memory, and a load
// the compiler knows to be from read-only memory (__ldg, a const __restrict__ pointer) may still be scheduled above it.  A
// kernel that does work before its wait passes every pointer to data of the kernel before it through this, after the
// wait: the pointer then comes out of an asm statement that follows the wait, and so do the loads through it.
template <class T>
NS_DEVINL const T* ns_after_wait(const T* ptr)
{
    asm volatile("" : "+l"(ptr) : : "memory");
    return ptr;
}
// Lets the next kernel on the stream start its prologue.
NS_DEVINL void ns_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

NS_DEVINL uint32_t ns_smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

NS_DEVINL void ns_mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
NS_DEVINL void ns_mbar_inval(uint32_t bar)
{
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
NS_DEVINL void ns_fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
NS_DEVINL void ns_fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
NS_DEVINL void ns_mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
NS_DEVINL void ns_mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
NS_DEVINL bool ns_mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` is a word in shared memory every role of the CTA polls: the first
// role whose wait runs out stores `code` to the device status block and raises the flag, the others
// leave their loops when they see it.  Returns false when the wait was given up.
NS_DEVINL bool ns_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code)
{
    if (ns_mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    uint32_t spins = 0;
    while (!ns_mbar_try_wait(bar, parity)) {
        if ((++spins & 0xFF) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > NS_WAIT_LIMIT_CYCLES) {
                *reinterpret_cast<volatile int*>(status) = code;  // plain store: the block is host memory
                *abort_flag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
    return true;
}

// TMA tiled loads, global -> this CTA's shared memory, completion counted on an mbarrier.
NS_DEVINL void ns_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
NS_DEVINL void ns_tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
// TMA tiled stores, this CTA's shared memory -> global, tracked by the issuing thread's bulk groups.
// Elements outside the tensor are clipped by the hardware.
NS_DEVINL void ns_tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
NS_DEVINL void ns_tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
NS_DEVINL void ns_tma_store_4d(const CUtensorMap* map, uint32_t src, int x, int y, int z, int w)
{
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
                 : "memory");
}
NS_DEVINL void ns_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of this thread's bulk groups are still reading shared memory
template <int N>
NS_DEVINL void ns_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// waits until at most N of this thread's bulk groups are incomplete
template <int N>
NS_DEVINL void ns_bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
NS_DEVINL void ns_st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

NS_DEVINL void ns_prefetch_tensormap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Tensor memory.
NS_DEVINL void ns_tmem_alloc(uint32_t slot_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
NS_DEVINL void ns_tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
NS_DEVINL void ns_tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
NS_DEVINL void ns_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
NS_DEVINL void ns_tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
NS_DEVINL void ns_tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
NS_DEVINL void ns_tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// All MMAs issued so far by this thread arrive on `bar` once they have completed.
NS_DEVINL void ns_tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- CTA pairs (clusters of two, tcgen05 cta_group::2): one thread of the even CTA issues MMAs that span both
// CTAs' shared and tensor memory.  A kernel uses either the cta_group::1 or the cta_group::2 forms, never both.
NS_DEVINL uint32_t ns_cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
NS_DEVINL void ns_cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
NS_DEVINL uint32_t ns_mapa(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
NS_DEVINL void ns_mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
NS_DEVINL uint32_t ns_ld_shared_cluster_u32(uint32_t cluster_addr)
{
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
    return v;
}
// TMA tiled load into this CTA's shared memory whose bytes are counted on an mbarrier of the pair's even CTA
// (`bar_cluster` is a shared::cluster address, from ns_mapa).
NS_DEVINL void ns_tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
// Executed by the same warp of both CTAs of the pair, with the same shared-memory offset.
NS_DEVINL void ns_tmem_alloc_pair(uint32_t slot_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
NS_DEVINL void ns_tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
NS_DEVINL void ns_tmem_dealloc_pair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// All MMAs issued so far by this thread arrive, once complete, on the mbarrier at this offset in every CTA of `mask`.
NS_DEVINL void ns_tc_commit_pair(uint32_t bar, uint16_t mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
                 : "memory");
}
NS_DEVINL void ns_mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
NS_DEVINL void ns_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
NS_DEVINL void ns_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
NS_DEVINL void ns_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
NS_DEVINL void ns_tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
NS_DEVINL void ns_tmem_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// Shared-memory matrix descriptors for tcgen05.mma (sm_100 format: version field = 1).
// Field offsets: start address [0,14), leading byte offset [16,30), stride byte offset [32,46) (all
// in 16-byte units), version [46,48), swizzle mode [61,64) (2 = 128-byte swizzle).
NS_DEVINL uint64_t ns_desc_base(uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    return (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
NS_DEVINL uint64_t ns_desc_at(uint64_t base, uint32_t smem_addr) { return base | uint64_t((smem_addr & 0x3FFFF) >> 4); }

// Instruction descriptor of kind::i8 / kind::f16: accumulator format [4,6) (1 = f32, 2 = s32), A format
// [7,10), B format [10,13) (f16 kinds: 1 = bf16; i8 kind: 1 = signed), A/B major [15],[16]
// (0 = K-major, 1 = MN-major), N>>3 at [17,23), M>>4 at [24,29).
NS_DEVINL constexpr uint32_t ns_idesc(uint32_t c_fmt, uint32_t ab_fmt, uint32_t a_mn, uint32_t b_mn, uint32_t m, uint32_t n)
{
    return (c_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

NS_DEVINL float ns_gelu_tanh(float v)
{
    // tanh approximation with the reference's constants (src/NeuralSharp/Backends/Cpu/
    // CpuBackend.Advanced.cs:770-772; GPU kernel bias_gelu_f32, Backends/Cuda/PtxKernels.Decoding.cs:93-114).
    const float k = 0.7978845608f, c = 0.044715f;
    float inner = __fmul_rn(k, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(c, v), v), v)));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner)));
}

// The same function for the epilogues of the int8 / bf16 products, where a tile's epilogue has to keep up with its main
// loop: 0.5 v (1 + tanh(u)) = v / (1 + exp(-2u)), one ex2.approx and one rcp.approx instead of tanhf (about 8 instructions
// against 30, no branch).  No cancellation anywhere, so the result is within about 1e-6 relative of the exact value on both
// tails; the float-output tests hold it to the oracle's tanhf form at 1e-5.
NS_DEVINL float ns_gelu_fast(float v)
{
    const float k2 = -2.0f * 0.7978845608f * 1.4426950408889634f, c = 0.044715f;
    const float arg = __fmul_rn(__fmul_rn(k2, v), fmaf(__fmul_rn(c, v), v, 1.0f));
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(arg));
    return __fdividef(v, __fadd_rn(1.0f, e));
}

NS_DEVINL float ns_bf16_bits_to_f32(uint16_t h) { return __uint_as_float(uint32_t(h) << 16); }
NS_DEVINL uint16_t ns_f32_to_bf16_bits(float f)
{
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
// two floats -> two bf16 (round to nearest even) in one word, `lo` in the low half: one conversion instruction
NS_DEVINL uint32_t ns_pack_bf16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

#endif  // __CUDACC__
