// Tensor-core products for sm_100a: int8 x int8 -> int32 (tcgen05 kind::i8) and bf16 x bf16 -> f32
// (kind::f16), accumulators in tensor memory, operands staged in shared memory by TMA.
//
// This is the replacement of the reference's only product kernel, matmul_f32
// (src/NeuralSharp/Backends/Cuda/PtxKernels.cs:484-627, launched by CudaBackend.BatchedMatMul,
// CudaBackend.cs:390-408), for the uses the decoder makes of it through Linear
// (src/NeuralSharp/Layers/Linear.cs:43-47), with the kernels that follow a product in the reference
// (add_rowvec_f32, bias_gelu_f32, add_f32) folded into the epilogue.
//
// Shape of one CTA (192 threads, persistent over output tiles):
//   warp 0      producer: one lane issues the TMA loads of a [128 x 128 B] tile of A and a
//               [BN x 128 B] tile of B per k-block into a STAGES-deep ring (128-byte swizzle)
//   warp 1      one lane issues tcgen05.mma (4 per k-block, each 32 bytes of K) into one of two
//               accumulators in tensor memory; tcgen05.commit releases the ring slot / hands the
//               accumulator to the epilogue
//   warps 2..5  epilogue: each warp owns the 32 accumulator lanes of its quadrant (warp % 4), reads
//               them 32 columns at a time with tcgen05.ld, applies scale / bias / GELU / residual
//               and stores; then hands the accumulator back, so the next tile's MMAs overlap.
// Every wait on an mbarrier is bounded (ns_mbar_wait); a wait that runs out stores a code to the
// device status block, all roles leave their loops, and tensor memory is released before exit.
#include "ns_common.cuh"

namespace {

constexpr int BM = 128;          // rows of A per tile = accumulator lanes
constexpr int BKB = 128;         // bytes of K per k-block = one swizzle atom
constexpr int GEMM_THREADS = 192;

enum { KIND_I8 = 0, KIND_BF16 = 1 };

struct GemmParams {
    int M, N, K;        // K in elements
    int k_blocks;       // ceil(K * elsize / 128)
    int k_splits;       // >= 1
    int kb_per_split;   // k-blocks per split
    int tiles_m, tiles_n;
    int epilogue;       // NS_EPI_*
    int out_dtype;      // NS_F32 / NS_BF16
    int residual_dtype;
    void* out;          // [M, N]
    int32_t* raw;       // optional exact accumulators (int8 kind only)
    const float* a_scale;
    const float* w_scale;
    const float* bias;
    const void* residual;
    void* partial;      // [k_splits, M, N] 32-bit words when k_splits > 1
    int* status;
    int status_base;    // code = status_base + role
};

template <int BN>
struct TileCfg {
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : (BN == 64 ? 8 : 8));
    static constexpr uint32_t A_BYTES = BM * BKB;
    static constexpr uint32_t B_BYTES = BN * BKB;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = (2 * BN) < 32 ? 32 : 2 * BN;
    static constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int item, int& tm, int& tn, int& split)
{
    // Items are ordered so that CTAs running at the same time share operands in L2: groups of 16
    // row tiles, rows fastest inside a group; splits of one tile are neighbours.
    split = item % p.k_splits;
    int t = item / p.k_splits;
    const int group_rows = 16;
    int per_group = group_rows * p.tiles_n;
    int g = t / per_group;
    int r = t - g * per_group;
    int rows_here = min(group_rows, p.tiles_m - g * group_rows);
    tm = g * group_rows + r % rows_here;
    tn = r / rows_here;
}

// value -> final output element
template <int KIND>
__device__ __forceinline__ float finish_value(const GemmParams& p, uint32_t bits, float a_scale, int col, const float* w_scale_bias)
{
    float v;
    if (KIND == KIND_I8) {
        v = __int2float_rn(static_cast<int32_t>(bits));
        v = __fmul_rn(v, a_scale);
        v = __fmul_rn(v, __ldg(&p.w_scale[col]));
    } else {
        v = __uint_as_float(bits);
    }
    if (p.epilogue != NS_EPI_NONE) v = __fadd_rn(v, __ldg(&p.bias[col]));
    if (p.epilogue == NS_EPI_BIAS_GELU) v = ns_gelu_tanh(v);
    (void)w_scale_bias;
    return v;
}

__device__ __forceinline__ float load_residual(const GemmParams& p, size_t idx)
{
    if (p.residual_dtype == NS_BF16) return ns_bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p.residual)[idx]);
    return reinterpret_cast<const float*>(p.residual)[idx];
}

template <int KIND, int BN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
ns_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p)
{
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag_storage;
    volatile int* abort_flag = &abort_flag_storage;

    const uint32_t smem_base = (ns_smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_items = p.tiles_m * p.tiles_n * p.k_splits;

    if (threadIdx.x == 0) {
        abort_flag_storage = 0;
        for (int s = 0; s < STAGES; s++) {
            ns_mbar_init(full_bar(s), 1);
            ns_mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            ns_mbar_init(tfull_bar(a), 1);
            ns_mbar_init(tempty_bar(a), 4);
        }
        ns_fence_barrier_init();
        ns_fence_proxy_async();
        ns_prefetch_tensormap(&tmA);
        ns_prefetch_tensormap(&tmB);
    }
    if (warp == 1) {
        ns_tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        ns_tmem_relinquish();
    }
    ns_tc_fence_before();
    __syncthreads();
    ns_tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

    constexpr int ELEMS_PER_KB = KIND == KIND_I8 ? 128 : 64;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int tm, tn, split;
                tile_coords(p, item, tm, tn, split);
                int kb0 = split * p.kb_per_split;
                int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
                for (int kb = kb0; kb < kb1; kb++) {
                    ok = ns_mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status, p.status_base + 1);
                    if (!ok) break;
                    uint32_t a_dst = smem_base + s * Cfg::STAGE_BYTES;
                    uint32_t b_dst = a_dst + Cfg::A_BYTES;
                    ns_mbar_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
                    ns_tma_load_2d(a_dst, &tmA, full_bar(s), kb * ELEMS_PER_KB, tm * BM);
                    if (!B_MN) {
                        ns_tma_load_2d(b_dst, &tmB, full_bar(s), kb * ELEMS_PER_KB, tn * BN);
                    } else {
                        // B stored [K, N]: boxes of 64 columns x 64 rows of K, one per 64 columns of the tile
#pragma unroll
                        for (int c = 0; c < BN / 64; c++)
                            ns_tma_load_2d(b_dst + c * (64 * 128), &tmB, full_bar(s), tn * BN + c * 64, kb * 64);
                    }
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = KIND == KIND_I8 ? ns_idesc(2, 1, 0, 0, BM, BN) : ns_idesc(1, 1, 0, B_MN ? 1 : 0, BM, BN);
            const uint64_t desc_k = ns_desc_base(16, 1024);            // K-major: 8-row groups 1024 B apart
            const uint64_t desc_mn = ns_desc_base(64 * 128, 1024);     // MN-major: 64-column blocks 8 KB apart, 8 k-rows 1 KB apart
            int s = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, local++) {
                int tm, tn, split;
                tile_coords(p, item, tm, tn, split);
                int kb0 = split * p.kb_per_split;
                int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                ok = ns_mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, p.status_base + 2);
                if (!ok) break;
                ns_tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    ok = ns_mbar_wait(full_bar(s), phase, abort_flag, p.status, p.status_base + 3);
                    if (!ok) break;
                    ns_tc_fence_after();
                    const uint32_t a_addr = smem_base + s * Cfg::STAGE_BYTES;
                    const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint64_t a_desc = ns_desc_at(desc_k, a_addr + kk * 32);
                        const uint64_t b_desc = B_MN ? ns_desc_at(desc_mn, b_addr + kk * (16 * 128)) : ns_desc_at(desc_k, b_addr + kk * 32);
                        const uint32_t accumulate = (kb > kb0 || kk > 0) ? 1u : 0u;
                        if (KIND == KIND_I8) ns_mma_i8(d_tmem, a_desc, b_desc, idesc, accumulate);
                        else ns_mma_f16(d_tmem, a_desc, b_desc, idesc, accumulate);
                    }
                    ns_tc_commit(empty_bar(s));
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (ok) ns_tc_commit(tfull_bar(acc));
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quad = warp & 3;
        int local = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, local++) {
            int tm, tn, split;
            tile_coords(p, item, tm, tn, split);
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            ok = ns_mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, p.status_base + 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            ns_tc_fence_after();
            const int row = tm * BM + quad * 32 + lane;
            const bool row_ok = row < p.M;
            const float a_scale = (KIND == KIND_I8 && row_ok && p.k_splits == 1) ? __ldg(&p.a_scale[row]) : 1.0f;
            const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t r[32];
                __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the divergent stores below
                ns_tmem_ld32(t_row + c * 32, r);
                ns_tc_wait_ld();
                const int col0 = tn * BN + c * 32;
                if (!row_ok || col0 >= p.N) continue;
                const bool full = col0 + 32 <= p.N;
                const size_t base = (size_t)row * p.N + col0;
                if (p.k_splits > 1) {
                    uint32_t* dst = reinterpret_cast<uint32_t*>(p.partial) + (size_t)split * p.M * p.N + base;
                    if (full && (p.N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; j++) dst[j] = r[j];
                    }
                    continue;
                }
                if (KIND == KIND_I8 && p.raw != nullptr) {
                    if (full && (p.N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(p.raw + base + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; j++) p.raw[base + j] = (int32_t)r[j];
                    }
                }
                if (p.out == nullptr) continue;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    int col = min(col0 + j, p.N - 1);
                    v[j] = finish_value<KIND>(p, r[j], a_scale, col, nullptr);
                }
                if (p.epilogue == NS_EPI_BIAS_RESIDUAL) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (col0 + j < p.N) v[j] = __fadd_rn(v[j], load_residual(p, base + j));
                }
                if (p.out_dtype == NS_F32) {
                    float* dst = reinterpret_cast<float*>(p.out) + base;
                    if (full && (p.N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; j++) dst[j] = v[j];
                    }
                } else {
                    uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) + base;
                    if (full && (p.N & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 pk;
                            pk.x = ns_f32_to_bf16_bits(v[j]) | (uint32_t(ns_f32_to_bf16_bits(v[j + 1])) << 16);
                            pk.y = ns_f32_to_bf16_bits(v[j + 2]) | (uint32_t(ns_f32_to_bf16_bits(v[j + 3])) << 16);
                            pk.z = ns_f32_to_bf16_bits(v[j + 4]) | (uint32_t(ns_f32_to_bf16_bits(v[j + 5])) << 16);
                            pk.w = ns_f32_to_bf16_bits(v[j + 6]) | (uint32_t(ns_f32_to_bf16_bits(v[j + 7])) << 16);
                            *reinterpret_cast<uint4*>(dst + j) = pk;
                        }
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; j++) dst[j] = ns_f32_to_bf16_bits(v[j]);
                    }
                }
            }
            ns_tc_fence_before();
            __syncwarp();
            if (lane == 0) ns_mbar_arrive(tempty_bar(acc));
        }
    }

    // ---------------------------------------------------------------- teardown
    ns_tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0 && threadIdx.x == 0) {
        // give loads that are still in flight time to land before shared memory is handed back
        long long t0 = clock64();
        while (clock64() - t0 < 400000) { }
    }
    __syncthreads();
    if (warp == 1) {
        ns_tc_fence_after();
        ns_tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// Sums split-K partials in split order and applies the epilogue.  One thread per 4 columns.
template <int KIND>
__global__ void ns_gemm_splitk_finish_kernel(const GemmParams p)
{
    const int64_t quads = (int64_t)p.M * ((p.N + 3) / 4);
    for (int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; q < quads; q += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(q / ((p.N + 3) / 4));
        const int col0 = (int)(q % ((p.N + 3) / 4)) * 4;
        const float a_scale = KIND == KIND_I8 ? __ldg(&p.a_scale[row]) : 1.0f;
        for (int j = 0; j < 4 && col0 + j < p.N; j++) {
            const size_t idx = (size_t)row * p.N + col0 + j;
            uint32_t bits;
            if (KIND == KIND_I8) {
                int32_t s = 0;
                for (int sp = 0; sp < p.k_splits; sp++) s += reinterpret_cast<const int32_t*>(p.partial)[(size_t)sp * p.M * p.N + idx];
                bits = (uint32_t)s;
                if (p.raw != nullptr) p.raw[idx] = s;
            } else {
                float s = 0.0f;
                for (int sp = 0; sp < p.k_splits; sp++) s = __fadd_rn(s, reinterpret_cast<const float*>(p.partial)[(size_t)sp * p.M * p.N + idx]);
                bits = __float_as_uint(s);
            }
            if (p.out == nullptr) continue;
            float v = finish_value<KIND>(p, bits, a_scale, col0 + j, nullptr);
            if (p.epilogue == NS_EPI_BIAS_RESIDUAL) v = __fadd_rn(v, load_residual(p, idx));
            if (p.out_dtype == NS_F32) reinterpret_cast<float*>(p.out)[idx] = v;
            else reinterpret_cast<uint16_t*>(p.out)[idx] = ns_f32_to_bf16_bits(v);
        }
    }
}

template <int KIND, int BN, bool B_MN>
int launch_gemm(NsDevice* d, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p)
{
    using Cfg = TileCfg<BN>;
    auto kernel = ns_gemm_tc_kernel<KIND, BN, B_MN>;
    static bool configured[64] = {false};
    if (!configured[d->ordinal]) {
        NS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM_BYTES));
        configured[d->ordinal] = true;
    }
    int items = p.tiles_m * p.tiles_n * p.k_splits;
    int grid = items < d->sm_count ? items : d->sm_count;
    kernel<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, d->stream>>>(tmA, tmB, p);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

template <int KIND, bool B_MN>
int dispatch_bn(NsDevice* d, int bn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p)
{
    switch (bn) {
        case 256: return launch_gemm<KIND, 256, B_MN>(d, tmA, tmB, p);
        case 128: return launch_gemm<KIND, 128, B_MN>(d, tmA, tmB, p);
        case 64: return launch_gemm<KIND, 64, B_MN>(d, tmA, tmB, p);
        default: return ns_fail(NS_ERR_ARGUMENT, "unsupported tile width %d", bn);
    }
}

// Tile width and split count: fill the SMs first (wide tiles when there are enough of them), then
// split K while every split still has at least 4 k-blocks.
void choose_tiling(const NsDevice* d, int M, int N, int k_blocks, int* bn_out, int* splits_out)
{
    const int tiles_m = (M + BM - 1) / BM;
    int bn = 256;
    if (d->force_bn) {
        bn = d->force_bn == 32 ? 64 : d->force_bn;
    } else {
        while (bn > 64 && tiles_m * ((N + bn - 1) / bn) < d->sm_count) bn >>= 1;
        while (bn > 64 && bn / 2 >= N) bn >>= 1;
    }
    int tiles = tiles_m * ((N + bn - 1) / bn);
    int splits = 1;
    if (d->force_splits) {
        splits = d->force_splits;
    } else if (tiles * 2 <= d->sm_count) {
        splits = d->sm_count / tiles;
        int max_by_k = k_blocks / 4;
        if (max_by_k < 1) max_by_k = 1;
        if (splits > max_by_k) splits = max_by_k;
        if (splits > 16) splits = 16;
    }
    if (splits > k_blocks) splits = k_blocks;
    if (splits < 1) splits = 1;
    *bn_out = bn;
    *splits_out = splits;
}

}  // namespace

// Shared by ns_qmatmul_i8, ns_matmul_bf16 and the Linear objects.
int ns_gemm_run(NsDevice* d, int kind, const void* a, const void* b, bool b_is_kn, int M, int N, int K, GemmParams p)
{
    const int elsize = kind == KIND_I8 ? 1 : 2;
    NS_REQUIRE(M > 0 && N > 0 && K > 0, NS_ERR_ARGUMENT, "product with an empty dimension (M=%d N=%d K=%d)", M, N, K);
    NS_REQUIRE(((int64_t)K * elsize) % 16 == 0, NS_ERR_ARGUMENT, "K=%d: a row of %d bytes is not a multiple of 16 bytes", K, K * elsize);
    NS_REQUIRE(!(b_is_kn && kind == KIND_I8), NS_ERR_ARGUMENT, "int8 weights must be stored [N,K]");
    NS_REQUIRE(!b_is_kn || (N % 8) == 0, NS_ERR_ARGUMENT, "N=%d must be a multiple of 8 when B is stored [K,N]", N);
    p.M = M; p.N = N; p.K = K;
    p.k_blocks = (int)(((int64_t)K * elsize + BKB - 1) / BKB);
    int bn, splits;
    choose_tiling(d, M, N, p.k_blocks, &bn, &splits);
    p.kb_per_split = (p.k_blocks + splits - 1) / splits;
    p.k_splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
    p.tiles_m = (M + BM - 1) / BM;
    p.tiles_n = (N + bn - 1) / bn;
    p.status = d->status_dev;
    p.status_base = kind == KIND_I8 ? 100 : 200;
    p.partial = nullptr;
    if (p.k_splits > 1) {
        int rc = ns_scratch_reserve(d, (size_t)p.k_splits * M * N * 4, &p.partial);
        if (rc != NS_OK) return rc;
    }
    CUtensorMap tmA, tmB;
    const CUtensorMapDataType dt = kind == KIND_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint32_t box_k = BKB / elsize;
    {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
        uint64_t strides[1] = {(uint64_t)K * elsize};
        uint32_t box[2] = {box_k, (uint32_t)BM};
        int rc = ns_make_tensor_map(&tmA, dt, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != NS_OK) return rc;
    }
    if (!b_is_kn) {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
        uint64_t strides[1] = {(uint64_t)K * elsize};
        uint32_t box[2] = {box_k, (uint32_t)bn};
        int rc = ns_make_tensor_map(&tmB, dt, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != NS_OK) return rc;
    } else {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
        uint64_t strides[1] = {(uint64_t)N * elsize};
        uint32_t box[2] = {64, 64};
        int rc = ns_make_tensor_map(&tmB, dt, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != NS_OK) return rc;
    }
    int rc;
    if (kind == KIND_I8) rc = dispatch_bn<KIND_I8, false>(d, bn, tmA, tmB, p);
    else if (!b_is_kn) rc = dispatch_bn<KIND_BF16, false>(d, bn, tmA, tmB, p);
    else rc = dispatch_bn<KIND_BF16, true>(d, bn, tmA, tmB, p);
    if (rc != NS_OK) return rc;
    if (p.k_splits > 1) {
        int64_t quads = (int64_t)M * ((N + 3) / 4);
        int64_t blocks = (quads + 255) / 256;
        if (blocks > (int64_t)d->sm_count * 8) blocks = (int64_t)d->sm_count * 8;
        if (kind == KIND_I8) ns_gemm_splitk_finish_kernel<KIND_I8><<<(unsigned)blocks, 256, 0, d->stream>>>(p);
        else ns_gemm_splitk_finish_kernel<KIND_BF16><<<(unsigned)blocks, 256, 0, d->stream>>>(p);
        NS_CUDA(cudaGetLastError());
    }
    return NS_OK;
}

static int check_epilogue(int epilogue, uint64_t bias, uint64_t residual, int residual_dtype, int out_dtype)
{
    NS_REQUIRE(epilogue >= NS_EPI_NONE && epilogue <= NS_EPI_BIAS_RESIDUAL, NS_ERR_ARGUMENT, "unknown epilogue %d", epilogue);
    NS_REQUIRE(epilogue == NS_EPI_NONE || bias != 0, NS_ERR_ARGUMENT, "epilogue %d needs a bias vector", epilogue);
    NS_REQUIRE(epilogue != NS_EPI_BIAS_RESIDUAL || residual != 0, NS_ERR_ARGUMENT, "epilogue NS_EPI_BIAS_RESIDUAL needs a residual matrix");
    NS_REQUIRE(residual_dtype == NS_F32 || residual_dtype == NS_BF16, NS_ERR_ARGUMENT, "residual dtype must be NS_F32 or NS_BF16");
    NS_REQUIRE(out_dtype == NS_F32 || out_dtype == NS_BF16, NS_ERR_ARGUMENT, "output dtype must be NS_F32 or NS_BF16");
    return NS_OK;
}

extern "C" int ns_qmatmul_i8(ns_device_t h, uint64_t aq, uint64_t a_scale, uint64_t wq, uint64_t w_scale, uint64_t bias,
                             uint64_t residual, int residual_dtype, int M, int N, int K, int epilogue, int out_dtype,
                             uint64_t y, uint64_t raw_s32)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(aq && wq && a_scale && w_scale, NS_ERR_ARGUMENT, "ns_qmatmul_i8: null operand");
    NS_REQUIRE(y != 0 || raw_s32 != 0, NS_ERR_ARGUMENT, "ns_qmatmul_i8: no output buffer");
    rc = check_epilogue(epilogue, bias, residual, residual_dtype, out_dtype);
    if (rc != NS_OK) return rc;
    GemmParams p = {};
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.residual_dtype = residual_dtype;
    p.out = reinterpret_cast<void*>(y);
    p.raw = reinterpret_cast<int32_t*>(raw_s32);
    p.a_scale = reinterpret_cast<const float*>(a_scale);
    p.w_scale = reinterpret_cast<const float*>(w_scale);
    p.bias = reinterpret_cast<const float*>(bias);
    p.residual = reinterpret_cast<const void*>(residual);
    return ns_gemm_run(d, KIND_I8, reinterpret_cast<const void*>(aq), reinterpret_cast<const void*>(wq), false, M, N, K, p);
}

extern "C" int ns_matmul_bf16(ns_device_t h, uint64_t a, uint64_t b, uint64_t c, int batch, int m, int n, int k, int transB,
                              uint64_t bias, uint64_t residual, int residual_dtype, int epilogue, int out_dtype)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(a && b && c, NS_ERR_ARGUMENT, "ns_matmul_bf16: null operand");
    NS_REQUIRE(batch >= 1, NS_ERR_ARGUMENT, "ns_matmul_bf16: batch must be at least 1");
    rc = check_epilogue(epilogue, bias, residual, residual_dtype, out_dtype);
    if (rc != NS_OK) return rc;
    const size_t out_el = out_dtype == NS_F32 ? 4 : 2;
    const size_t res_el = residual_dtype == NS_F32 ? 4 : 2;
    for (int bi = 0; bi < batch; bi++) {
        GemmParams p = {};
        p.epilogue = epilogue;
        p.out_dtype = out_dtype;
        p.residual_dtype = residual_dtype;
        p.out = reinterpret_cast<void*>(c + (uint64_t)bi * m * n * out_el);
        p.bias = reinterpret_cast<const float*>(bias);
        p.residual = residual ? reinterpret_cast<const void*>(residual + (uint64_t)bi * m * n * res_el) : nullptr;
        rc = ns_gemm_run(d, KIND_BF16, reinterpret_cast<const void*>(a + (uint64_t)bi * m * k * 2),
                         reinterpret_cast<const void*>(b + (uint64_t)bi * k * n * 2), transB == 0, m, n, k, p);
        if (rc != NS_OK) return rc;
    }
    return NS_OK;
}
