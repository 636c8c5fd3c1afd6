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
//               them 32 columns at a time with tcgen05.ld, applies scale / bias / GELU / residual,
//               writes the [32 rows x 128 B] block to shared memory (swizzled, conflict-free) and
//               one lane sends it to global memory with a TMA store, which writes whole lines and
//               clips at the matrix edge; then hands the accumulator back, so the next tile's MMAs
//               overlap.  (Storing straight from registers, one row per thread, cost 31 us per
//               128 x 256 float tile: 16-byte pieces of 32 different lines per instruction.)
// Every wait on an mbarrier is bounded (ns_mbar_wait); a wait that runs out stores a code to the
// device status block, all roles leave their loops, and tensor memory is released before exit.
#include <stdlib.h>
#include <string.h>

#define NS_TAIL_DEVICE_CODE
#include "ns_gemm.cuh"
#include "ns_tail.cuh"

namespace {

constexpr int BM = 128;          // rows of A per tile = accumulator lanes
constexpr int BKB = 128;         // bytes of K per k-block = one swizzle atom
constexpr int GEMM_THREADS = 192;
constexpr uint32_t EPI_BUF_BYTES = 4096;                    // 32 rows x 128 B
constexpr uint32_t EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;       // 4 warps x 2 buffers

struct StoreMaps {
    CUtensorMap out;   // [M, N] of the output type, box 32 rows x 128 B (f32) or 64 B (bf16)
    CUtensorMap raw;   // [M, N] int32
    CUtensorMap part;  // [k_splits, M, N] 32-bit words
};

template <int BN>
struct TileCfg {
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr uint32_t A_BYTES = BM * BKB;
    static constexpr uint32_t B_BYTES = BN * BKB;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN;
    static constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + 256;
};

__device__ __forceinline__ void tile_coords(const NsGemmParams& p, int item, int& tm, int& tn, int& split)
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

// accumulator bits -> output value (without the residual)
template <int KIND>
__device__ __forceinline__ float finish_value(const NsGemmParams& p, uint32_t bits, float a_scale, float w_scale, float bias)
{
    if (KIND == NS_KIND_I8) return ns_gemm_finish_i8(p, static_cast<int32_t>(bits), a_scale, w_scale, bias);
    float v = __uint_as_float(bits);
    if (p.epilogue != NS_EPI_NONE) v = __fadd_rn(v, bias);
    if (p.epilogue == NS_EPI_BIAS_GELU) v = ns_gelu_fast(v);
    return v;
}

__device__ __forceinline__ float load_residual(const NsGemmParams& p, size_t idx)
{
    return ns_gemm_residual(p, idx);
}

// Adds residual[row, col0 .. col0+32) to v.  Vector loads when the row pitch allows.
__device__ __forceinline__ void add_residual32(const NsGemmParams& p, size_t base, int col0, float (&v)[32])
{
    const bool full = col0 + 32 <= p.N;
    if (p.residual_dtype == NS_F32 && full && (p.N & 3) == 0) {
        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.residual) + base);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float4 r4 = src[j];
            v[4 * j] = __fadd_rn(v[4 * j], r4.x); v[4 * j + 1] = __fadd_rn(v[4 * j + 1], r4.y);
            v[4 * j + 2] = __fadd_rn(v[4 * j + 2], r4.z); v[4 * j + 3] = __fadd_rn(v[4 * j + 3], r4.w);
        }
    } else if (p.residual_dtype == NS_BF16 && full && (p.N & 7) == 0) {
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.residual) + base);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint4 r4 = src[j];
            const uint32_t w[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
            for (int t = 0; t < 4; t++) {
                v[8 * j + 2 * t] = __fadd_rn(v[8 * j + 2 * t], __uint_as_float(w[t] << 16));
                v[8 * j + 2 * t + 1] = __fadd_rn(v[8 * j + 2 * t + 1], __uint_as_float(w[t] & 0xFFFF0000u));
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++)
            if (col0 + j < p.N) v[j] = __fadd_rn(v[j], load_residual(p, base + j));
    }
}

// While a tile's MMAs are still running its epilogue warps are idle: each lane asks L2 for the part of its row of the
// residual matrix that the tile's epilogue will add (columns [col_begin, col_end), clipped to the matrix), so that the
// epilogue's loads, 64 to 128 bytes per lane and chunk at a pitch of a whole row, wait for L2 and not for HBM.
__device__ __forceinline__ void prefetch_residual_row(const NsGemmParams& p, int row, int col_begin, int col_end)
{
    if (p.epilogue != NS_EPI_BIAS_RESIDUAL || p.out == nullptr || p.residual == nullptr || row >= p.M) return;
    const size_t el = p.residual_dtype == NS_F32 ? 4 : 2;
    if (col_end > p.N) col_end = p.N;
    if (col_begin >= col_end) return;
    const char* base = reinterpret_cast<const char*>(p.residual);
    const uint64_t first = (reinterpret_cast<uint64_t>(base) + ((size_t)row * p.N + col_begin) * el) & ~uint64_t(127);
    const uint64_t last = reinterpret_cast<uint64_t>(base) + ((size_t)row * p.N + col_end) * el - 1;
    for (uint64_t a = first; a <= last; a += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
}

// Writes this warp's [32 rows x WORDS*4 bytes] block into a staging buffer with the swizzle the
// store's tensor map expects (128-byte rows: 16-byte piece q of row r at q ^ (r & 7); 64-byte rows:
// q ^ ((r >> 1) & 3)), then lane 0 queues the TMA store.  Two buffers alternate; before a buffer is
// written again the store that last read it must have finished reading (wait_group.read 1).
template <int WORDS>
__device__ __forceinline__ void stage_and_store(uint32_t buf, int lane, const uint32_t (&w)[32], const CUtensorMap* map, int x, int y, int z,
                                                bool three_d, bool single = false)
{
    if (lane == 0) {
        if (single) ns_bulk_wait_read<0>();
        else ns_bulk_wait_read<1>();
    }
    __syncwarp();
#pragma unroll
    for (int q = 0; q < WORDS / 4; q++) {
        const int sw = WORDS == 32 ? (q ^ (lane & 7)) : (q ^ ((lane >> 1) & 3));
        ns_st_shared_v4(buf + lane * (WORDS * 4) + sw * 16, w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
    ns_fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
        if (three_d) ns_tma_store_3d(map, buf, x, y, z);
        else ns_tma_store_2d(map, buf, x, y);
        ns_bulk_commit();
    }
}

// Per-tile constants of one epilogue warp.
struct EpiCtx {
    int lane, row0, row, split;
    bool row_ok;
    float a_scale;
    uint32_t bufs;   // two staging buffers (one when `single`)
    int nbuf;        // stores queued so far (selects the buffer)
    bool single;     // one staging buffer: a second warp on the same scheduler covers the wait for its store
    // a tile shared by two clusters (pair kernel, k-blocks dealt out evenly):
    int sk_dump;               // >= 0: this part's accumulators go to slab sk_dump of the work area instead of the output
    const uint32_t* sk_add;    // non-null: the other part's accumulators of this thread's row (256 words), added before the epilogue
    int sk_row, sk_col;        // first row of this warp and first column of the chunk inside the 256 x 256 tile
};

// Finishes 32 columns [col0, col0+32) of this thread's row from accumulator words r and sends them out.
// Column scales and biases are read with 16-byte loads at a warp-uniform address (one L1 access
// serves the warp); the ragged last chunk of a row and unaligned vectors take the scalar path.
template <int KIND>
__device__ __forceinline__ void epilogue_chunk(const NsGemmParams& p, const StoreMaps& sm, EpiCtx& cx, const uint32_t (&r)[32], int col0)
{
    const size_t base = (size_t)cx.row * p.N + col0;
    if (cx.sk_dump >= 0) {
        stage_and_store<32>(cx.bufs + (cx.single ? 0 : (cx.nbuf & 1)) * EPI_BUF_BYTES, cx.lane, r, &sm.part, cx.sk_col, cx.sk_row, cx.sk_dump, true, cx.single);
        cx.nbuf++;
        return;
    }
    if (p.k_splits > 1) {
        if (p.tma_store) {
            stage_and_store<32>(cx.bufs + (cx.single ? 0 : (cx.nbuf & 1)) * EPI_BUF_BYTES, cx.lane, r, &sm.part, col0, cx.row0, cx.split, true, cx.single);
            cx.nbuf++;
        } else if (cx.row_ok) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(p.partial) + (size_t)cx.split * p.M * p.N + base;
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col0 + j < p.N) dst[j] = r[j];
        }
        return;
    }
    if (KIND == NS_KIND_I8 && p.raw != nullptr) {
        if (p.tma_store) {
            stage_and_store<32>(cx.bufs + (cx.single ? 0 : (cx.nbuf & 1)) * EPI_BUF_BYTES, cx.lane, r, &sm.raw, col0, cx.row0, 0, false, cx.single);
            cx.nbuf++;
        } else if (cx.row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col0 + j < p.N) p.raw[base + j] = (int32_t)r[j];
        }
    }
    if (p.out == nullptr) return;

    float v[32];
    const bool vec_ok = p.vec_cols && col0 + 32 <= p.N;
    float4 bv[8];
    if (vec_ok && p.epilogue != NS_EPI_NONE) {
        const float4* b4 = reinterpret_cast<const float4*>(p.bias + col0);
#pragma unroll
        for (int q = 0; q < 8; q++) bv[q] = __ldg(b4 + q);
    }
    if (KIND == NS_KIND_I8) {
        if (vec_ok) {
            const float4* ws4 = reinterpret_cast<const float4*>(p.w_scale + col0);
            float4 wsv[8];
#pragma unroll
            for (int q = 0; q < 8; q++) wsv[q] = __ldg(ws4 + q);
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float4 w4 = wsv[q];
                v[4 * q] = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)r[4 * q]), cx.a_scale), w4.x);
                v[4 * q + 1] = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)r[4 * q + 1]), cx.a_scale), w4.y);
                v[4 * q + 2] = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)r[4 * q + 2]), cx.a_scale), w4.z);
                v[4 * q + 3] = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)r[4 * q + 3]), cx.a_scale), w4.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                v[j] = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)r[j]), cx.a_scale), __ldg(&p.w_scale[min(col0 + j, p.N - 1)]));
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
    }
    if (p.epilogue != NS_EPI_NONE) {
        if (vec_ok) {
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float4 t = bv[q];
                v[4 * q] = __fadd_rn(v[4 * q], t.x); v[4 * q + 1] = __fadd_rn(v[4 * q + 1], t.y);
                v[4 * q + 2] = __fadd_rn(v[4 * q + 2], t.z); v[4 * q + 3] = __fadd_rn(v[4 * q + 3], t.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __fadd_rn(v[j], __ldg(&p.bias[min(col0 + j, p.N - 1)]));
        }
        if (p.epilogue == NS_EPI_BIAS_GELU) {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = ns_gelu_fast(v[j]);
        } else if (p.epilogue == NS_EPI_BIAS_RESIDUAL && cx.row_ok) {
            add_residual32(p, base, col0, v);
        }
    }
    if (p.out_dtype == NS_F32) {
        if (p.tma_store) {
            uint32_t w[32];
#pragma unroll
            for (int j = 0; j < 32; j++) w[j] = __float_as_uint(v[j]);
            stage_and_store<32>(cx.bufs + (cx.single ? 0 : (cx.nbuf & 1)) * EPI_BUF_BYTES, cx.lane, w, &sm.out, col0, cx.row0, 0, false, cx.single);
            cx.nbuf++;
        } else if (cx.row_ok) {
            float* dst = reinterpret_cast<float*>(p.out) + base;
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col0 + j < p.N) dst[j] = v[j];
        }
    } else {
        if (p.tma_store) {
            uint32_t w[32];
#pragma unroll
            for (int j = 0; j < 16; j++)
                w[j] = ns_pack_bf16x2(v[2 * j], v[2 * j + 1]);
            stage_and_store<16>(cx.bufs + (cx.single ? 0 : (cx.nbuf & 1)) * EPI_BUF_BYTES, cx.lane, w, &sm.out, col0, cx.row0, 0, false, cx.single);
            cx.nbuf++;
        } else if (cx.row_ok) {
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) + base;
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col0 + j < p.N) dst[j] = ns_f32_to_bf16_bits(v[j]);
        }
    }
}

// TAIL: the launch has NS_TAIL_THREADS threads (warps 6 and 7 idle during the product) and is followed, in the same
// kernel, by the row operator of ns_tail.cuh; queued stores are then waited for until COMPLETE, not only until read.
template <int KIND, int BN, bool B_MN, bool TAIL>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const StoreMaps& sm, const NsGemmParams& p)
{
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag_storage;
    volatile int* abort_flag = &abort_flag_storage;

    const uint32_t smem_base = (ns_smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_base = smem_base + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_base = epi_base + EPI_BYTES;
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

    constexpr int ELEMS_PER_KB = KIND == NS_KIND_I8 ? 128 : 64;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            const uint32_t stage_tx = (uint32_t)p.a_rows * BKB + Cfg::B_BYTES;
            auto load_b = [&](int s, int kb, int tn) {
                const uint32_t b_dst = smem_base + s * Cfg::STAGE_BYTES + Cfg::A_BYTES;
                if (!B_MN) {
                    ns_tma_load_2d(b_dst, &tmB, full_bar(s), kb * ELEMS_PER_KB, tn * BN);
                } else {
                    // B stored [K, N]: boxes of 64 columns x 64 rows of K, one per 64 columns of the tile
#pragma unroll
                    for (int c = 0; c < BN / 64; c++)
                        ns_tma_load_2d(b_dst + c * (64 * 128), &tmB, full_bar(s), tn * BN + c * 64, kb * 64);
                }
            };
            // When B holds weights, which no kernel of the step writes (p.prefetch_b, set by the Linear objects only):
            // the first ring-full of B tiles is requested before waiting for the previous kernel, so its HBM latency
            // overlaps that kernel's tail.  A caller's own B may have been written by the kernel just before this one.
            int armed = 0;
            if (p.prefetch_b && (int)blockIdx.x < n_items) {
                int tm, tn, split;
                tile_coords(p, blockIdx.x, tm, tn, split);
                const int kb0 = split * p.kb_per_split;
                const int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
                armed = min(STAGES, kb1 - kb0);
                for (int i = 0; i < armed; i++) {
                    ns_mbar_expect_tx(full_bar(i), stage_tx);
                    load_b(i, kb0 + i, tn);
                }
            }
            ns_pdl_wait();
            ns_pdl_trigger();
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int tm, tn, split;
                tile_coords(p, item, tm, tn, split);
                int kb0 = split * p.kb_per_split;
                int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
                for (int kb = kb0; kb < kb1; kb++) {
                    const uint32_t a_dst = smem_base + s * Cfg::STAGE_BYTES;
                    if (armed > 0) {
                        armed--;   // slot already armed and its B tile on the way
                    } else {
                        ok = ns_mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status, p.status_base + 1);
                        if (!ok) break;
                        ns_mbar_expect_tx(full_bar(s), stage_tx);
                        load_b(s, kb, tn);
                    }
                    ns_tma_load_2d(a_dst, &tmA, full_bar(s), kb * ELEMS_PER_KB, tm * BM);
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = KIND == NS_KIND_I8 ? ns_idesc(2, 1, 0, 0, BM, BN) : ns_idesc(1, 1, 0, B_MN ? 1 : 0, BM, BN);
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
                        if (KIND == NS_KIND_I8) ns_mma_i8(d_tmem, a_desc, b_desc, idesc, accumulate);
                        else ns_mma_f16(d_tmem, a_desc, b_desc, idesc, accumulate);
                    }
                    ns_tc_commit(empty_bar(s));
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (ok) ns_tc_commit(tfull_bar(acc));
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- epilogue
        const int quad = warp & 3;
        EpiCtx cx;
        cx.lane = lane;
        cx.bufs = epi_base + (warp - 2) * 2 * EPI_BUF_BYTES;
        cx.nbuf = 0;
        cx.single = false;
        cx.sk_dump = -1; cx.sk_add = nullptr; cx.sk_row = 0; cx.sk_col = 0;
        int local = 0;
        bool ok = true;
        ns_pdl_wait();   // a_scale, residual and every output buffer belong to the previous kernel until it is done
        const float* a_scales = ns_after_wait(p.a_scale);
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, local++) {
            int tm, tn, split;
            tile_coords(p, item, tm, tn, split);
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            cx.row0 = tm * BM + quad * 32;
            cx.row = cx.row0 + lane;
            cx.row_ok = cx.row < p.M;
            cx.split = split;
            // While the tile's MMAs are still running: fetch this row's scale and pull the tile's column scales and
            // biases into L1 (each tile has other columns, so without this every 32-column chunk below would wait
            // for a round trip to L2).
            // (a product that only leaves exact accumulators, p.out == null, has no scales or bias)
            cx.a_scale = (KIND == NS_KIND_I8 && cx.row_ok && p.k_splits == 1 && p.out != nullptr) ? __ldg(&a_scales[cx.row]) : 1.0f;
            if (p.k_splits == 1 && warp == 2 && p.out != nullptr) {
                const int pc = tn * BN + (lane & 7) * 32;
                if (lane < BN / 32 && pc < p.N) {
                    if (KIND == NS_KIND_I8) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.w_scale + pc));
                    if (p.epilogue != NS_EPI_NONE) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.bias + pc));
                }
            }
            if (p.k_splits == 1) prefetch_residual_row(p, cx.row, tn * BN, tn * BN + BN);
            ok = ns_mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, p.status_base + 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            ns_tc_fence_after();
            const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
            const bool warp_has_rows = cx.row0 < p.M;
            // Two register sets: the tensor-memory load of the next 32 columns is in flight while
            // the current 32 are finished (tcgen05.ld has a latency of several hundred cycles).
            uint32_t ra[32], rb[32];
            __syncwarp();
            ns_tmem_ld32(t_row, ra);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c += 2) {
                ns_tc_wait_ld();
                __syncwarp();
                ns_tmem_ld32(t_row + (c + 1) * 32, rb);
                if (warp_has_rows && tn * BN + c * 32 < p.N) epilogue_chunk<KIND>(p, sm, cx, ra, tn * BN + c * 32);
                ns_tc_wait_ld();
                __syncwarp();
                if (c + 2 < BN / 32) ns_tmem_ld32(t_row + (c + 2) * 32, ra);
                if (warp_has_rows && tn * BN + (c + 1) * 32 < p.N) epilogue_chunk<KIND>(p, sm, cx, rb, tn * BN + (c + 1) * 32);
            }
            ns_tc_fence_before();
            __syncwarp();
            if (lane == 0) ns_mbar_arrive(tempty_bar(acc));
        }
        // shared memory must stay valid until every queued store has read it; the stores themselves are
        // complete when the grid is -- unless a second phase of this launch reads them: then they are waited for
        // until complete, and made visible to the other SMs
        if (lane == 0) {
            if (TAIL) { ns_bulk_wait<0>(); __threadfence(); }
            else ns_bulk_wait_read<0>();
        }
        __syncwarp();
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

template <int KIND, int BN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
ns_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ StoreMaps sm, const NsGemmParams p)
{
    gemm_tc_body<KIND, BN, B_MN, false>(tmA, tmB, sm, p);
}

// The int8 product of a decoding step followed, in the same launch, by the row operator `tail` describes.
template <int BN>
__global__ void __launch_bounds__(NS_TAIL_THREADS, 1)
ns_gemm_tail_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ StoreMaps sm, const NsGemmParams p, const __grid_constant__ NsTail tail)
{
    ns_tail::stamp(tail, 0);
    gemm_tc_body<NS_KIND_I8, BN, false, true>(tmA, tmB, sm, p);
    ns_tail::run(tail);
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair kernel for large products (no K split; weights stored [N, K] or, for bf16, [K, N] read through MN-major
// descriptors as in the single-CTA kernel).
//
// With one CTA per 128 x 256 tile every k-block needs 48 KB from L2 (16 KB of A, 32 KB of B) for 512 tensor-core
// cycles of int8 (or bf16) work, and an SM takes in about 64 bytes per cycle: 768 cycles of loading per 512 cycles
// of math.  Measured: 128 x 128 tiles (32 KB per k-block for half the math) take 65 % of the time of 128 x 256
// tiles, not 50 %: the loop runs at the speed of the loads.  Here two CTAs of a cluster work on one 256 x 256
// tile: each loads its own 128 rows of A and HALF of the B tile (128 of its 256 rows), 32 KB per k-block, and the
// even CTA's MMA thread issues tcgen05.mma.cta_group::2, which multiplies the pair's 256 rows of A with all 256
// rows of B, reading each half of B from the shared memory of the CTA that loaded it.  Each CTA ends up with its
// own 128 x 256 accumulator in its own tensor memory and runs the same epilogue as the single-CTA kernel.
//
// Barriers: full[s] lives in the even CTA and counts the bytes of both CTAs' loads (each TMA names the even CTA's
// barrier); empty[s] and acc_full[a] exist in both CTAs and are signalled by a tcgen05.commit that arrives in both;
// acc_empty[a] lives in the even CTA and is arrived on by the 8 epilogue warps of the pair (the odd CTA's remotely).
// The two CTAs synchronise as a cluster after setting up barriers and before freeing tensor memory, so neither
// touches the other's shared memory outside that window.
struct PairCfg {
    static constexpr int BN = 256;                 // columns of the pair's tile
    static constexpr int BN_HALF = 128;            // rows of B one CTA loads
    static constexpr int STAGES = 5;
    static constexpr uint32_t A_BYTES = BM * BKB;
    static constexpr uint32_t B_BYTES = BN_HALF * BKB;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN;
    static constexpr uint32_t PAIR_EPI_BYTES = 8 * 2 * EPI_BUF_BYTES;   // 8 epilogue warps x 2 staging buffers
    static constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + PAIR_EPI_BYTES + 256;
};

// p.tiles_m / p.tiles_n count 256 x 256 tiles here.  Groups of 8 tile rows, rows fastest: the clusters running at
// the same time share A rows and B columns in L2.
__device__ __forceinline__ void pair_coords(const NsGemmParams& p, int item, int& tm, int& tn)
{
    const int group_rows = 8;
    const int per_group = group_rows * p.tiles_n;
    const int g = item / per_group;
    const int r = item - g * per_group;
    const int rows_here = min(group_rows, p.tiles_m - g * group_rows);
    tm = g * group_rows + r % rows_here;
    tn = r / rows_here;
}

constexpr int PAIR_THREADS = 320;   // producer warp, MMA warp, 8 epilogue warps

// r += the other part's accumulators of the same 32 columns (a tile shared by two clusters).  Exact for int32; float
// accumulators are added in a fixed order (this part + the other part), so results do not depend on timing.
template <int KIND>
__device__ __forceinline__ void add_other_part(uint32_t (&r)[32], const uint32_t* __restrict__ src)
{
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const uint4 t = __ldcg(s4 + q);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; j++)
            r[4 * q + j] = KIND == NS_KIND_I8 ? (uint32_t)((int32_t)r[4 * q + j] + (int32_t)w[j])
                                              : __float_as_uint(__fadd_rn(__uint_as_float(r[4 * q + j]), __uint_as_float(w[j])));
    }
}

// The work of cluster `cluster` of `n_clusters`.  Plain mode: tiles cluster, cluster + n_clusters, ... whole.  Even mode
// (p.streamk): the tiles' k-blocks are numbered through (tile-major) and dealt out in equal contiguous shares, so a
// share begins with the LAST k-blocks of one tile, continues with whole tiles and ends with the FIRST k-blocks of
// another.  The cluster that holds a tile's first k-blocks finishes the tile (it reaches them last); the one that
// holds its last k-blocks computes them first and leaves the accumulators in the work area.
struct PairWork {
    int count;          // items of this cluster
    int first;          // first tile (even mode)
    long long u0, u1;   // unit range (even mode)
};
__device__ __forceinline__ PairWork pair_work(const NsGemmParams& p, int cluster, int n_clusters, int n_items)
{
    PairWork w;
    if (!p.streamk) {
        w.count = cluster < n_items ? (n_items - cluster + n_clusters - 1) / n_clusters : 0;
        w.first = cluster; w.u0 = 0; w.u1 = 0;
        return w;
    }
    const long long total = (long long)n_items * p.k_blocks;
    w.u0 = total * cluster / n_clusters;
    w.u1 = total * (cluster + 1) / n_clusters;
    w.first = (int)(w.u0 / p.k_blocks);
    w.count = w.u1 > w.u0 ? (int)((w.u1 - 1) / p.k_blocks) - w.first + 1 : 0;
    return w;
}
// item i of the cluster: tile, k-block range, and what happens to the accumulators (0 = finish as usual, 1 = leave them
// in the work area (slab = cluster), 2 = add the part the NEXT cluster left in slab cluster + 1, then finish)
__device__ __forceinline__ void pair_item(const NsGemmParams& p, const PairWork& w, int cluster, int n_clusters, int i, int& tile, int& kb0, int& kb1,
                                          int& role)
{
    if (!p.streamk) {
        tile = cluster + i * n_clusters; kb0 = 0; kb1 = p.k_blocks; role = 0;
        return;
    }
    tile = w.first + i;
    const long long t0 = (long long)tile * p.k_blocks;
    kb0 = (int)(w.u0 > t0 ? w.u0 - t0 : 0);
    kb1 = (int)(w.u1 < t0 + p.k_blocks ? w.u1 - t0 : p.k_blocks);
    role = kb0 > 0 ? 1 : (kb1 < p.k_blocks ? 2 : 0);
}

template <int KIND, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
ns_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ StoreMaps sm, const NsGemmParams p)
{
    using Cfg = PairCfg;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int BN = Cfg::BN;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag_storage;
    volatile int* abort_flag = &abort_flag_storage;

    const uint32_t smem_base = (ns_smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_base = smem_base + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_base = epi_base + Cfg::PAIR_EPI_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ns_cluster_ctarank();        // 0: issues the MMAs
    const int cluster = blockIdx.x >> 1;
    const int n_clusters = gridDim.x >> 1;
    const int n_items = p.tiles_m * p.tiles_n;
    const PairWork work = pair_work(p, cluster, n_clusters, n_items);

    if (threadIdx.x == 0) {
        abort_flag_storage = 0;
        for (int s = 0; s < STAGES; s++) {
            ns_mbar_init(full_bar(s), 1);
            ns_mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            ns_mbar_init(tfull_bar(a), 1);
            ns_mbar_init(tempty_bar(a), 16);           // 8 epilogue warps of each CTA
        }
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(tmem_slot), "r"(0xFFFFFFFFu) : "memory");
        ns_fence_barrier_init();
        ns_fence_proxy_async();
        ns_prefetch_tensormap(&tmA);
        ns_prefetch_tensormap(&tmB);
    }
    __syncthreads();
    if (warp == 1) {
        ns_tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
        ns_tmem_relinquish_pair();
    }
    ns_tc_fence_before();
    ns_cluster_sync();                                 // both CTAs' barriers exist before anything remote happens
    ns_tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
    if (tmem_base == 0xFFFFFFFFu) tmem_base = ns_ld_shared_cluster_u32(ns_mapa(tmem_slot, rank ^ 1u));

    constexpr int ELEMS_PER_KB = KIND == NS_KIND_I8 ? 128 : 64;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int i = 0; i < work.count && ok; i++) {
                int item, kb0, kb1, role, tm, tn;
                pair_item(p, work, cluster, n_clusters, i, item, kb0, kb1, role);
                pair_coords(p, item, tm, tn);
                const int row0 = tm * 256 + (int)rank * BM;
                const int brow0 = tn * BN + (int)rank * Cfg::BN_HALF;
                for (int kb = kb0; kb < kb1; kb++) {
                    ok = ns_mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status, p.status_base + 11);
                    if (!ok) break;
                    // the even CTA's barrier counts the four boxes of the pair (boxes that reach past the matrix
                    // edge are zero-filled and still count in full)
                    if (rank == 0) ns_mbar_expect_tx(full_bar(s), 2 * Cfg::STAGE_BYTES);
                    const uint32_t bar = ns_mapa(full_bar(s), 0);
                    const uint32_t a_dst = smem_base + s * Cfg::STAGE_BYTES;
                    ns_tma_load_2d_pair(a_dst, &tmA, bar, kb * ELEMS_PER_KB, row0);
                    if (!B_MN) {
                        ns_tma_load_2d_pair(a_dst + Cfg::A_BYTES, &tmB, bar, kb * ELEMS_PER_KB, brow0);
                    } else {
                        // B stored [K, N]: this CTA's 128 columns as two boxes of 64 columns x 64 rows of K
                        ns_tma_load_2d_pair(a_dst + Cfg::A_BYTES, &tmB, bar, brow0, kb * 64);
                        ns_tma_load_2d_pair(a_dst + Cfg::A_BYTES + 64 * 128, &tmB, bar, brow0 + 64, kb * 64);
                    }
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
            // the commits that free the last ring slots arrive in this CTA's shared memory: see them land before leaving
            for (int i = 0; i < STAGES && ok; i++) {
                ok = ns_mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status, p.status_base + 15);
                if (++s == STAGES) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (even CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = KIND == NS_KIND_I8 ? ns_idesc(2, 1, 0, 0, 256, BN) : ns_idesc(1, 1, 0, B_MN ? 1 : 0, 256, BN);
            const uint64_t desc_k = ns_desc_base(16, 1024);
            const uint64_t desc_mn = ns_desc_base(64 * 128, 1024);     // MN-major: 64-column blocks 8 KB apart, 8 k-rows 1 KB apart
            int s = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int i = 0; i < work.count && ok; i++, local++) {
                int item, kb0, kb1, role;
                pair_item(p, work, cluster, n_clusters, i, item, kb0, kb1, role);
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                ok = ns_mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, p.status_base + 12);
                if (!ok) break;
                ns_tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    ok = ns_mbar_wait(full_bar(s), phase, abort_flag, p.status, p.status_base + 13);
                    if (!ok) break;
                    ns_tc_fence_after();
                    const uint32_t a_addr = smem_base + s * Cfg::STAGE_BYTES;
                    const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint64_t a_desc = ns_desc_at(desc_k, a_addr + kk * 32);
                        const uint64_t b_desc = B_MN ? ns_desc_at(desc_mn, b_addr + kk * (16 * 128)) : ns_desc_at(desc_k, b_addr + kk * 32);
                        const uint32_t accumulate = (kb > kb0 || kk > 0) ? 1u : 0u;
                        if (KIND == NS_KIND_I8) ns_mma_i8_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
                        else ns_mma_f16_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
                    }
                    ns_tc_commit_pair(empty_bar(s), 3);       // the ring slot is free in both CTAs
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (ok) ns_tc_commit_pair(tfull_bar(acc), 3);   // both CTAs' epilogues may read their accumulator
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
        // Eight warps: two per tensor-memory lane quadrant (a warp reads the lanes of quadrant warp % 4), each taking one
        // half of the 256 columns, so every scheduler has a second warp to issue while the first waits on tensor memory,
        // on its column vectors or on its store.
        const int quad = warp & 3;
        const int c_begin = ((warp - 2) >> 2) * (BN / 64);
        const int c_end = c_begin + BN / 64;
        EpiCtx cx;
        cx.lane = lane;
        cx.bufs = epi_base + (warp - 2) * 2 * EPI_BUF_BYTES;
        cx.nbuf = 0;
        cx.single = false;
        cx.split = 0;
        cx.sk_dump = -1; cx.sk_add = nullptr; cx.sk_row = 0; cx.sk_col = 0;
        int local = 0;
        bool ok = true;
        const uint32_t tempty_even0 = ns_mapa(tempty_bar(0), 0), tempty_even1 = ns_mapa(tempty_bar(1), 0);
        for (int i = 0; i < work.count && ok; i++, local++) {
            int item, kb0, kb1, role, tm, tn;
            pair_item(p, work, cluster, n_clusters, i, item, kb0, kb1, role);
            pair_coords(p, item, tm, tn);
            // a tile shared with a neighbouring cluster: its last k-blocks (computed here first) go to the work area, or its
            // first k-blocks (computed here last) are completed with what the next cluster left there
            cx.sk_dump = role == 1 ? cluster : -1;
            cx.sk_row = (int)rank * BM + quad * 32;
            const uint32_t* other_part = role == 2 ? p.sk_work + ((size_t)(cluster + 1) * 256 + cx.sk_row + lane) * 256 : nullptr;
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            cx.row0 = tm * 256 + (int)rank * BM + quad * 32;
            cx.row = cx.row0 + lane;
            cx.row_ok = cx.row < p.M;
            cx.a_scale = (KIND == NS_KIND_I8 && cx.row_ok && p.out != nullptr) ? __ldg(&p.a_scale[cx.row]) : 1.0f;
            if (warp == 2 && p.out != nullptr) {
                const int pc = tn * BN + (lane & 7) * 32;
                if (lane < BN / 32 && pc < p.N) {
                    if (KIND == NS_KIND_I8) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.w_scale + pc));
                    if (p.epilogue != NS_EPI_NONE) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.bias + pc));
                }
            }
            if (role != 1) prefetch_residual_row(p, cx.row, tn * BN + c_begin * 32, tn * BN + c_end * 32);
            ok = ns_mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, p.status_base + 14);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            ns_tc_fence_after();
            if (role == 2) {
                // the next cluster computed its part of this tile first of all, long ago; the wait is bounded all the same
                if (lane == 0) {
                    const long long t0 = clock64();
                    uint32_t seen;
                    for (;;) {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.sk_flags + cluster + 1) : "memory");
                        if (seen >= 16u) break;
                        if (*abort_flag != 0 || clock64() - t0 > NS_WAIT_LIMIT_CYCLES) {
                            *reinterpret_cast<volatile int*>(p.status) = p.status_base + 16;
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        __nanosleep(64);
                    }
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
            const bool warp_has_rows = cx.row0 < p.M;
            uint32_t ra[32];
            __syncwarp();
#pragma unroll 1
            for (int c = c_begin; c < c_end; c++) {
                ns_tmem_ld32(t_row + c * 32, ra);
                ns_tc_wait_ld();
                __syncwarp();
                if (warp_has_rows && tn * BN + c * 32 < p.N) {
                    cx.sk_col = c * 32;
                    if (other_part != nullptr) add_other_part<KIND>(ra, other_part + c * 32);
                    epilogue_chunk<KIND>(p, sm, cx, ra, tn * BN + c * 32);
                }
            }
            ns_tc_fence_before();
            __syncwarp();
            if (lane == 0) ns_mbar_arrive_cluster(acc ? tempty_even1 : tempty_even0);
            if (role == 1) {
                // this warp's share of the part is in the work area once its stores are complete: count it in
                if (lane == 0) {
                    ns_bulk_wait<0>();
                    __threadfence();
                    atomicAdd(p.sk_flags + cluster, 1u);
                }
                __syncwarp();
            }
        }
        if (lane == 0) ns_bulk_wait_read<0>();
        __syncwarp();
    }

    // ---------------------------------------------------------------- teardown
    ns_tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0 && threadIdx.x == 0) {
        long long t0 = clock64();
        while (clock64() - t0 < 400000) { }
    }
    // neither CTA may leave (or free tensor memory) while the other's MMAs, loads or arrivals can still reach it
    ns_cluster_sync();
    if (warp == 1) {
        ns_tc_fence_after();
        ns_tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    }
}

// Sums split-K partials in split order and applies the epilogue.  One thread per 4 columns.
template <int KIND>
__global__ void ns_gemm_splitk_finish_kernel(const NsGemmParams p)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    const int qpr = (p.N + 3) / 4;
    const int64_t quads = (int64_t)p.M * qpr;
    const bool vec = (p.N & 3) == 0;
    for (int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; q < quads; q += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(q / qpr);
        const int col0 = (int)(q % qpr) * 4;
        const float a_scale = KIND == NS_KIND_I8 ? __ldg(&p.a_scale[row]) : 1.0f;
        const size_t idx0 = (size_t)row * p.N + col0;
        uint32_t bits[4];
        if (KIND == NS_KIND_I8) {
            int32_t s[4] = {0, 0, 0, 0};
            for (int sp = 0; sp < p.k_splits; sp++) {
                const int32_t* src = reinterpret_cast<const int32_t*>(p.partial) + (size_t)sp * p.M * p.N + idx0;
                if (vec) {
                    int4 t = *reinterpret_cast<const int4*>(src);
                    s[0] += t.x; s[1] += t.y; s[2] += t.z; s[3] += t.w;
                } else {
                    for (int j = 0; j < 4 && col0 + j < p.N; j++) s[j] += src[j];
                }
            }
            for (int j = 0; j < 4; j++) bits[j] = (uint32_t)s[j];
        } else {
            float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int sp = 0; sp < p.k_splits; sp++) {
                const float* src = reinterpret_cast<const float*>(p.partial) + (size_t)sp * p.M * p.N + idx0;
                if (vec) {
                    float4 t = *reinterpret_cast<const float4*>(src);
                    s[0] = __fadd_rn(s[0], t.x); s[1] = __fadd_rn(s[1], t.y); s[2] = __fadd_rn(s[2], t.z); s[3] = __fadd_rn(s[3], t.w);
                } else {
                    for (int j = 0; j < 4 && col0 + j < p.N; j++) s[j] = __fadd_rn(s[j], src[j]);
                }
            }
            for (int j = 0; j < 4; j++) bits[j] = __float_as_uint(s[j]);
        }
        for (int j = 0; j < 4 && col0 + j < p.N; j++) {
            const size_t idx = idx0 + j;
            if (KIND == NS_KIND_I8 && p.raw != nullptr) p.raw[idx] = (int32_t)bits[j];
            if (p.out == nullptr) continue;
            float v = finish_value<KIND>(p, bits[j], a_scale, KIND == NS_KIND_I8 ? __ldg(&p.w_scale[col0 + j]) : 1.0f,
                                         p.epilogue != NS_EPI_NONE ? __ldg(&p.bias[col0 + j]) : 0.0f);
            if (p.epilogue == NS_EPI_BIAS_RESIDUAL) v = __fadd_rn(v, load_residual(p, idx));
            if (p.out_dtype == NS_F32) reinterpret_cast<float*>(p.out)[idx] = v;
            else reinterpret_cast<uint16_t*>(p.out)[idx] = ns_f32_to_bf16_bits(v);
        }
    }
}

template <int BN>
int launch_gemm_tail(NsDevice* d, const CUtensorMap& tmA, const CUtensorMap& tmB, const StoreMaps& sm, const NsGemmParams& p, const NsTail& tail)
{
    using Cfg = TileCfg<BN>;
    auto kernel = ns_gemm_tail_kernel<BN>;
    static bool configured[64] = {false};
    if (!configured[d->ordinal]) {
        NS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM_BYTES));
        configured[d->ordinal] = true;
    }
    // every CTA must be resident while CTAs wait for one another: one per SM (the kernel's shared memory allows no more)
    int items = p.tiles_m * p.tiles_n * p.k_splits;
    int grid = items < d->sm_count ? items : d->sm_count;
    NS_CUDA(ns_launch_pdl(kernel, dim3(grid), dim3(NS_TAIL_THREADS), Cfg::SMEM_BYTES, d->stream, tmA, tmB, sm, p, tail));
    return NS_OK;
}

template <int KIND, int BN, bool B_MN>
int launch_gemm(NsDevice* d, const CUtensorMap& tmA, const CUtensorMap& tmB, const StoreMaps& sm, const NsGemmParams& p)
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
    NS_CUDA(ns_launch_pdl(kernel, dim3(grid), dim3(GEMM_THREADS), Cfg::SMEM_BYTES, d->stream, tmA, tmB, sm, p));
    return NS_OK;
}

template <int KIND, bool B_MN>
int pair_max_clusters(NsDevice* d, int* out)
{
    auto kernel = ns_gemm_pair_kernel<KIND, B_MN>;
    static int max_clusters[64] = {0};
    if (max_clusters[d->ordinal] == 0) {
        NS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairCfg::SMEM_BYTES));
        // how many pairs the device can hold at once (a GPC with an odd number of free SMs leaves one unpaired)
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(d->sm_count & ~1);
        q.blockDim = dim3(PAIR_THREADS);
        q.dynamicSmemBytes = PairCfg::SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        q.attrs = attr;
        q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &q) != cudaSuccess || n <= 0) { cudaGetLastError(); n = d->sm_count / 2; }
        if (n > d->sm_count / 2) n = d->sm_count / 2;
        max_clusters[d->ordinal] = n;
    }
    *out = max_clusters[d->ordinal];
    return NS_OK;
}

template <int KIND, bool B_MN>
int launch_pair(NsDevice* d, const CUtensorMap& tmA, const CUtensorMap& tmB, const StoreMaps& sm, const NsGemmParams& p, int clusters)
{
    auto kernel = ns_gemm_pair_kernel<KIND, B_MN>;
    NS_CUDA(ns_launch_plain(kernel, dim3(2 * clusters), dim3(PAIR_THREADS), PairCfg::SMEM_BYTES, d->stream, tmA, tmB, sm, p));
    return NS_OK;
}

template <int KIND, bool B_MN>
int dispatch_bn(NsDevice* d, int bn, const CUtensorMap& tmA, const CUtensorMap& tmB, const StoreMaps& sm, const NsGemmParams& p)
{
    switch (bn) {
        case 256: return launch_gemm<KIND, 256, B_MN>(d, tmA, tmB, sm, p);
        case 128: return launch_gemm<KIND, 128, B_MN>(d, tmA, tmB, sm, p);
        case 64: return launch_gemm<KIND, 64, B_MN>(d, tmA, tmB, sm, p);
        default: return ns_fail(NS_ERR_ARGUMENT, "unsupported tile width %d", bn);
    }
}

}  // namespace

// Tile width and split count.  Several row tiles: the widest tile that still fills the SMs, no split.  One row tile
// (M <= 128, the weight-streaming case): wide tiles, so every k-row of a [K, N] weight is read in long contiguous
// pieces, and K split until about every SM has a CTA while each split keeps at least 4 k-blocks (measured: the
// narrow-tile / no-split choice was 1.6x slower on M=8, N=14336, K=4096).
void ns_gemm_choose_tiling(const NsDevice* d, int M, int N, int k_blocks, int* bn_out, int* splits_out, bool b_is_kn)
{
    const int tiles_m = (M + BM - 1) / BM;
    int bn = 256;
    if (d->force_bn) {
        bn = d->force_bn == NS_TUNE_NARROW ? 64 : (d->force_bn == NS_TUNE_PAIR ? 256 : d->force_bn);
    } else if (tiles_m == 1) {
        bn = b_is_kn ? 256 : 128;
        while (bn > 64 && bn / 2 >= N) bn >>= 1;
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
        if (splits > 8) splits = 8;
    }
    if (splits > k_blocks) splits = k_blocks;
    if (splits < 1) splits = 1;
    *bn_out = bn;
    *splits_out = splits;
}

int ns_gemm_run(NsDevice* d, int kind, const void* a, const void* b, bool b_is_kn, int M, int N, int K, NsGemmParams p,
                void* partial_override, size_t partial_override_bytes, void** deferred_partial, int* deferred_splits, NsTail* tail)
{
    NS_REQUIRE(tail == nullptr || (kind == NS_KIND_I8 && !b_is_kn && M <= NS_TAIL_MAX_ROWS), NS_ERR_ARGUMENT,
               "a product with a second phase is an int8 product of at most %d rows", NS_TAIL_MAX_ROWS);
    const bool peer_tail = tail != nullptr && tail->kind == NS_TAIL_PEER;
    void* tail_partial = nullptr;
    int tail_splits = 0;
    if (tail != nullptr && !peer_tail) { deferred_partial = &tail_partial; deferred_splits = &tail_splits; }
    const bool deferred = deferred_partial != nullptr && deferred_splits != nullptr;
    NS_REQUIRE(!deferred || kind == NS_KIND_I8, NS_ERR_ARGUMENT, "a deferred epilogue exists for int8 products only");
    const int elsize = kind == NS_KIND_I8 ? 1 : 2;
    NS_REQUIRE(M > 0 && N > 0 && K > 0, NS_ERR_ARGUMENT, "product with an empty dimension (M=%d N=%d K=%d)", M, N, K);
    NS_REQUIRE(((int64_t)K * elsize) % 16 == 0, NS_ERR_ARGUMENT, "K=%d: a row of %d bytes is not a multiple of 16 bytes", K, K * elsize);
    NS_REQUIRE(!(b_is_kn && kind == NS_KIND_I8), NS_ERR_ARGUMENT, "int8 weights must be stored [N,K]");
    NS_REQUIRE(!b_is_kn || (N % 8) == 0, NS_ERR_ARGUMENT, "N=%d must be a multiple of 8 when B is stored [K,N]", N);
    p.M = M; p.N = N; p.K = K;
    // One to eight rows of int8 activations: the row-streaming kernel on the CUDA cores (a tuning override keeps
    // the tensor-core kernels, as does a deferred epilogue).
    if (kind == NS_KIND_I8 && !deferred && tail == nullptr && d->force_bn == 0 && d->force_splits == 0 && ns_gemv_i8_fits(M, K) &&
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0)
        return ns_gemv_i8_run(d, p, a, b);
    // Nine to sixteen rows whose K fits the registers of one CTA: the streaming kernel (weights straight into registers,
    // mma.sync, K summed inside the CTA, epilogue in the same launch).  NS_B200_STREAM=0 keeps the tcgen05 kernels.
    static int stream_env = -1;
    if (stream_env < 0) { const char* e = getenv("NS_B200_STREAM"); stream_env = (e != nullptr && e[0] == '0') ? 0 : 1; }
    if (stream_env == 1 && kind == NS_KIND_I8 && !deferred && tail == nullptr && d->force_bn == 0 && d->force_splits == 0 && ns_stream_i8_fits(M, K) &&
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0)
        return ns_stream_i8_run(d, p, a, b);
    p.k_blocks = (int)(((int64_t)K * elsize + BKB - 1) / BKB);
    int bn, splits;
    ns_gemm_choose_tiling(d, M, N, p.k_blocks, &bn, &splits, b_is_kn);
    // Large products with [N, K] weights go to the CTA-pair kernel (256 x 256 tiles over two SMs): whenever 256-wide
    // tiles without a K split were chosen and there are at least two row tiles.  The test hook NS_TUNE_PAIR forces it,
    // a tile width of 256 forces the single-CTA kernel.
    if (peer_tail) {
        // The ranks exchange float partial rows, so K stays whole; narrow tiles spread the weight stream over more SMs.
        splits = 1;
        if (d->force_bn == 0) bn = 64;
    }
    if (d->force_bn == NS_TUNE_PAIR && d->force_splits == 2) splits = 1;   // test hook: pair kernel, k-blocks dealt out evenly
    const bool pair = tail == nullptr && splits == 1 && M > BM && (d->force_bn == NS_TUNE_PAIR || (d->force_bn == 0 && bn == 256));
    p.kb_per_split = (p.k_blocks + splits - 1) / splits;
    p.k_splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
    p.tiles_m = pair ? (M + 255) / 256 : (M + BM - 1) / BM;
    p.tiles_n = (N + bn - 1) / bn;
    // CTA-pair kernel: how many clusters, and whether the last wave would leave many of them idle.  128 tiles on 74
    // clusters are 1.73 waves that take the time of 2: then the tiles' k-blocks are dealt out evenly instead (every
    // cluster gets tiles * k_blocks / clusters of them; a tile that straddles two clusters is completed through a work
    // area).  The test hook NS_TUNE_PAIR with a split count of 2 forces that mode on small shapes.
    int pair_clusters = 0;
    p.streamk = 0;
    p.sk_work = nullptr;
    p.sk_flags = nullptr;
    if (pair) {
        int max_c = 0;
        int prc = kind == NS_KIND_I8 ? pair_max_clusters<NS_KIND_I8, false>(d, &max_c)
                  : (!b_is_kn ? pair_max_clusters<NS_KIND_BF16, false>(d, &max_c) : pair_max_clusters<NS_KIND_BF16, true>(d, &max_c));
        if (prc != NS_OK) return prc;
        const int items = p.tiles_m * p.tiles_n;
        pair_clusters = items < max_c ? items : max_c;
        const bool forced = d->force_bn == NS_TUNE_PAIR && d->force_splits == 2 && items >= 3 && p.k_blocks >= 2;
        if (forced) pair_clusters = (items * 3 + 3) / 4 < max_c ? (items * 3 + 3) / 4 : max_c;
        const int waves = (items + pair_clusters - 1) / pair_clusters;
        // Measured (2048 x 4096 x 4096): 50 us this way against 30 us with whole tiles -- every cluster then runs three
        // epilogues of about 9 us (its share of a tile dumped, a whole tile, a share completed) where it ran two, and the
        // epilogue, not the tensor pipe, is what a short launch waits for.  So the even deal stays off unless asked for
        // (NS_B200_STREAMK=1 in the environment, or the test hook).
        static int sk_env = -1;
        if (sk_env < 0) { const char* e = getenv("NS_B200_STREAMK"); sk_env = (e != nullptr && e[0] == '1') ? 1 : 0; }
        const bool uneven = sk_env == 1 && items > pair_clusters && (int64_t)items * 100 < (int64_t)waves * pair_clusters * 93;
        if ((uneven && p.k_blocks >= 8) || (forced && pair_clusters < items)) {
            const size_t work_bytes = (size_t)(pair_clusters + 1) * 256 * 256 * 4;
            void* block = nullptr;
            int src = ns_scratch_reserve(d, work_bytes + 4096, &block);
            if (src != NS_OK) return src;
            p.streamk = 1;
            p.sk_work = reinterpret_cast<uint32_t*>(block);
            p.sk_flags = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(block) + work_bytes);
            NS_CUDA(cudaMemsetAsync(p.sk_flags, 0, 4096, d->stream));
        }
    }
    p.status = d->status_dev;
    p.status_base = kind == NS_KIND_I8 ? 100 : 200;
    p.partial = nullptr;
    if (p.k_splits > 1) {
        const size_t need = (size_t)p.k_splits * M * N * 4;
        if (partial_override != nullptr) {
            NS_REQUIRE(need <= partial_override_bytes, NS_ERR_MEMORY, "split-K partial sums need %zu bytes, the fixed scratch block holds %zu",
                       need, partial_override_bytes);
            p.partial = partial_override;
        } else {
            int rc = ns_scratch_reserve(d, need, &p.partial);
            if (rc != NS_OK) return rc;
        }
    } else if (deferred) {
        // K not split: the kernel writes its exact accumulators as the one slab and nothing else
        void* slab = nullptr;
        int rc = ns_scratch_reserve(d, (size_t)M * N * 4, &slab);
        if (rc != NS_OK) return rc;
        p.raw = reinterpret_cast<int32_t*>(slab);
        p.out = nullptr;
        p.epilogue = NS_EPI_NONE;
    }
    CUtensorMap tmA, tmB;
    StoreMaps sm;
    memset(&sm, 0, sizeof(sm));
    const CUtensorMapDataType dt = kind == NS_KIND_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint32_t box_k = BKB / elsize;
    int rc;
    {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
        uint64_t strides[1] = {(uint64_t)K * elsize};
        // 64 rows are enough for M <= 64: the other accumulator lanes are never stored
        p.a_rows = M <= 64 ? 64 : BM;
        uint32_t box[2] = {box_k, (uint32_t)p.a_rows};
        rc = ns_make_tensor_map(&tmA, dt, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != NS_OK) return rc;
    }
    if (!b_is_kn) {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
        uint64_t strides[1] = {(uint64_t)K * elsize};
        uint32_t box[2] = {box_k, (uint32_t)(pair ? PairCfg::BN_HALF : bn)};
        rc = ns_make_tensor_map(&tmB, dt, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != NS_OK) return rc;
    } else {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
        uint64_t strides[1] = {(uint64_t)N * elsize};
        uint32_t box[2] = {64, 64};
        rc = ns_make_tensor_map(&tmB, dt, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != NS_OK) return rc;
    }
    // Output maps.  A TMA store needs a 16-byte aligned base and row pitch; otherwise the kernel
    // falls back to stores from registers.
    const size_t out_el = p.out_dtype == NS_F32 ? 4 : 2;
    bool tma_ok = (N * 4) % 16 == 0;
    if (p.k_splits == 1) {
        if (p.out != nullptr) tma_ok = tma_ok && ((size_t)N * out_el) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
        if (p.raw != nullptr) tma_ok = tma_ok && (reinterpret_cast<uintptr_t>(p.raw) & 15) == 0;
    } else {
        tma_ok = tma_ok && (reinterpret_cast<uintptr_t>(p.partial) & 15) == 0 && ((size_t)M * N * 4) % 16 == 0;
    }
    p.tma_store = tma_ok ? 1 : 0;
    p.vec_cols = ((reinterpret_cast<uintptr_t>(p.w_scale) | reinterpret_cast<uintptr_t>(p.bias)) & 15) == 0 ? 1 : 0;
    if (p.streamk) {
        uint64_t dims[3] = {256, 256, (uint64_t)(pair_clusters + 1)};
        uint64_t strides[2] = {256 * 4, 256 * 256 * 4};
        uint32_t box[3] = {32, 32, 1};
        rc = ns_make_tensor_map(&sm.part, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.sk_work, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != NS_OK) return rc;
    }
    if (tma_ok) {
        if (p.k_splits > 1) {
            uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)p.k_splits};
            uint64_t strides[2] = {(uint64_t)N * 4, (uint64_t)M * N * 4};
            uint32_t box[3] = {32, 32, 1};
            rc = ns_make_tensor_map(&sm.part, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.partial, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc != NS_OK) return rc;
        } else {
            uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
            uint32_t box[2] = {32, 32};
            if (p.out != nullptr) {
                uint64_t strides[1] = {(uint64_t)N * out_el};
                rc = p.out_dtype == NS_F32
                         ? ns_make_tensor_map(&sm.out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p.out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)
                         : ns_make_tensor_map(&sm.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
                if (rc != NS_OK) return rc;
            }
            if (p.raw != nullptr) {
                uint64_t strides[1] = {(uint64_t)N * 4};
                rc = ns_make_tensor_map(&sm.raw, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, p.raw, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
                if (rc != NS_OK) return rc;
            }
        }
    }
    if (tail != nullptr) {
        if (!peer_tail) {
            tail->partial = reinterpret_cast<const int32_t*>(p.k_splits > 1 ? p.partial : reinterpret_cast<void*>(p.raw));
            tail->splits = p.k_splits;
        }
        tail->sync = d->sync_words;
        tail->status = d->status_dev;
        tail->times = d->tail_times;
        switch (bn) {
            case 256: return launch_gemm_tail<256>(d, tmA, tmB, sm, p, *tail);
            case 128: return launch_gemm_tail<128>(d, tmA, tmB, sm, p, *tail);
            default: return launch_gemm_tail<64>(d, tmA, tmB, sm, p, *tail);
        }
    }
    if (pair) {
        if (kind == NS_KIND_I8) rc = launch_pair<NS_KIND_I8, false>(d, tmA, tmB, sm, p, pair_clusters);
        else if (!b_is_kn) rc = launch_pair<NS_KIND_BF16, false>(d, tmA, tmB, sm, p, pair_clusters);
        else rc = launch_pair<NS_KIND_BF16, true>(d, tmA, tmB, sm, p, pair_clusters);
    }
    else if (kind == NS_KIND_I8) rc = dispatch_bn<NS_KIND_I8, false>(d, bn, tmA, tmB, sm, p);
    else if (!b_is_kn) rc = dispatch_bn<NS_KIND_BF16, false>(d, bn, tmA, tmB, sm, p);
    else rc = dispatch_bn<NS_KIND_BF16, true>(d, bn, tmA, tmB, sm, p);
    if (rc != NS_OK) return rc;
    if (deferred) {
        *deferred_partial = p.k_splits > 1 ? p.partial : reinterpret_cast<void*>(p.raw);
        *deferred_splits = p.k_splits;
        return NS_OK;
    }
    if (p.k_splits > 1) {
        int64_t quads = (int64_t)M * ((N + 3) / 4);
        int64_t blocks = (quads + 255) / 256;
        if (blocks > (int64_t)d->sm_count * 8) blocks = (int64_t)d->sm_count * 8;
        if (kind == NS_KIND_I8) NS_CUDA(ns_launch_plain(ns_gemm_splitk_finish_kernel<NS_KIND_I8>, dim3((unsigned)blocks), dim3(256), 0, d->stream, p));
        else NS_CUDA(ns_launch_plain(ns_gemm_splitk_finish_kernel<NS_KIND_BF16>, dim3((unsigned)blocks), dim3(256), 0, d->stream, p));
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
    NsGemmParams p = {};
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.residual_dtype = residual_dtype;
    p.out = reinterpret_cast<void*>(y);
    p.raw = reinterpret_cast<int32_t*>(raw_s32);
    p.a_scale = reinterpret_cast<const float*>(a_scale);
    p.w_scale = reinterpret_cast<const float*>(w_scale);
    p.bias = reinterpret_cast<const float*>(bias);
    p.residual = reinterpret_cast<const void*>(residual);
    return ns_gemm_run(d, NS_KIND_I8, reinterpret_cast<const void*>(aq), reinterpret_cast<const void*>(wq), false, M, N, K, p);
}

extern "C" int ns_bench_i8_mainloop(ns_device_t h, uint64_t aq, uint64_t wq, int M, int N, int K)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(aq && wq, NS_ERR_ARGUMENT, "ns_bench_i8_mainloop: null operand");
    NS_REQUIRE(M > 8, NS_ERR_ARGUMENT, "ns_bench_i8_mainloop: meant for the tensor-core kernels (M > 8)");
    // no output and no raw accumulators: the epilogue warps read tensor memory and hand the accumulator back
    NsGemmParams p = {};
    p.epilogue = NS_EPI_NONE;
    p.out_dtype = NS_F32;
    p.residual_dtype = NS_F32;
    return ns_gemm_run(d, NS_KIND_I8, reinterpret_cast<const void*>(aq), reinterpret_cast<const void*>(wq), false, M, N, K, p);
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
        NsGemmParams p = {};
        p.epilogue = epilogue;
        p.out_dtype = out_dtype;
        p.residual_dtype = residual_dtype;
        p.out = reinterpret_cast<void*>(c + (uint64_t)bi * m * n * out_el);
        p.bias = reinterpret_cast<const float*>(bias);
        p.residual = residual ? reinterpret_cast<const void*>(residual + (uint64_t)bi * m * n * res_el) : nullptr;
        rc = ns_gemm_run(d, NS_KIND_BF16, reinterpret_cast<const void*>(a + (uint64_t)bi * m * k * 2),
                         reinterpret_cast<const void*>(b + (uint64_t)bi * k * n * 2), transB == 0, m, n, k, p);
        if (rc != NS_OK) return rc;
    }
    return NS_OK;
}
