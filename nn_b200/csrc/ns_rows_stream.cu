// Row operators over MANY bf16 rows (a prompt read: tens of thousands of rows of 1024 to 8192 columns): int8 row
// quantisation and LayerNorm -> int8.  The reference's row operators are one thread per row (layernorm_fused_f32,
// src/NeuralSharp/Backends/Cuda/PtxKernels.Decoding.cs:61-90); the int8 rows are this library's (q = clamp(rint(x /
// scale)), scale = absmax / 127, as ns_quantize_rows_i8 states).
//
// These kernels move 3 bytes per element and spend 7 (quantisation) to 16 (LayerNorm) instructions on it, which puts
// them near the point where the instruction issue of a SM (its logic pipe above all) and its share of HBM take the same
// time.  So: a lane holds 32 to 64 elements (a row belongs to a GROUP of 1, 2 or 4 warps) and 16 to 24 warps are resident,
// the bytes in flight are held by shared memory instead of registers (every group owns a ring of STAGES row buffers filled
// by bulk asynchronous copies, cp.async.bulk with an mbarrier per buffer; the copy of row i + STAGES is issued as soon as
// row i sits in registers), row maxima are taken on packed bf16 pairs, and the rounding needs no division per element and
// no test for NaNs (ns_rows::quant8<false>): a row with a NaN or an infinity in it, or a scale too small to invert, is found
// by its maximum and takes the plain divisions.  Lane l of warp w of a group holds the 16-byte vectors (w * VEC + k) * 32 + l (k < VEC):
// shared-memory reads and global stores are contiguous across a warp.  A group's warps meet at a named barrier once per
// reduction, exchanging their partial results through shared memory.
//
// Every wait is bounded: a group whose copy does not arrive within about a second writes status 600 + warps per row, waits
// once more, bounded, for the copies it still has in flight, and returns.
#include "ns_rows.cuh"

namespace {

constexpr int RS_THREADS = 256;
constexpr int RS_WARPS = RS_THREADS / 32;

template <int COLS, int WPR, int STAGES, bool LN>
struct RsCfg {
    static constexpr int GROUPS = RS_WARPS / WPR;                 // rows a CTA works on at a time
    static constexpr int ROW_BYTES = COLS * 2;
    static constexpr int VEC = COLS / (WPR * 32 * 8);             // 16-byte vectors per lane
    static constexpr int RING_BYTES = GROUPS * STAGES * ROW_BYTES;
    static constexpr int PARAM_BYTES = LN ? COLS * 8 : 0;         // gamma and beta as float
    static constexpr int BAR_OFFSET = RING_BYTES + PARAM_BYTES;
    static constexpr int XCHG_OFFSET = BAR_OFFSET + GROUPS * STAGES * 8;
    static constexpr int NV = COLS / 256;                         // 32-vector pieces of a row: a sum is taken piece by piece, in piece order
    static constexpr int XCHG_WORDS = 2 * 5 * NV;                 // per group: two row parities x (four reductions + the outcome of the wait) x pieces (>= warps)
    static constexpr int SMEM_BYTES = XCHG_OFFSET + GROUPS * XCHG_WORDS * 4;
    static_assert(COLS % (WPR * 256) == 0 && VEC >= 1, "a lane holds whole 16-byte vectors");
};

NS_DEVINL void rs_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// One try with a suspend-time hint: the warp sleeps in the instruction until the phase completes or about `ns` nanoseconds have
// passed, instead of spinning through issue slots that the group's working warps need.
NS_DEVINL bool rs_try_wait(uint32_t bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

NS_DEVINL bool rs_wait(uint32_t bar, uint32_t parity)
{
    if (rs_try_wait(bar, parity, 20000u)) return true;
    const long long t0 = clock64();
    while (!rs_try_wait(bar, parity, 20000u)) {
        if (clock64() - t0 > NS_WAIT_LIMIT_CYCLES) return false;
    }
    return true;
}

NS_DEVINL void rs_group_barrier(int group, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(threads) : "memory");
}

// per bf16 half: the larger magnitude of m and a (sign arbitrary), NaN if either is one
NS_DEVINL uint32_t rs_absmax2(uint32_t m, uint32_t a)
{
    uint32_t r;
    asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(a));
    return r;
}
// the larger magnitude of the two halves as a float; +infinity when a NaN or an infinity is in play
NS_DEVINL float rs_absmax_or_inf(uint32_t mm)
{
    const float f0 = __uint_as_float((mm << 16) & 0x7FFFFFFFu), f1 = __uint_as_float(mm & 0x7FFF0000u);
    return (f0 <= 3.4028234e38f && f1 <= 3.4028234e38f) ? fmaxf(f0, f1) : __uint_as_float(0x7F800000u);
}

template <int COLS, int WPR, int STAGES, bool LN>
__global__ void __launch_bounds__(RS_THREADS) ns_rows_stream_kernel(const uint16_t* __restrict__ x, const float* __restrict__ gamma,
                                                                    const float* __restrict__ beta, int64_t rows, float eps, int8_t* __restrict__ q,
                                                                    float* __restrict__ scale, int* status, int64_t drop_row)
{
    using Cfg = RsCfg<COLS, WPR, STAGES, LN>;
    constexpr int VEC = Cfg::VEC;
    extern __shared__ __align__(128) uint8_t rs_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / WPR, sub = warp % WPR;
    uint8_t* ring = rs_smem + (size_t)group * STAGES * Cfg::ROW_BYTES;
    // gamma and beta in two planes each (elements 0-3 and 4-7 of every 8-element vector): a warp's 16-byte reads are contiguous
    const float4* s_gamma = reinterpret_cast<const float4*>(rs_smem + Cfg::RING_BYTES);
    const float4* s_beta = s_gamma + COLS / 4;
    const uint32_t bar0 = ns_smem_u32(rs_smem + Cfg::BAR_OFFSET) + (uint32_t)group * STAGES * 8;
    float* xchg = reinterpret_cast<float*>(rs_smem + Cfg::XCHG_OFFSET) + group * Cfg::XCHG_WORDS;
    const bool producer = sub == 0 && lane == 0;

    if (producer) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) ns_mbar_init(bar0 + 8 * s, 1);
        ns_fence_barrier_init();
    }
    __syncthreads();
    ns_pdl_wait();      // x (and gamma, beta) may be the work of the kernel before this one
    ns_pdl_trigger();

    const int64_t n_groups = (int64_t)gridDim.x * Cfg::GROUPS;
    const int64_t first = (int64_t)blockIdx.x * Cfg::GROUPS + group;
    auto issue = [&](int slot, int64_t r) {
        if (r == drop_row) return;      // test hook (-1 otherwise): this row's copy never comes
        ns_mbar_expect_tx(bar0 + 8 * slot, Cfg::ROW_BYTES);
        rs_bulk_load(ns_smem_u32(ring + (size_t)slot * Cfg::ROW_BYTES), x + (size_t)r * COLS, Cfg::ROW_BYTES, bar0 + 8 * slot);
    };
    if (producer) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            const int64_t r = first + s * n_groups;
            if (r < rows) issue(s, r);
        }
    }
    if (LN) {
        float4* dst = reinterpret_cast<float4*>(rs_smem + Cfg::RING_BYTES);
        for (int i = threadIdx.x; i < COLS / 4; i += RS_THREADS) {
            const int at = (i & 1) * (COLS / 8) + (i >> 1);
            dst[at] = *reinterpret_cast<const float4*>(gamma + 4 * i);
            dst[COLS / 4 + at] = *reinterpret_cast<const float4*>(beta + 4 * i);
        }
        __syncthreads();
    }

    bool failed = false;
    int i = 0;
    for (int64_t r = first; r < rows; r += n_groups, i++) {
        const int slot = i % STAGES;
        const bool ok = __all_sync(0xffffffffu, rs_wait(bar0 + 8 * slot, (uint32_t)(i / STAGES) & 1u));   // one outcome per warp
        float* words = xchg + (i & 1) * 5 * Cfg::NV;
        // reduction `which` (0..3) of this row over the group; with `first_of_row` the outcomes of the warps' waits travel along
        auto group_reduce = [&](float v, bool is_max, int which, bool first_of_row, bool* all_ok) {
            v = ns_rows::warp_reduce(v, is_max);
            if (WPR == 1) {
                if (first_of_row) *all_ok = ok;
                return v;
            }
            if (lane == 0) {
                words[which * Cfg::NV + sub] = v;
                if (first_of_row) words[4 * Cfg::NV + sub] = ok ? 1.0f : 0.0f;
            }
            rs_group_barrier(group, WPR * 32);
            float t = words[which * Cfg::NV];
#pragma unroll
            for (int w = 1; w < WPR; w++) t = is_max ? fmaxf(t, words[which * Cfg::NV + w]) : t + words[which * Cfg::NV + w];
            if (first_of_row) {
                bool a = true;
#pragma unroll
                for (int w = 0; w < WPR; w++) a = a && words[4 * Cfg::NV + w] != 0.0f;
                *all_ok = a;
            }
            return t;
        };
        // A SUM over the row in the order of ns_rows::block_sum_pieces: vector by vector (its eight elements left to right, done
        // by the caller), the 32 vectors of a piece by the xor-shuffle tree, the pieces one after the other -- so LayerNorm
        // gives the same bits whichever kernel family a pass takes.  part[k] is this lane's vector of piece sub * VEC + k.
        auto group_sum = [&](const float (&part)[VEC], int which, bool first_of_row, bool* all_ok) {
            float t[VEC];
#pragma unroll
            for (int k = 0; k < VEC; k++) t[k] = ns_rows::warp_reduce(part[k], false);
            if (WPR == 1) {
                if (first_of_row) *all_ok = ok;
                float r = t[0];
#pragma unroll
                for (int k = 1; k < VEC; k++) r += t[k];
                return r;
            }
            if (lane == 0) {
#pragma unroll
                for (int k = 0; k < VEC; k++) words[which * Cfg::NV + sub * VEC + k] = t[k];
                if (first_of_row) words[4 * Cfg::NV + sub] = ok ? 1.0f : 0.0f;
            }
            rs_group_barrier(group, WPR * 32);
            float r = words[which * Cfg::NV];
#pragma unroll
            for (int v = 1; v < Cfg::NV; v++) r += words[which * Cfg::NV + v];
            if (first_of_row) {
                bool a = true;
#pragma unroll
                for (int w = 0; w < WPR; w++) a = a && words[4 * Cfg::NV + w] != 0.0f;
                *all_ok = a;
            }
            return r;
        };
        uint4 raw[VEC];
        if (ok) {
            const uint4* src = reinterpret_cast<const uint4*>(ring + (size_t)slot * Cfg::ROW_BYTES) + sub * VEC * 32 + lane;
#pragma unroll
            for (int k = 0; k < VEC; k++) raw[k] = src[k * 32];
        } else {
#pragma unroll
            for (int k = 0; k < VEC; k++) raw[k] = make_uint4(0, 0, 0, 0);
        }
        const int64_t next = r + (int64_t)STAGES * n_groups;
        const int vec0 = sub * VEC * 32 + lane;                    // this lane's vector k is vec0 + 32 k
        int8_t* q_row = q + (size_t)r * COLS + (size_t)vec0 * 8;
        bool all_ok = true;

        if (!LN) {
            uint32_t m[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                m[0] = rs_absmax2(m[0], raw[k].x); m[1] = rs_absmax2(m[1], raw[k].y);
                m[2] = rs_absmax2(m[2], raw[k].z); m[3] = rs_absmax2(m[3], raw[k].w);
            }
            // every warp's reduced value depends on all of its reads of the buffer, and the group has met: it may be refilled
            float amax = group_reduce(rs_absmax_or_inf(rs_absmax2(rs_absmax2(m[0], m[1]), rs_absmax2(m[2], m[3]))), true, 0, true, &all_ok);
            if (!all_ok) { failed = true; break; }
            if (producer && next < rows) issue(slot, next);
            bool plain = !(amax <= 3.4028234e38f);
            if (plain) {            // the rule's maximum ignores NaNs
                float a = 0.0f;
#pragma unroll
                for (int k = 0; k < VEC; k++) {
                    float t[8];
                    ns_rows::widen8(raw[k], t);
#pragma unroll
                    for (int j = 0; j < 8; j++) a = fmaxf(a, fabsf(t[j]));
                }
                amax = group_reduce(a, true, 1, false, nullptr);
            }
            const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
            if (producer) scale[r] = sc;
            const float rcp = __frcp_rn(sc);
            plain = plain || !(rcp <= 3.4028234e38f);
            if (!plain) {
#pragma unroll
                for (int k = 0; k < VEC; k++) {
                    float t[8];
                    ns_rows::widen8(raw[k], t);
                    uint32_t lo, hi;
                    ns_rows::quant8<false>(t, sc, rcp, lo, hi);
                    *reinterpret_cast<uint2*>(q_row + (size_t)k * 256) = make_uint2(lo, hi);
                }
            } else {
                for (int k = 0; k < VEC; k++) {
                    float t[8];
                    ns_rows::widen8(raw[k], t);
                    uint32_t lo = 0u, hi = 0u;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        lo |= (uint32_t)(uint8_t)ns_rows::quant_one(t[j], sc) << (8 * j);
                        hi |= (uint32_t)(uint8_t)ns_rows::quant_one(t[4 + j], sc) << (8 * j);
                    }
                    *reinterpret_cast<uint2*>(q_row + (size_t)k * 256) = make_uint2(lo, hi);
                }
            }
        } else {
            float v[VEC * 8];
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                float t[8];
                ns_rows::widen8(raw[k], t);
#pragma unroll
                for (int j = 0; j < 8; j++) v[k * 8 + j] = t[j];
            }
            float part[VEC];
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                float t = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) t += v[k * 8 + j];
                part[k] = t;
            }
            const float mean = group_sum(part, 0, true, &all_ok) / (float)COLS;
            if (!all_ok) { failed = true; break; }
            if (producer && next < rows) issue(slot, next);
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                float t = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) { v[k * 8 + j] -= mean; t = fmaf(v[k * 8 + j], v[k * 8 + j], t); }
                part[k] = t;
            }
            const float inv = 1.0f / sqrtf(group_sum(part, 1, false, nullptr) / (float)COLS + eps);
            uint32_t m[2] = {0u, 0u};
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                const int vec = vec0 + 32 * k;
                const float4 g0 = s_gamma[vec], g1 = s_gamma[COLS / 8 + vec], b0 = s_beta[vec], b1 = s_beta[COLS / 8 + vec];
                const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float h0 = __fadd_rn(__fmul_rn(__fmul_rn(v[k * 8 + j], inv), g[j]), b[j]);
                    const float h1 = __fadd_rn(__fmul_rn(__fmul_rn(v[k * 8 + j + 1], inv), g[j + 1]), b[j + 1]);
                    const uint32_t hb = ns_pack_bf16x2(h0, h1);     // the bf16 rounding of the normalised row
                    m[(j >> 1) & 1] = rs_absmax2(m[(j >> 1) & 1], hb);
                    v[k * 8 + j] = __uint_as_float(hb << 16);
                    v[k * 8 + j + 1] = __uint_as_float(hb & 0xFFFF0000u);
                }
            }
            float amax = group_reduce(rs_absmax_or_inf(rs_absmax2(m[0], m[1])), true, 2, false, nullptr);
            bool plain = !(amax <= 3.4028234e38f);
            if (plain) {
                float a = 0.0f;
#pragma unroll
                for (int j = 0; j < VEC * 8; j++) a = fmaxf(a, fabsf(v[j]));
                amax = group_reduce(a, true, 3, false, nullptr);
            }
            const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
            if (producer) scale[r] = sc;
            const float rcp = __frcp_rn(sc);
            plain = plain || !(rcp <= 3.4028234e38f);
            if (!plain) {
#pragma unroll
                for (int k = 0; k < VEC; k++) {
                    uint32_t lo, hi;
                    ns_rows::quant8<false>(v + k * 8, sc, rcp, lo, hi);
                    *reinterpret_cast<uint2*>(q_row + (size_t)k * 256) = make_uint2(lo, hi);
                }
            } else {
                for (int k = 0; k < VEC; k++) {
                    uint32_t lo = 0u, hi = 0u;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        lo |= (uint32_t)(uint8_t)ns_rows::quant_one(v[k * 8 + j], sc) << (8 * j);
                        hi |= (uint32_t)(uint8_t)ns_rows::quant_one(v[k * 8 + 4 + j], sc) << (8 * j);
                    }
                    *reinterpret_cast<uint2*>(q_row + (size_t)k * 256) = make_uint2(lo, hi);
                }
            }
        }
    }
    if (failed) {
        if (producer) *reinterpret_cast<volatile int*>(status) = 600 + WPR;
        // the copies still on their way into this CTA's buffers get one more bounded wait before the CTA gives its memory back
        for (int j = 0; j < STAGES; j++) {
            const int64_t idx = (int64_t)i + j;
            if (first + idx * n_groups < rows) rs_wait(bar0 + 8 * (uint32_t)(idx % STAGES), (uint32_t)(idx / STAGES) & 1u);
        }
    }
}

template <int COLS, int WPR, int STAGES, bool LN>
cudaError_t rs_launch(NsDevice* d, const uint16_t* x, const float* gamma, const float* beta, int64_t rows, float eps, int8_t* q, float* scale)
{
    using Cfg = RsCfg<COLS, WPR, STAGES, LN>;
    auto* kernel = ns_rows_stream_kernel<COLS, WPR, STAGES, LN>;
    static int ctas_per_sm[64] = {0};
    int& per_sm = ctas_per_sm[d->ordinal & 63];
    if (per_sm == 0) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        int n = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, RS_THREADS, (size_t)Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        per_sm = n < 1 ? 1 : n;
    }
    int64_t ctas = (rows + Cfg::GROUPS - 1) / Cfg::GROUPS;
    const int64_t cap = (int64_t)d->sm_count * per_sm;
    if (ctas > cap) ctas = cap;
    return ns_launch_plain(kernel, dim3((unsigned)ctas), dim3(RS_THREADS), (size_t)Cfg::SMEM_BYTES, d->stream, x, gamma, beta, rows, eps, q, scale,
                           d->status_dev, (int64_t)d->rows_drop);
}

}  // namespace

// Whether the many-row kernels take rows of `cols` bf16 elements.
bool ns_rows_stream_fits(bool layernorm, int64_t rows, int cols)
{
    if (rows < ns_rows::MANY_ROWS) return false;
    return cols == 1024 || cols == 2048 || cols == 4096 || (!layernorm && cols == 8192);
}

// Shapes measured on 32768 rows: quantisation is fastest with 64 elements per lane (rows of 8192: 138 us against 160 with 32,
// 89 % of the HBM rate), LayerNorm with 32 (rows of 2048: 82 us against 89; it holds the row as floats, so 64 per lane
// leave 16 warps per SM).
cudaError_t ns_rows_stream_quantize(NsDevice* d, const uint16_t* x, int64_t rows, int cols, int8_t* q, float* scale)
{
    switch (cols) {
        case 1024: return rs_launch<1024, 1, 3, false>(d, x, nullptr, nullptr, rows, 0.0f, q, scale);
        case 2048: return rs_launch<2048, 1, 2, false>(d, x, nullptr, nullptr, rows, 0.0f, q, scale);
        case 4096: return rs_launch<4096, 2, 2, false>(d, x, nullptr, nullptr, rows, 0.0f, q, scale);
        default: return rs_launch<8192, 4, 2, false>(d, x, nullptr, nullptr, rows, 0.0f, q, scale);
    }
}

cudaError_t ns_rows_stream_layernorm(NsDevice* d, const uint16_t* x, const float* gamma, const float* beta, int64_t rows, int cols, float eps, int8_t* q,
                                     float* scale)
{
    switch (cols) {
        case 1024: return rs_launch<1024, 1, 3, true>(d, x, gamma, beta, rows, eps, q, scale);
        case 2048: return rs_launch<2048, 2, 3, true>(d, x, gamma, beta, rows, eps, q, scale);
        default: return rs_launch<4096, 4, 2, true>(d, x, gamma, beta, rows, eps, q, scale);
    }
}
