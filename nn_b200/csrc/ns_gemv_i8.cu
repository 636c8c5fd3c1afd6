// int8 product for one to eight activation rows (single-sequence and small-batch decoding steps): an HBM-streaming
// kernel on the CUDA cores.  With so few rows the tensor cores would multiply padding; what bounds the product is
// reading the weights once, N * K bytes.
//
// Reference path: Linear.Forward -> Tensor.MatMul -> matmul_f32 (src/NeuralSharp/Backends/Cuda/PtxKernels.cs, one
// thread per output element striding down a weight column; src/NeuralSharp/Tensor.Advanced.cs:29-106).  Here, as in
// the tensor-core path, the weights are int8 [N, K] with one scale per output channel, the activations int8 with one
// scale per row, the sums exact int32 and the epilogue ((float)acc * a_scale) * w_scale + bias (+ GELU / residual).
//
// Work split.  A weight row is cut into pieces of 512 bytes: a warp reads a piece with one 16-byte load per lane.
// Warp w of a CTA owns pieces w * CPW .. w * CPW + CPW - 1 of EVERY row the CTA handles, so the activations that meet
// those bytes (MR rows x CPW x 16 bytes per lane) are loaded once into registers and stay there.  A CTA takes a
// contiguous range of N / gridDim.x columns (the ranges differ by at most one column, so all SMs finish together)
// and walks it four (eight for one or two rows) columns at a time; the loads of the next group are issued as soon as
// a register slot is consumed, so every warp keeps four or eight pieces (2 - 4 KB) in flight.  Per column: 4 * MR
// dp4a per lane and piece, then a transposing butterfly over the lanes (MR - 1 + log2(32 / MR) shuffles instead of
// 5 * MR) that leaves row r's sum in lane r * 32 / MR, one shared-memory word per (warp, column, row), and after a
// CTA barrier one thread per (column, row) adds the warps' words and applies the epilogue.  Its per-column operands
// were fetched before the barrier, and the words are double-buffered, so a group costs one barrier.
//
// Measured (K = N = 4096, CUDA events, operands rotated beyond L2): 5.3 / 5.5 / 8.0 us at 1 / 4 / 8 rows against
// 9.9 - 10.0 us for the tensor-core kernel with split K and its second pass.  At 16 rows the dp4a and shuffle issue
// rate makes this kernel slower (11.5 against 10.2 us), so products of nine rows and more stay on the tensor cores.
#include "ns_gemm.cuh"

namespace {

// columns per group (= pieces in flight per warp and activation piece): eight for one or two rows, where the
// registers allow it and a CTA's whole share of columns is then fetched in one or two rounds of loads
__host__ __device__ constexpr int gv_cols(int mr) { return mr <= 2 ? 8 : 4; }
constexpr int GV_MAX_WARPS = 16;

__device__ __forceinline__ int4 gv_load_stream(const int8_t* ptr)
{
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

// Sums v[r] over the 32 lanes for every r < MR; returns row (lane * MR / 32)'s total (in all lanes of that row's group).
template <int MR>
__device__ __forceinline__ int gv_reduce_rows(int (&v)[MR], int lane)
{
    int o = 16;
#pragma unroll
    for (int cnt = MR; cnt > 1; cnt >>= 1) {
        const int half = cnt >> 1;
        const bool up = (lane & o) != 0;      // lanes with this bit set keep the upper half of the rows
#pragma unroll
        for (int i = 0; i < half; i++) {
            const int send = up ? v[i] : v[i + half];
            const int keep = up ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
        o >>= 1;
    }
    int r = v[0];
#pragma unroll
    for (; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

template <int MR, int CPW>
__global__ void __launch_bounds__(GV_MAX_WARPS * 32, 1)
ns_gemv_i8_kernel(const NsGemmParams p, const int8_t* __restrict__ a, const int8_t* __restrict__ w)
{
    constexpr int GV_COLS = gv_cols(MR);
    __shared__ int red[2][GV_MAX_WARPS][GV_COLS][MR];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int col_begin = (int)((int64_t)blockIdx.x * p.N / gridDim.x);
    const int col_end = (int)((int64_t)(blockIdx.x + 1) * p.N / gridDim.x);

    int kb[CPW];
    bool kv[CPW];
#pragma unroll
    for (int c = 0; c < CPW; c++) {
        kb[c] = ((warp * CPW + c) * 32 + lane) * 16;
        kv[c] = kb[c] < p.K;
    }
    int4 wv[GV_COLS][CPW];
    auto load_col = [&](int slot, int n) {
#pragma unroll
        for (int c = 0; c < CPW; c++)
            wv[slot][c] = (n < col_end && kv[c]) ? gv_load_stream(w + (size_t)n * p.K + kb[c]) : make_int4(0, 0, 0, 0);
    };
    // A Linear's weights are written by no kernel on the stream: their first columns are fetched while the kernel before this
    // one is still running (the launch is programmatic); everything else waits for it.
    if (p.prefetch_b) {
#pragma unroll
        for (int s = 0; s < GV_COLS; s++) load_col(s, col_begin + s);
    }
    ns_pdl_wait();
    ns_pdl_trigger();       // after the wait, as everywhere in the library: with the trigger before it, replayed graphs of a step gave other tokens
    a = ns_after_wait(a);                                   // the activations and their scales are the previous kernel's
    const float* a_scales = ns_after_wait(p.a_scale);
    if (!p.prefetch_b) {
#pragma unroll
        for (int s = 0; s < GV_COLS; s++) load_col(s, col_begin + s);
    }

    // this lane's activation bytes, all rows
    int4 x[CPW][MR];
#pragma unroll
    for (int c = 0; c < CPW; c++)
#pragma unroll
        for (int m = 0; m < MR; m++)
            x[c][m] = (m < p.M && kv[c]) ? __ldg(reinterpret_cast<const int4*>(a + (size_t)m * p.K + kb[c])) : make_int4(0, 0, 0, 0);

    // the threads of the epilogue: thread t finishes (row t / GV_COLS, column t % GV_COLS) of every group
    const int f_row = threadIdx.x / GV_COLS, f_col = threadIdx.x % GV_COLS;
    const bool f_row_ok = threadIdx.x < GV_COLS * MR && f_row < p.M;
    const float a_scale = (f_row_ok && p.out != nullptr) ? __ldg(&a_scales[f_row]) : 1.0f;
    constexpr int LANES_PER_ROW = 32 / MR;

    int buf = 0;
    for (int n0 = col_begin; n0 < col_end; n0 += GV_COLS, buf ^= 1) {
        // operands of this group's epilogue, in flight while the group is summed
        const int fn = n0 + f_col;
        const bool f_ok = f_row_ok && fn < col_end;
        const size_t f_idx = (size_t)f_row * p.N + fn;
        float f_ws = 1.0f, f_bias = 0.0f, f_res = 0.0f;
        if (f_ok && p.out != nullptr) {
            f_ws = __ldg(&p.w_scale[fn]);
            if (p.epilogue != NS_EPI_NONE) f_bias = __ldg(&p.bias[fn]);
            if (p.epilogue == NS_EPI_BIAS_RESIDUAL) f_res = ns_gemm_residual(p, f_idx);
        }
#pragma unroll
        for (int s = 0; s < GV_COLS; s++) {
            int acc[MR];
#pragma unroll
            for (int m = 0; m < MR; m++) acc[m] = 0;
#pragma unroll
            for (int c = 0; c < CPW; c++) {
                const int4 wq = wv[s][c];
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    acc[m] = __dp4a(wq.x, x[c][m].x, acc[m]);
                    acc[m] = __dp4a(wq.y, x[c][m].y, acc[m]);
                    acc[m] = __dp4a(wq.z, x[c][m].z, acc[m]);
                    acc[m] = __dp4a(wq.w, x[c][m].w, acc[m]);
                }
            }
            load_col(s, n0 + GV_COLS + s);     // the slot is free: fetch the same column of the next group
            const int tot = gv_reduce_rows<MR>(acc, lane);
            if ((lane & (LANES_PER_ROW - 1)) == 0) red[buf][warp][s][lane / LANES_PER_ROW] = tot;
        }
        __syncthreads();
        if (f_ok) {
            int sum = 0;
            for (int wi = 0; wi < warps; wi++) sum += red[buf][wi][f_col][f_row];
            if (p.raw != nullptr) p.raw[f_idx] = sum;
            if (p.out != nullptr) {
                float v = ns_gemm_finish_i8(p, sum, a_scale, f_ws, f_bias);
                if (p.epilogue == NS_EPI_BIAS_RESIDUAL) v = __fadd_rn(v, f_res);
                if (p.out_dtype == NS_F32) reinterpret_cast<float*>(p.out)[f_idx] = v;
                else reinterpret_cast<uint16_t*>(p.out)[f_idx] = ns_f32_to_bf16_bits(v);
            }
        }
        // no second barrier: the next group writes the other buffer, and the one after it comes after the next barrier
    }
}

template <int MR, int CPW>
int launch_gemv(NsDevice* d, const NsGemmParams& p, const void* a, const void* w, int warps)
{
    constexpr int GV_COLS = gv_cols(MR);
    auto kernel = ns_gemv_i8_kernel<MR, CPW>;
    static int ctas_per_sm[GV_MAX_WARPS + 1] = {0};
    if (ctas_per_sm[warps] == 0) {
        int n = 0;
        NS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, warps * 32, 0));
        const int cap = 32 / warps < 1 ? 1 : 32 / warps;     // 32 resident warps per SM are plenty of loads in flight
        ctas_per_sm[warps] = n < 1 ? 1 : (n > cap ? cap : n);
    }
    int64_t grid = (int64_t)d->sm_count * ctas_per_sm[warps];
    // at least one group of columns per CTA
    const int64_t groups = (p.N + GV_COLS - 1) / GV_COLS;
    if (grid > groups) grid = groups;
    NS_CUDA(ns_launch_pdl(kernel, dim3((unsigned)grid), dim3(warps * 32), 0, d->stream, p, reinterpret_cast<const int8_t*>(a),
                          reinterpret_cast<const int8_t*>(w)));
    return NS_OK;
}

}  // namespace

bool ns_gemv_i8_fits(int M, int K)
{
    if (M < 1 || M > 8 || K % 16 != 0) return false;
    const int mr = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
    const int pieces = (K + 511) / 512;
    const int cpw_max = 16 / mr < 4 ? 16 / mr : 4;      // 64 activation registers per lane at most
    return pieces <= GV_MAX_WARPS * cpw_max;
}

int ns_gemv_i8_run(NsDevice* d, const NsGemmParams& p, const void* a, const void* w)
{
    NS_REQUIRE(ns_gemv_i8_fits(p.M, p.K), NS_ERR_ARGUMENT, "M=%d K=%d does not fit the row-streaming int8 kernel", p.M, p.K);
    const int mr = p.M <= 1 ? 1 : p.M <= 2 ? 2 : p.M <= 4 ? 4 : 8;
    const int pieces = (p.K + 511) / 512;
    int cpw = 1;
    while (pieces > GV_MAX_WARPS * cpw) cpw *= 2;
    // three and four rows: two pieces per warp halve the lane-summing butterflies per dp4a, which is what bounds them
    // (32768 x 8192 weights: 57.7 -> 43.6 us = 6.17 TB/s); at eight rows the same change gained 6 % there and lost
    // at K = 2048, so eight rows keep one piece per warp
    if (mr == 4 && cpw == 1 && pieces >= 4) cpw = 2;
    // one warp per CPW pieces of a row; the epilogue needs a thread per (column of a group, row) (a warp without a
    // piece adds zeros)
    int warps = (pieces + cpw - 1) / cpw;
    if (warps * 32 < gv_cols(mr) * mr) warps = (gv_cols(mr) * mr + 31) / 32;
#define GV_CASE(MR_, CPW_) \
    if (mr == MR_ && cpw == CPW_) return launch_gemv<MR_, CPW_>(d, p, a, w, warps);
    GV_CASE(1, 1) GV_CASE(1, 2) GV_CASE(1, 4)
    GV_CASE(2, 1) GV_CASE(2, 2) GV_CASE(2, 4)
    GV_CASE(4, 1) GV_CASE(4, 2) GV_CASE(4, 4)
    GV_CASE(8, 1) GV_CASE(8, 2)
#undef GV_CASE
    return ns_fail(NS_ERR_ARGUMENT, "no row-streaming int8 kernel for M=%d K=%d", p.M, p.K);
}
