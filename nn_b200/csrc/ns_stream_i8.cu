// int8 product for 9 to 16 activation rows (the decoding step of a small batch): an HBM-streaming kernel in ONE launch --
// the weights go from global memory straight into registers, the K split is summed inside the CTA, and the epilogue runs
// in the same kernel.  (The kernel is written for up to four 16-row tiles; more than one is not dispatched, see below.)
//
// Reference path: Linear.Forward -> Tensor.MatMul -> matmul_f32 (src/NeuralSharp/Backends/Cuda/PtxKernels.cs:484-627) at a
// tiny row count (m = batch, one new position each: the hot loop of a cached decoding step, src/NeuralSharp/Layers/
// Sequential.cs:59-80).  As everywhere in this library the weights are int8 [N, K] with one scale per output channel, the
// activations int8 with one scale per row, the sums exact int32 and the epilogue ((float)acc * a_scale) * w_scale + bias
// (+ GELU / residual), operation for operation that of the other int8 kernels, so results are bit-identical to theirs.
//
// Why not the tcgen05 kernel: with 64 rows that kernel is a chain of dependent round trips (barrier and tensor-memory
// set-up, TMA of the activations, MMA, accumulator read, store of partial sums, their completion: 4.7 us for
// 64 x 2048 x 2048 with L2-resident weights) followed by a second kernel that adds the K splits -- for 4 to 17 MB of weights
// that stream in 0.6 to 2.6 us.  Here the chain is: load, multiply, add across warps, store.  The multiply is the
// warp-level mma.sync.m16n8k32 (s8 x s8 -> s32): 16 activation rows against 8 weight rows per instruction, which is the
// shape of this problem.  Its rate matters, though: measured on B200 the warp-level int8 MMA sustains about one
// m16n8k32 per 12.6 cycles and SM (~190 TOPS for the whole GPU, against thousands for tcgen05), so the kernel is bound by
// the weight stream only at ONE 16-row tile: 16 x 4096 x 4096 takes 5.9 us against 9.1 us for the tcgen05 kernel with its
// second pass, but 64 x 8192 x 2048 takes 11.8 us against 10.3 and 64 x 32000 x 2048 32.7 us against 19.3.  Products of 17
// rows and more therefore stay on the tcgen05 kernels.
//
// Work split (the row-streaming kernel's, ns_gemv_i8.cu, with the dot products on the tensor cores).  K is cut into
// groups of 64 bytes; warp w of the 16 warps of a CTA owns KGW consecutive groups of EVERY weight row the CTA handles, so
// the activations that meet them (MT x 16 rows x KGW x 64 bytes) are loaded once into registers as A fragments and stay
// there.  A CTA takes a contiguous range of 8-column tiles and walks it G tiles at a time: per tile and group one
// 16-byte load per lane (8 weight rows x 64 bytes per warp), two mma.sync per 16-row tile; the loads of the next G tiles
// are issued as soon as a register slot is consumed.  Then every warp leaves its partial sums in shared memory, and
// after a barrier one thread per (row, column pair) adds the 16 warps' words and applies the epilogue.
//
// Fragment layout.  In m16n8k32 a lane (g = lane / 4, q = lane % 4) holds of A the bytes k = 4q..4q+3 and 16+4q..16+4q+3
// of rows g and g + 8, and of B the same k bytes of weight row g.  Any permutation of k may be applied to A and B alike:
// a lane loads the 16 consecutive bytes 16q..16q+15 of its row of a 64-byte group and feeds words 0,1 to one mma and
// words 2,3 to a second -- the same words of A and of B meet, every byte of the group is used once.
#include "ns_gemm.cuh"

namespace {

constexpr int ST_WARPS = 16;
constexpr int ST_THREADS = ST_WARPS * 32;

__device__ __forceinline__ uint4 st_load_stream(const int8_t* ptr)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

__device__ __forceinline__ void st_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: 16-row tiles of activations (M <= 16 MT).  KGW: 64-byte K groups per warp (K <= 16 * KGW * 64).  G: 8-column tiles per round.
template <int MT, int KGW, int G>
__global__ void __launch_bounds__(ST_THREADS, 1)
ns_stream_i8_kernel(const NsGemmParams p, const int8_t* __restrict__ a, const int8_t* __restrict__ w)
{
    extern __shared__ int st_red[];   // [ST_WARPS][G * MT * 32 lanes * 4] partial sums of one round
    constexpr int ROUND_WORDS = G * MT * 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int n_tiles = (p.N + 7) >> 3;
    const int tile_begin = (int)((int64_t)blockIdx.x * n_tiles / gridDim.x);
    const int tile_end = (int)((int64_t)(blockIdx.x + 1) * n_tiles / gridDim.x);

    // this lane's byte offset inside a row for each of its K groups (a group past the end of K contributes zeros)
    int koff[KGW];
    bool kv[KGW];
#pragma unroll
    for (int c = 0; c < KGW; c++) {
        koff[c] = (warp * KGW + c) * 64 + q * 16;
        kv[c] = koff[c] < p.K;
    }
    uint4 bw[G][KGW];
    auto load_tile = [&](int slot, int tile) {
        // weight row of this lane in the tile; rows past N repeat the last row (their columns are never stored)
        const int n = min(tile * 8 + g, p.N - 1);
#pragma unroll
        for (int c = 0; c < KGW; c++)
            bw[slot][c] = (tile < tile_end && kv[c]) ? st_load_stream(w + (size_t)n * p.K + koff[c]) : make_uint4(0, 0, 0, 0);
    };
    // Weights of a Linear object are not written by the kernel before this one: their first tiles may be requested
    // before that kernel has finished.  A caller's own operands wait.
    if (p.prefetch_b) {
#pragma unroll
        for (int s = 0; s < G; s++) load_tile(s, tile_begin + s);
    }
    ns_pdl_wait();
    ns_pdl_trigger();
    a = ns_after_wait(a);                                   // the activations and their scales are the previous kernel's
    const float* a_scales = ns_after_wait(p.a_scale);
    if (!p.prefetch_b) {
#pragma unroll
        for (int s = 0; s < G; s++) load_tile(s, tile_begin + s);
    }

    // A fragments: rows g and g + 8 of every 16-row tile, this warp's K groups
    uint4 alo[MT][KGW], ahi[MT][KGW];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int c = 0; c < KGW; c++) {
            const int r0 = mt * 16 + g, r1 = r0 + 8;
            alo[mt][c] = (r0 < p.M && kv[c]) ? __ldg(reinterpret_cast<const uint4*>(a + (size_t)r0 * p.K + koff[c])) : make_uint4(0, 0, 0, 0);
            ahi[mt][c] = (r1 < p.M && kv[c]) ? __ldg(reinterpret_cast<const uint4*>(a + (size_t)r1 * p.K + koff[c])) : make_uint4(0, 0, 0, 0);
        }

    // the threads of the epilogue: thread t finishes two adjacent columns of one row of every round
    //   t = ((mt * G + s) * 32 + lane') * 2 + hi  ->  row = mt * 16 + g' + 8 hi, columns 2 q', 2 q' + 1 of tile s
    const int f_hi = threadIdx.x & 1, f_lane = (threadIdx.x >> 1) & 31, f_pair = threadIdx.x >> 6;
    const int f_mt = f_pair / G, f_s = f_pair % G;
    const int f_row = f_mt * 16 + (f_lane >> 2) + 8 * f_hi;
    const bool f_active = f_pair < MT * G && f_row < p.M;
    const float a_scale = (f_active && p.out != nullptr) ? __ldg(&a_scales[f_row]) : 1.0f;

    for (int t0 = tile_begin; t0 < tile_end; t0 += G) {
        // operands of this round's epilogue, in flight while the round is summed
        const int f_col = (t0 + f_s) * 8 + (f_lane & 3) * 2;
        const bool f_ok0 = f_active && t0 + f_s < tile_end && f_col < p.N;
        const bool f_ok1 = f_ok0 && f_col + 1 < p.N;
        const size_t f_idx = (size_t)f_row * p.N + f_col;
        float f_ws[2] = {1.0f, 1.0f}, f_bias[2] = {0.0f, 0.0f}, f_res[2] = {0.0f, 0.0f};
        if (f_ok0 && p.out != nullptr) {
            f_ws[0] = __ldg(&p.w_scale[f_col]);
            if (f_ok1) f_ws[1] = __ldg(&p.w_scale[f_col + 1]);
            if (p.epilogue != NS_EPI_NONE) {
                f_bias[0] = __ldg(&p.bias[f_col]);
                if (f_ok1) f_bias[1] = __ldg(&p.bias[f_col + 1]);
            }
            if (p.epilogue == NS_EPI_BIAS_RESIDUAL) {
                f_res[0] = ns_gemm_residual(p, f_idx);
                if (f_ok1) f_res[1] = ns_gemm_residual(p, f_idx + 1);
            }
        }
        int acc[G][MT][4];
#pragma unroll
        for (int s = 0; s < G; s++) {
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[s][mt][i] = 0;
#pragma unroll
            for (int c = 0; c < KGW; c++) {
                const uint4 b = bw[s][c];
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    st_mma(acc[s][mt], alo[mt][c].x, ahi[mt][c].x, alo[mt][c].y, ahi[mt][c].y, b.x, b.y);
                    st_mma(acc[s][mt], alo[mt][c].z, ahi[mt][c].z, alo[mt][c].w, ahi[mt][c].w, b.z, b.w);
                }
            }
            load_tile(s, t0 + G + s);      // the slot is free: fetch the same tile of the next round
        }
        // partial sums of this warp: [tile s][mt][lane][4 words]
        int* mine = st_red + warp * ROUND_WORDS;
#pragma unroll
        for (int s = 0; s < G; s++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
                *reinterpret_cast<int4*>(mine + ((mt * G + s) * 32 + lane) * 4) = make_int4(acc[s][mt][0], acc[s][mt][1], acc[s][mt][2], acc[s][mt][3]);
        __syncthreads();
        if (f_ok0) {
            int s0 = 0, s1 = 0;
            const int* src = st_red + (f_pair * 32 + f_lane) * 4 + f_hi * 2;
#pragma unroll
            for (int wi = 0; wi < ST_WARPS; wi++) {
                const int2 v = *reinterpret_cast<const int2*>(src + wi * ROUND_WORDS);
                s0 += v.x; s1 += v.y;
            }
            if (p.raw != nullptr) {
                p.raw[f_idx] = s0;
                if (f_ok1) p.raw[f_idx + 1] = s1;
            }
            if (p.out != nullptr) {
                float v0 = ns_gemm_finish_i8(p, s0, a_scale, f_ws[0], f_bias[0]);
                float v1 = ns_gemm_finish_i8(p, s1, a_scale, f_ws[1], f_bias[1]);
                if (p.epilogue == NS_EPI_BIAS_RESIDUAL) { v0 = __fadd_rn(v0, f_res[0]); v1 = __fadd_rn(v1, f_res[1]); }
                if (p.out_dtype == NS_F32) {
                    float* dst = reinterpret_cast<float*>(p.out) + f_idx;
                    dst[0] = v0;
                    if (f_ok1) dst[1] = v1;
                } else {
                    uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) + f_idx;
                    dst[0] = ns_f32_to_bf16_bits(v0);
                    if (f_ok1) dst[1] = ns_f32_to_bf16_bits(v1);
                }
            }
        }
        __syncthreads();   // the words are written again by the next round
    }
}

template <int MT, int KGW, int G>
int launch_stream(NsDevice* d, const NsGemmParams& p, const void* a, const void* w)
{
    auto kernel = ns_stream_i8_kernel<MT, KGW, G>;
    constexpr size_t smem = (size_t)ST_WARPS * G * MT * 128 * sizeof(int);
    static bool configured[64] = {false};
    if (!configured[d->ordinal]) {
        NS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[d->ordinal] = true;
    }
    // one CTA per SM; at least one round of tiles per CTA
    const int tiles = (p.N + 7) / 8;
    const int rounds = (tiles + G - 1) / G;
    const int grid = rounds < d->sm_count ? rounds : d->sm_count;
    NS_CUDA(ns_launch_pdl(kernel, dim3((unsigned)grid), dim3(ST_THREADS), smem, d->stream, p, reinterpret_cast<const int8_t*>(a),
                          reinterpret_cast<const int8_t*>(w)));
    return NS_OK;
}

}  // namespace

// Shapes the kernel takes: 9..16 rows (one 16-row tile: with more the warp-level MMA rate, not the weight stream, bounds it),
// K a multiple of 16 up to 8192 (16 warps x 8 groups of 64 bytes in registers), 16-byte aligned operands.
bool ns_stream_i8_fits(int M, int K)
{
    if (M < 9 || M > 16 || K % 16 != 0) return false;
    const int groups = (K + 63) / 64;
    return (groups + ST_WARPS - 1) / ST_WARPS <= 8;
}

int ns_stream_i8_run(NsDevice* d, const NsGemmParams& p, const void* a, const void* w)
{
    NS_REQUIRE(ns_stream_i8_fits(p.M, p.K), NS_ERR_ARGUMENT, "M=%d K=%d does not fit the streaming int8 kernel", p.M, p.K);
    const int groups = (p.K + 63) / 64;
    const int kgw = (groups + ST_WARPS - 1) / ST_WARPS;
    if (kgw <= 1) return launch_stream<1, 1, 2>(d, p, a, w);
    if (kgw <= 2) return launch_stream<1, 2, 2>(d, p, a, w);
    if (kgw <= 4) return launch_stream<1, 4, 2>(d, p, a, w);
    return launch_stream<1, 8, 1>(d, p, a, w);
}
