// A row of activations held in the REGISTERS of one CTA: the building block of the fast row kernels (LayerNorm with
// int8 output, int8 row quantisation, and the fused epilogue + LayerNorm + quantisation of the decoding step).
//
// The reference runs its row operators with one THREAD per row (layernorm_fused_f32, src/NeuralSharp/Backends/Cuda/
// PtxKernels.Decoding.cs:61-90).  Here a CTA owns a row of cols = VPT * threads * 8 elements: thread t holds the
// 8-element vectors j * threads + t (j < VPT), so loads and stores are 16-byte (8-byte for int8) and contiguous across
// the CTA, nothing is staged in shared memory, and a reduction is five shuffles, one shared-memory word per warp and
// ONE barrier (each reduction of a row has its own words).  One warp per row was measured too: with 64 to 256
// elements per lane the divisions of the quantisation make a single warp issue-bound (20 us for rows of 8192).
#pragma once

#include "ns_common.cuh"

namespace ns_rows {

constexpr int MAX_WARPS = 8;

struct RowShared {
    float red[3][MAX_WARPS];   // one set of per-warp partials per reduction of a row pass
};

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    const int warps = blockDim.x >> 5;
    if (warps == 1) return v;
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < warps; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

__device__ __forceinline__ int8_t quant_one(float v, float scale)
{
    float q = rintf(__fdiv_rn(v, scale));
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return (int8_t)q;
}

// 8 bf16 values (one 16-byte vector) -> 8 floats
__device__ __forceinline__ void widen8(const uint4 raw, float (&v)[8])
{
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int t = 0; t < 4; t++) {
        v[2 * t] = __uint_as_float(w[t] << 16);
        v[2 * t + 1] = __uint_as_float(w[t] & 0xFFFF0000u);
    }
}

// first column of vector j of this thread
__device__ __forceinline__ int vec_col(int j) { return (j * (int)blockDim.x + (int)threadIdx.x) * 8; }

// Row quantisation of values in registers: scale = absmax / 127 (1 for a zero row), q = clamp(rint(x / scale)).
// `red` must not be in use by another reduction of the same pass; a __syncthreads() separates passes (rows).
template <int VPT>
__device__ __forceinline__ void quantize_row(const float (&x)[VPT * 8], int8_t* __restrict__ q_row, float* __restrict__ scale_out, float* red)
{
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT * 8; i++) amax = fmaxf(amax, fabsf(x[i]));
    amax = block_reduce(amax, true, red);
    const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) *scale_out = sc;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int t = 0; t < 4; t++) {
            lo |= (uint32_t)(uint8_t)quant_one(x[j * 8 + t], sc) << (8 * t);
            hi |= (uint32_t)(uint8_t)quant_one(x[j * 8 + 4 + t], sc) << (8 * t);
        }
        *reinterpret_cast<uint2*>(q_row + vec_col(j)) = make_uint2(lo, hi);
    }
}

// LayerNorm of the row in registers (statistics in float: mean, then centred variance), rounded to bf16, then quantised.
// gamma and beta are fetched before the first reduction so that their latency hides behind it.
template <int VPT>
__device__ __forceinline__ void layernorm_quantize_row(float (&x)[VPT * 8], const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                                       int cols, int8_t* __restrict__ q_row, float* __restrict__ scale_out, RowShared& sh)
{
    float4 g[VPT][2], b[VPT][2];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const int col = vec_col(j);
        g[j][0] = __ldg(reinterpret_cast<const float4*>(gamma + col)); g[j][1] = __ldg(reinterpret_cast<const float4*>(gamma + col + 4));
        b[j][0] = __ldg(reinterpret_cast<const float4*>(beta + col)); b[j][1] = __ldg(reinterpret_cast<const float4*>(beta + col + 4));
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT * 8; i++) s += x[i];
    const float mean = block_reduce(s, false, sh.red[0]) / (float)cols;
    float v2 = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT * 8; i++) { const float d = x[i] - mean; v2 += d * d; }
    const float inv = 1.0f / sqrtf(block_reduce(v2, false, sh.red[1]) / (float)cols + eps);
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const float gg[8] = {g[j][0].x, g[j][0].y, g[j][0].z, g[j][0].w, g[j][1].x, g[j][1].y, g[j][1].z, g[j][1].w};
        const float bb[8] = {b[j][0].x, b[j][0].y, b[j][0].z, b[j][0].w, b[j][1].x, b[j][1].y, b[j][1].z, b[j][1].w};
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const float h = __fadd_rn(__fmul_rn(__fmul_rn(x[j * 8 + t] - mean, inv), gg[t]), bb[t]);
            x[j * 8 + t] = ns_bf16_bits_to_f32(ns_f32_to_bf16_bits(h));
        }
    }
    quantize_row<VPT>(x, q_row, scale_out, sh.red[2]);
}

// ---- many rows: one WARP per row.  With thousands of rows every SM holds dozens of independent warps, each with all of
// its row's loads in flight at once, which a CTA walking its rows one after another (a chain of three barriers per
// row) cannot match: LayerNorm -> int8 of 32768 x 2048 ran at 1.1 TB/s with a CTA per row.  Lane l holds the vectors
// k * 32 + l (k < VEC), cols = VEC * 256.
__device__ __forceinline__ float warp_reduce(float v, bool is_max)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    return v;
}

template <int VEC>
__device__ __forceinline__ void warp_quantize_row(const float (&x)[VEC * 8], int8_t* __restrict__ q_row, float* __restrict__ scale_out, int lane)
{
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC * 8; i++) amax = fmaxf(amax, fabsf(x[i]));
    amax = warp_reduce(amax, true);
    const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    if (lane == 0) *scale_out = sc;
#pragma unroll
    for (int k = 0; k < VEC; k++) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int t = 0; t < 4; t++) {
            lo |= (uint32_t)(uint8_t)quant_one(x[k * 8 + t], sc) << (8 * t);
            hi |= (uint32_t)(uint8_t)quant_one(x[k * 8 + 4 + t], sc) << (8 * t);
        }
        *reinterpret_cast<uint2*>(q_row + (size_t)(k * 32 + lane) * 8) = make_uint2(lo, hi);
    }
}

template <int VEC>
__device__ __forceinline__ void warp_layernorm_quantize_row(float (&x)[VEC * 8], const float* __restrict__ gamma, const float* __restrict__ beta,
                                                            float eps, int8_t* __restrict__ q_row, float* __restrict__ scale_out, int lane)
{
    constexpr int COLS = VEC * 256;
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC * 8; i++) s += x[i];
    const float mean = warp_reduce(s, false) / (float)COLS;
    float v2 = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC * 8; i++) { const float d = x[i] - mean; v2 += d * d; }
    const float inv = 1.0f / sqrtf(warp_reduce(v2, false) / (float)COLS + eps);
#pragma unroll
    for (int k = 0; k < VEC; k++) {
        const int col = (k * 32 + lane) * 8;
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + col)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + col + 4));
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + col)), b1 = __ldg(reinterpret_cast<const float4*>(beta + col + 4));
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const float h = __fadd_rn(__fmul_rn(__fmul_rn(x[k * 8 + t] - mean, inv), g[t]), b[t]);
            x[k * 8 + t] = ns_bf16_bits_to_f32(ns_f32_to_bf16_bits(h));
        }
    }
    warp_quantize_row<VEC>(x, q_row, scale_out, lane);
}

// Rows at and above this count take the warp-per-row kernels.
constexpr int64_t MANY_ROWS = 2048;

// CTA shape for rows of `cols` elements (cols % 256 == 0): threads = min(256, cols / 8), vectors per thread = cols / 8 /
// threads.  Returns false when the row does not fit the register-resident kernels (more than 4 vectors per thread).
inline bool row_shape(int cols, unsigned* threads, int* vpt)
{
    if (cols <= 0 || cols % 256 != 0) return false;
    const int vecs = cols / 8;
    const int t = vecs < 256 ? vecs : 256;
    if (vecs % t != 0) return false;
    const int v = vecs / t;
    if (v != 1 && v != 2 && v != 4) return false;
    *threads = (unsigned)t;
    *vpt = v;
    return true;
}

}  // namespace ns_rows
