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

constexpr int MAX_VPT = 4;

struct RowShared {
    float red[3][MAX_VPT * MAX_WARPS];   // one set of partials (a word per 32-vector piece of the row) per reduction of a row pass
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

// A SUM over the row in the library's one order, whichever kernel takes it: vector by vector (part[j]: the eight elements of
// this thread's vector j, left to right), the 32 vectors of a piece (a warp's vectors j) by the xor-shuffle tree, the pieces
// one after the other in the order of their columns (piece j * warps + warp).  The many-row kernels (ns_rows_stream.cu) and the
// second phase of the product kernel (ns_tail.cuh) sum in the same order, so LayerNorm gives the same bits in all of them.
template <int VPT>
__device__ __forceinline__ float block_sum_pieces(const float (&part)[VPT], float* red)
{
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5;
    float t[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        float v = part[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        t[j] = v;
    }
    if (VPT == 1 && warps == 1) return t[0];
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int j = 0; j < VPT; j++) red[j * warps + warp] = t[j];
    }
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < VPT * warps; w++) r += red[w];
    return r;
}

__device__ __forceinline__ int8_t quant_one(float v, float scale)
{
    float q = rintf(__fdiv_rn(v, scale));
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return (int8_t)q;
}

// Eight values -> eight int8 bytes (lo: values 0-3, hi: 4-7), bit for bit what quant_one gives, without eight IEEE
// divisions.  Precondition: rcp = __frcp_rn(scale), scale = (row maximum) / 127.
// With u = 2^-15 (a float's ulp in [256, 512)): s_hi = x * rcp + 384.5 + 4u and s_lo = x * rcp + 384.5 - 4u, one fused
// rounding each.  x * rcp is within 0.25u of the real quotient (|quotient| <= 127.0001), the rounded quotient d the rule
// asks for within 0.125u, a fused rounding adds 0.5u: d + 384.5 lies in [s_lo + 3u, s_hi - 3u].  So when no integer lies in
// (s_lo, s_hi] -- the two floors agree -- d + 0.5 is no integer either and floor(s_hi) - 384 is d rounded to nearest,
// ties included (there is none).  The floors come from an add of 2^23 rounded toward zero, which leaves floor(s) in the low
// mantissa bits; its low byte is 128 + n, n with its top bit flipped (undone on the packed bytes).  Vectors whose floors
// differ somewhere (the quotient within 5u of a half-integer: one value in 4000) take the divisions; with FINITE_CHECK so do
// vectors with a NaN, an infinity or a quotient beyond +-127 in play (the high bits of the floor are then not those of
// 2^23 + 256..511) -- a caller that has ruled those out for the whole row saves that test.
template <bool FINITE_CHECK>
__device__ __forceinline__ void quant8(const float* x, float scale, float rcp, uint32_t& lo, uint32_t& hi)
{
    constexpr float U = 1.0f / 32768.0f, OFFSET_HI = 384.5f + 4.0f * U, OFFSET_LO = 384.5f - 4.0f * U, TWO23 = 8388608.0f;
    uint32_t b[8], differ = 0u, range = 0u;
#pragma unroll
    for (int t = 0; t < 8; t++) {
        const uint32_t n_hi = __float_as_uint(__fadd_rz(fmaf(x[t], rcp, OFFSET_HI), TWO23));
        const uint32_t n_lo = __float_as_uint(__fadd_rz(fmaf(x[t], rcp, OFFSET_LO), TWO23));
        differ |= n_hi ^ n_lo;
        if (FINITE_CHECK) range |= n_hi ^ 0x4B000100u;
        b[t] = n_hi;
    }
    if (differ != 0u || (range & 0xFFFFFF00u) != 0u) {
#pragma unroll
        for (int t = 0; t < 8; t++) b[t] = (uint32_t)(uint8_t)quant_one(x[t], scale) ^ 0x80u;
    }
    lo = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410) ^ 0x80808080u;
    hi = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410) ^ 0x80808080u;
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
    const float rcp = __frcp_rn(sc);
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        uint32_t lo, hi;
        quant8<true>(x + j * 8, sc, rcp, lo, hi);
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
    float part[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) s += x[j * 8 + i];
        part[j] = s;
    }
    const float mean = block_sum_pieces<VPT>(part, sh.red[0]) / (float)cols;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        float v2 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) { const float d = x[j * 8 + i] - mean; v2 = fmaf(d, d, v2); }
        part[j] = v2;
    }
    const float inv = 1.0f / sqrtf(block_sum_pieces<VPT>(part, sh.red[1]) / (float)cols + eps);
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

__device__ __forceinline__ float warp_reduce(float v, bool is_max)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    return v;
}

// Rows at and above this count take the many-row kernels of ns_rows_stream.cu.
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

// Many bf16 rows at once through rings of row buffers in shared memory (ns_rows_stream.cu).
bool ns_rows_stream_fits(bool layernorm, int64_t rows, int cols);
cudaError_t ns_rows_stream_quantize(NsDevice* d, const uint16_t* x, int64_t rows, int cols, int8_t* q, float* scale);
cudaError_t ns_rows_stream_layernorm(NsDevice* d, const uint16_t* x, const float* gamma, const float* beta, int64_t rows, int cols, float eps, int8_t* q,
                                     float* scale);
