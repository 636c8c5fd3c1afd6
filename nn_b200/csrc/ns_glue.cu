// Row-wise operators of the bf16 / int8 decoder path: int8 row quantisation, LayerNorm with the
// quantisation of the next product's input folded in, token + position embedding, greedy argmax, the
// device-side position counter, and synthetic-input generation for benchmarks.
//
// Reference counterparts: layernorm_fused_f32 (src/NeuralSharp/Backends/Cuda/PtxKernels.Decoding.cs:
// 61-90), gather_f32 (PtxKernels.Advanced.cs:504-523) used by Embedding and PositionalEncoding
// (src/NeuralSharp/Layers/Embedding.cs:38, Layers/Attention.cs:268-269), argmax_f32
// (PtxKernels.Advanced.cs:144-152), affine_f32 on the position counter (Layers/Decoding.cs:121-127).
// The reference runs each of these with one thread per row; here a CTA handles a row.
#include <math.h>

#include "ns_common.cuh"
#include "ns_rows.cuh"

namespace {

constexpr int ROW_THREADS = 256;

__device__ __forceinline__ float warp_max_f(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum_f(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float block_reduce_f(float v, bool is_max, float* red)
{
    v = is_max ? warp_max_f(v) : warp_sum_f(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < ROW_THREADS / 32; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

__device__ __forceinline__ float load_elem(const void* x, int dtype, size_t i)
{
    return dtype == NS_BF16 ? ns_bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(x)[i]) : reinterpret_cast<const float*>(x)[i];
}

__device__ __forceinline__ int8_t quant_one(float v, float scale)
{
    float q = rintf(__fdiv_rn(v, scale));
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return (int8_t)q;
}

// scale[r] = absmax / 127 (1 for an all-zero row); q = clamp(rint(x / scale), -127, 127)
__global__ void __launch_bounds__(ROW_THREADS) ns_quantize_rows_kernel(const void* __restrict__ x, int dtype, int64_t rows, int cols,
                                                                      int8_t* __restrict__ q, float* __restrict__ scale)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    __shared__ float red[ROW_THREADS / 32];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const size_t base = (size_t)r * cols;
        float amax = 0.0f;
        for (int j = threadIdx.x; j < cols; j += ROW_THREADS) amax = fmaxf(amax, fabsf(load_elem(x, dtype, base + j)));
        amax = block_reduce_f(amax, true, red);
        const float s = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
        if (threadIdx.x == 0) scale[r] = s;
        for (int j = threadIdx.x; j < cols; j += ROW_THREADS) q[base + j] = quant_one(load_elem(x, dtype, base + j), s);
    }
}

// LayerNorm of one row per CTA.  Statistics in float, two passes (mean, then centred variance).
// out_dtype NS_F32 / NS_BF16: y = LN(x).  NS_I8: the bf16-rounded LN(x) is quantised per row.
// The normalised row is kept in shared memory (cols floats) between the passes.
__global__ void __launch_bounds__(ROW_THREADS) ns_layernorm_kernel(const void* __restrict__ x, int in_dtype, const float* __restrict__ gamma,
                                                                  const float* __restrict__ beta, int64_t rows, int cols, float eps,
                                                                  int out_dtype, void* __restrict__ y, float* __restrict__ y_scale)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    extern __shared__ float rowbuf[];
    __shared__ float red[ROW_THREADS / 32];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const size_t base = (size_t)r * cols;
        float s = 0.0f;
        for (int j = threadIdx.x; j < cols; j += ROW_THREADS) {
            float v = load_elem(x, in_dtype, base + j);
            rowbuf[j] = v;
            s += v;
        }
        const float mean = block_reduce_f(s, false, red) / (float)cols;
        float v2 = 0.0f;
        for (int j = threadIdx.x; j < cols; j += ROW_THREADS) { float dlt = rowbuf[j] - mean; v2 += dlt * dlt; }
        const float var = block_reduce_f(v2, false, red);
        const float inv = 1.0f / sqrtf(var / (float)cols + eps);
        float amax = 0.0f;
        for (int j = threadIdx.x; j < cols; j += ROW_THREADS) {
            float h = __fadd_rn(__fmul_rn(__fmul_rn(rowbuf[j] - mean, inv), gamma[j]), beta[j]);
            if (out_dtype == NS_F32) {
                reinterpret_cast<float*>(y)[base + j] = h;
            } else {
                uint16_t hb = ns_f32_to_bf16_bits(h);
                if (out_dtype == NS_BF16) reinterpret_cast<uint16_t*>(y)[base + j] = hb;
                else { float hr = ns_bf16_bits_to_f32(hb); rowbuf[j] = hr; amax = fmaxf(amax, fabsf(hr)); }
            }
        }
        if (out_dtype == NS_I8) {
            amax = block_reduce_f(amax, true, red);
            const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
            if (threadIdx.x == 0) y_scale[r] = sc;
            for (int j = threadIdx.x; j < cols; j += ROW_THREADS) reinterpret_cast<int8_t*>(y)[base + j] = quant_one(rowbuf[j], sc);
        }
        __syncthreads();
    }
}

// ---- register-resident rows (cols % 256 == 0, 16-byte aligned): one CTA per row, see ns_rows.cuh
template <int VPT, bool F32IN>
__global__ void ns_quantize_rows_reg_kernel(const void* __restrict__ x, int64_t rows, int cols, int8_t* __restrict__ q, float* __restrict__ scale)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    __shared__ ns_rows::RowShared sh;
    int it = 0;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, it ^= 1) {
        float v[VPT * 8];
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const int col = ns_rows::vec_col(j);
            if (F32IN) {
                const float* row = reinterpret_cast<const float*>(x) + (size_t)r * cols;
                const float4 a = *reinterpret_cast<const float4*>(row + col), b = *reinterpret_cast<const float4*>(row + col + 4);
                v[j * 8] = a.x; v[j * 8 + 1] = a.y; v[j * 8 + 2] = a.z; v[j * 8 + 3] = a.w;
                v[j * 8 + 4] = b.x; v[j * 8 + 5] = b.y; v[j * 8 + 6] = b.z; v[j * 8 + 7] = b.w;
            } else {
                float t[8];
                ns_rows::widen8(*reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + (size_t)r * cols + col), t);
#pragma unroll
                for (int i = 0; i < 8; i++) v[j * 8 + i] = t[i];
            }
        }
        ns_rows::quantize_row<VPT>(v, q + (size_t)r * cols, scale + r, sh.red[it]);   // alternating words: no barrier between rows
    }
}

// LayerNorm of bf16 rows -> bf16 rounding -> int8 rows + scales
template <int VPT>
__global__ void ns_layernorm_q_reg_kernel(const uint16_t* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                          int64_t rows, int cols, float eps, int8_t* __restrict__ y, float* __restrict__ y_scale)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    __shared__ ns_rows::RowShared sh;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float v[VPT * 8];
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            float t[8];
            ns_rows::widen8(*reinterpret_cast<const uint4*>(x + (size_t)r * cols + ns_rows::vec_col(j)), t);
#pragma unroll
            for (int i = 0; i < 8; i++) v[j * 8 + i] = t[i];
        }
        ns_rows::layernorm_quantize_row<VPT>(v, gamma, beta, eps, cols, y + (size_t)r * cols, y_scale + r, sh);
    }
}

inline unsigned grid_rows(const NsDevice* d, int64_t rows);

template <bool F32IN>
cudaError_t launch_quantize_reg(NsDevice* d, unsigned threads, int vpt, const void* x, int64_t rows, int cols, int8_t* q, float* scale)
{
    const dim3 grid(grid_rows(d, rows)), block(threads);
    switch (vpt) {
        case 1: return ns_launch_plain(ns_quantize_rows_reg_kernel<1, F32IN>, grid, block, 0, d->stream, x, rows, cols, q, scale);
        case 2: return ns_launch_plain(ns_quantize_rows_reg_kernel<2, F32IN>, grid, block, 0, d->stream, x, rows, cols, q, scale);
        default: return ns_launch_plain(ns_quantize_rows_reg_kernel<4, F32IN>, grid, block, 0, d->stream, x, rows, cols, q, scale);
    }
}
cudaError_t launch_layernorm_q_reg(NsDevice* d, unsigned threads, int vpt, const uint16_t* x, const float* gamma, const float* beta, int64_t rows,
                                   int cols, float eps, int8_t* y, float* y_scale)
{
    const dim3 grid(grid_rows(d, rows)), block(threads);
    switch (vpt) {
        case 1: return ns_launch_plain(ns_layernorm_q_reg_kernel<1>, grid, block, 0, d->stream, x, gamma, beta, rows, cols, eps, y, y_scale);
        case 2: return ns_launch_plain(ns_layernorm_q_reg_kernel<2>, grid, block, 0, d->stream, x, gamma, beta, rows, cols, eps, y, y_scale);
        default: return ns_launch_plain(ns_layernorm_q_reg_kernel<4>, grid, block, 0, d->stream, x, gamma, beta, rows, cols, eps, y, y_scale);
    }
}

// y[b, i, :] = tok[ids[b, i], :] + pos[p0 + i, :], p0 read from device memory; ids clamped to the table
// as the reference's gather kernel does.
__global__ void ns_embed_pos_kernel(const int32_t* __restrict__ ids, const void* __restrict__ tok, const void* __restrict__ pos, int table_dtype,
                                    const int32_t* __restrict__ pos_dev, int batch, int steps, int dim, int vocab, int max_pos,
                                    int out_dtype, void* __restrict__ y)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    const int p0 = pos_dev ? pos_dev[0] : 0;
    const int64_t n = (int64_t)batch * steps * dim;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        const int dcol = (int)(e % dim);
        const int64_t tokn = e / dim;
        const int i = (int)(tokn % steps);
        int id = ids[tokn];
        id = id < 0 ? 0 : (id > vocab - 1 ? vocab - 1 : id);
        int pp = p0 + i;
        pp = pp > max_pos - 1 ? max_pos - 1 : pp;
        float v = __fadd_rn(load_elem(tok, table_dtype, (size_t)id * dim + dcol), load_elem(pos, table_dtype, (size_t)pp * dim + dcol));
        if (out_dtype == NS_F32) reinterpret_cast<float*>(y)[e] = v;
        else reinterpret_cast<uint16_t*>(y)[e] = ns_f32_to_bf16_bits(v);
    }
}

// First maximum per row -> int32 id.  One CTA per row.
__global__ void __launch_bounds__(ROW_THREADS) ns_argmax_i32_kernel(const float* __restrict__ x, int rows, int cols, int64_t row_stride,
                                                                    int32_t* __restrict__ ids)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    __shared__ float bv[ROW_THREADS / 32];
    __shared__ int bi[ROW_THREADS / 32];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xs = x + (size_t)r * row_stride;
        float best = -INFINITY;
        int idx = 0x7fffffff;
        if ((cols & 3) == 0 && (reinterpret_cast<uintptr_t>(xs) & 15) == 0) {
            // 16-byte loads, four in flight; a thread meets its indices in increasing order, so "strictly greater" keeps the
            // first maximum
            const float4* x4 = reinterpret_cast<const float4*>(xs);
            const int n4 = cols >> 2;
            for (int j0 = threadIdx.x; j0 < n4; j0 += 4 * ROW_THREADS) {
                float4 t[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = j0 + u * ROW_THREADS;
                    t[u] = j < n4 ? x4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = (j0 + u * ROW_THREADS) * 4;
                    if (j < cols) {
                        const float v[4] = {t[u].x, t[u].y, t[u].z, t[u].w};
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            if (idx == 0x7fffffff || v[e] > best) { best = v[e]; idx = j + e; }
                    }
                }
            }
        } else {
            for (int j = threadIdx.x; j < cols; j += ROW_THREADS) {
                float v = xs[j];
                if (idx == 0x7fffffff || v > best) { best = v; idx = j; }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
        }
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();
        if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float b = bv[0];
            int i0 = bi[0];
            for (int w = 1; w < ROW_THREADS / 32; w++)
                if (bi[w] != 0x7fffffff && (i0 == 0x7fffffff || bv[w] > b || (bv[w] == b && bi[w] < i0))) { b = bv[w]; i0 = bi[w]; }
            ids[r] = i0 == 0x7fffffff ? 0 : i0;
        }
    }
}

__global__ void ns_add_i32_kernel(int32_t* p, int32_t delta)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    p[0] += delta;
}

__global__ void ns_convert_kernel(const void* __restrict__ x, int in_dtype, void* __restrict__ y, int out_dtype, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = load_elem(x, in_dtype, i);
        if (out_dtype == NS_F32) reinterpret_cast<float*>(y)[i] = v;
        else reinterpret_cast<uint16_t*>(y)[i] = ns_f32_to_bf16_bits(v);
    }
}

// Synthetic inputs for benchmarks: counter-based hash -> uniform -> Box-Muller (the construction the
// reference uses in CounterRandom, src/NeuralSharp/Backends/Backend.cs:285-298, and Tensor.Normal,
// src/NeuralSharp/Tensor.cs:148-165).  Element i depends only on (seed, i).
__device__ __forceinline__ uint32_t mix32(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
    return h;
}
__device__ __forceinline__ uint32_t hash2(uint32_t seed, uint64_t index, uint32_t lane)
{
    uint32_t lo = (uint32_t)index, hi = (uint32_t)(index >> 32);
    uint32_t h = mix32(seed * 0x9E3779B9u + 0x7F4A7C15u + lane);
    h = mix32(h ^ (lo * 0x85EBCA6Bu));
    h = mix32(h ^ (hi * 0xC2B2AE35u) ^ 0x27D4EB2Fu);
    return h;
}
__global__ void ns_fill_normal_kernel(void* __restrict__ y, int dtype, int64_t n, uint32_t seed, float mean, float std)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float u1 = 1.0f - (float)(hash2(seed, (uint64_t)i, 0) >> 8) * (1.0f / 16777216.0f);
        float u2 = (float)(hash2(seed, (uint64_t)i, 1) >> 8) * (1.0f / 16777216.0f);
        float v = mean + std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        if (dtype == NS_F32) reinterpret_cast<float*>(y)[i] = v;
        else if (dtype == NS_BF16) reinterpret_cast<uint16_t*>(y)[i] = ns_f32_to_bf16_bits(v);
        else reinterpret_cast<int8_t*>(y)[i] = (int8_t)fminf(fmaxf(rintf(v), -127.0f), 127.0f);
    }
}
__global__ void ns_fill_ids_kernel(int32_t* __restrict__ y, int64_t n, uint32_t seed, uint32_t bound)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = (int32_t)(hash2(seed, (uint64_t)i, 2) % bound);
}

inline unsigned grid_rows(const NsDevice* d, int64_t rows)
{
    int64_t cap = (int64_t)d->sm_count * 8;
    return (unsigned)(rows < cap ? (rows < 1 ? 1 : rows) : cap);
}
inline unsigned grid_elems(const NsDevice* d, int64_t n, int threads)
{
    int64_t blocks = (n + threads - 1) / threads;
    int64_t cap = (int64_t)d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

#define NS_ENTER(h)                          \
    NsDevice* d = ns_dev(h);                 \
    {                                        \
        int _rc = ns_device_make_current(d); \
        if (_rc != NS_OK) return _rc;        \
    }

extern "C" int ns_quantize_rows_i8(ns_device_t h, uint64_t x, int in_dtype, int64_t rows, int cols, uint64_t q, uint64_t scale)
{
    NS_ENTER(h);
    NS_REQUIRE(x && q && scale, NS_ERR_ARGUMENT, "ns_quantize_rows_i8: null operand");
    NS_REQUIRE(in_dtype == NS_F32 || in_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_quantize_rows_i8: input must be NS_F32 or NS_BF16");
    NS_REQUIRE(rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_quantize_rows_i8: bad shape");
    if (rows == 0) return NS_OK;
    unsigned threads = 0;
    int vpt = 0;
    if (in_dtype == NS_BF16 && ((x | q) & 15) == 0 && ns_rows_stream_fits(false, rows, cols)) {
        NS_CUDA(ns_rows_stream_quantize(d, reinterpret_cast<const uint16_t*>(x), rows, cols, reinterpret_cast<int8_t*>(q), reinterpret_cast<float*>(scale)));
        return NS_OK;
    }
    if (((x | q) & 15) == 0 && ns_rows::row_shape(cols, &threads, &vpt)) {
        if (in_dtype == NS_F32)
            NS_CUDA(launch_quantize_reg<true>(d, threads, vpt, reinterpret_cast<const void*>(x), rows, cols, reinterpret_cast<int8_t*>(q), reinterpret_cast<float*>(scale)));
        else
            NS_CUDA(launch_quantize_reg<false>(d, threads, vpt, reinterpret_cast<const void*>(x), rows, cols, reinterpret_cast<int8_t*>(q), reinterpret_cast<float*>(scale)));
        return NS_OK;
    }
    ns_launch_plain(ns_quantize_rows_kernel, dim3(grid_rows(d, rows)), dim3(ROW_THREADS), 0, d->stream, reinterpret_cast<const void*>(x), in_dtype, rows, cols,
                                                                              reinterpret_cast<int8_t*>(q), reinterpret_cast<float*>(scale));
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_layernorm(ns_device_t h, uint64_t x, int in_dtype, uint64_t gamma, uint64_t beta, int64_t rows, int cols, float eps,
                            int out_dtype, uint64_t y, uint64_t y_scale)
{
    NS_ENTER(h);
    NS_REQUIRE(x && gamma && beta && y, NS_ERR_ARGUMENT, "ns_layernorm: null operand");
    NS_REQUIRE(in_dtype == NS_F32 || in_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_layernorm: input must be NS_F32 or NS_BF16");
    NS_REQUIRE(out_dtype == NS_F32 || out_dtype == NS_BF16 || out_dtype == NS_I8, NS_ERR_ARGUMENT, "ns_layernorm: bad output dtype");
    NS_REQUIRE(out_dtype != NS_I8 || y_scale != 0, NS_ERR_ARGUMENT, "ns_layernorm: int8 output needs a scale buffer");
    NS_REQUIRE(rows >= 0 && cols > 0 && cols <= 16384, NS_ERR_ARGUMENT, "ns_layernorm: cols must be in [1, 16384]");
    if (rows == 0) return NS_OK;
    unsigned threads = 0;
    int vpt = 0;
    if (in_dtype == NS_BF16 && out_dtype == NS_I8 && ((x | y | gamma | beta) & 15) == 0 && ns_rows_stream_fits(true, rows, cols)) {
        NS_CUDA(ns_rows_stream_layernorm(d, reinterpret_cast<const uint16_t*>(x), reinterpret_cast<const float*>(gamma), reinterpret_cast<const float*>(beta), rows,
                                         cols, eps, reinterpret_cast<int8_t*>(y), reinterpret_cast<float*>(y_scale)));
        return NS_OK;
    }
    if (in_dtype == NS_BF16 && out_dtype == NS_I8 && ((x | y | gamma | beta) & 15) == 0 && ns_rows::row_shape(cols, &threads, &vpt)) {
        // the decoder's case: the row lives in the registers of its CTA
        NS_CUDA(launch_layernorm_q_reg(d, threads, vpt, reinterpret_cast<const uint16_t*>(x), reinterpret_cast<const float*>(gamma),
                                       reinterpret_cast<const float*>(beta), rows, cols, eps, reinterpret_cast<int8_t*>(y), reinterpret_cast<float*>(y_scale)));
        return NS_OK;
    }
    size_t smem = (size_t)cols * sizeof(float);
    static bool configured[64] = {false};
    if (smem > 48 * 1024 && !configured[d->ordinal]) {
        NS_CUDA(cudaFuncSetAttribute(ns_layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4));
        configured[d->ordinal] = true;
    }
    ns_launch_plain(ns_layernorm_kernel, dim3(grid_rows(d, rows)), dim3(ROW_THREADS), smem, d->stream, reinterpret_cast<const void*>(x), in_dtype,
                                                                             reinterpret_cast<const float*>(gamma), reinterpret_cast<const float*>(beta),
                                                                             rows, cols, eps, out_dtype, reinterpret_cast<void*>(y),
                                                                             reinterpret_cast<float*>(y_scale));
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_embed_pos(ns_device_t h, uint64_t ids, uint64_t tok_table, uint64_t pos_table, int table_dtype, uint64_t pos_dev,
                            int batch, int steps, int dim, int vocab, int max_pos, int out_dtype, uint64_t y)
{
    NS_ENTER(h);
    NS_REQUIRE(ids && tok_table && pos_table && y, NS_ERR_ARGUMENT, "ns_embed_pos: null operand");
    NS_REQUIRE(table_dtype == NS_F32 || table_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_embed_pos: tables must be NS_F32 or NS_BF16");
    NS_REQUIRE(out_dtype == NS_F32 || out_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_embed_pos: output must be NS_F32 or NS_BF16");
    NS_REQUIRE(batch >= 0 && steps >= 0 && dim > 0 && vocab > 0 && max_pos > 0, NS_ERR_ARGUMENT, "ns_embed_pos: bad shape");
    int64_t n = (int64_t)batch * steps * dim;
    if (n == 0) return NS_OK;
    ns_launch_plain(ns_embed_pos_kernel, dim3(grid_elems(d, n, 256)), dim3(256), 0, d->stream, reinterpret_cast<const int32_t*>(ids), reinterpret_cast<const void*>(tok_table),
                                                                     reinterpret_cast<const void*>(pos_table), table_dtype,
                                                                     reinterpret_cast<const int32_t*>(pos_dev), batch, steps, dim, vocab, max_pos,
                                                                     out_dtype, reinterpret_cast<void*>(y));
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_argmax_i32(ns_device_t h, uint64_t x, int rows, int cols, int64_t row_stride, uint64_t ids)
{
    NS_ENTER(h);
    NS_REQUIRE(x && ids && rows >= 0 && cols > 0 && row_stride >= cols, NS_ERR_ARGUMENT, "ns_argmax_i32: bad argument");
    if (rows == 0) return NS_OK;
    ns_launch_plain(ns_argmax_i32_kernel, dim3(grid_rows(d, rows)), dim3(ROW_THREADS), 0, d->stream, reinterpret_cast<const float*>(x), rows, cols, row_stride,
                                                                           reinterpret_cast<int32_t*>(ids));
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_add_i32(ns_device_t h, uint64_t counter, int32_t delta)
{
    NS_ENTER(h);
    NS_REQUIRE(counter != 0, NS_ERR_ARGUMENT, "ns_add_i32: null counter");
    ns_launch_plain(ns_add_i32_kernel, dim3(1), dim3(1), 0, d->stream, reinterpret_cast<int32_t*>(counter), delta);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_convert(ns_device_t h, uint64_t x, int in_dtype, uint64_t y, int out_dtype, int64_t n)
{
    NS_ENTER(h);
    NS_REQUIRE(x && y && n >= 0, NS_ERR_ARGUMENT, "ns_convert: bad argument");
    NS_REQUIRE((in_dtype == NS_F32 || in_dtype == NS_BF16) && (out_dtype == NS_F32 || out_dtype == NS_BF16), NS_ERR_ARGUMENT,
               "ns_convert: dtypes must be NS_F32 or NS_BF16");
    if (n == 0) return NS_OK;
    ns_convert_kernel<<<grid_elems(d, n, 256), 256, 0, d->stream>>>(reinterpret_cast<const void*>(x), in_dtype, reinterpret_cast<void*>(y), out_dtype, n);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_fill_normal(ns_device_t h, uint64_t y, int dtype, int64_t n, uint32_t seed, float mean, float std)
{
    NS_ENTER(h);
    NS_REQUIRE(y && n >= 0, NS_ERR_ARGUMENT, "ns_fill_normal: bad argument");
    NS_REQUIRE(dtype == NS_F32 || dtype == NS_BF16 || dtype == NS_I8, NS_ERR_ARGUMENT, "ns_fill_normal: dtype must be NS_F32, NS_BF16 or NS_I8");
    if (n == 0) return NS_OK;
    ns_fill_normal_kernel<<<grid_elems(d, n, 256), 256, 0, d->stream>>>(reinterpret_cast<void*>(y), dtype, n, seed, mean, std);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_fill_ids(ns_device_t h, uint64_t y, int64_t n, uint32_t seed, uint32_t bound)
{
    NS_ENTER(h);
    NS_REQUIRE(y && n >= 0 && bound > 0, NS_ERR_ARGUMENT, "ns_fill_ids: bad argument");
    if (n == 0) return NS_OK;
    ns_fill_ids_kernel<<<grid_elems(d, n, 256), 256, 0, d->stream>>>(reinterpret_cast<int32_t*>(y), n, seed, bound);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

// ------------------------------------------------------------------------------------------------
// Tensor-parallel helpers: what follows the reduction of row-shard partial sums, and the greedy
// token choice over a vocabulary split across ranks.
// ------------------------------------------------------------------------------------------------
namespace {

// y = (partial + bias[col]) + residual, the order of the fused epilogue
__global__ void ns_bias_residual_kernel(const float* __restrict__ partial, const float* __restrict__ bias, const void* __restrict__ residual,
                                        int residual_dtype, int64_t n, int cols, int out_dtype, void* __restrict__ y)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = partial[i];
        if (bias) v = __fadd_rn(v, bias[i % cols]);
        if (residual) v = __fadd_rn(v, load_elem(residual, residual_dtype, i));
        if (out_dtype == NS_F32) reinterpret_cast<float*>(y)[i] = v;
        else reinterpret_cast<uint16_t*>(y)[i] = ns_f32_to_bf16_bits(v);
    }
}

// per row: first maximum of this rank's column slice -> (value, global column index)
__global__ void __launch_bounds__(ROW_THREADS) ns_argmax_partial_kernel(const float* __restrict__ x, int rows, int cols, int64_t row_stride,
                                                                        int col_offset, float* __restrict__ out_val, int32_t* __restrict__ out_idx)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    __shared__ float bv[ROW_THREADS / 32];
    __shared__ int bi[ROW_THREADS / 32];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xs = x + (size_t)r * row_stride;
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int j = threadIdx.x; j < cols; j += ROW_THREADS) {
            float v = xs[j];
            if (idx == 0x7fffffff || v > best) { best = v; idx = j; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
        }
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();
        if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float b = bv[0];
            int i0 = bi[0];
            for (int w = 1; w < ROW_THREADS / 32; w++)
                if (bi[w] != 0x7fffffff && (i0 == 0x7fffffff || bv[w] > b || (bv[w] == b && bi[w] < i0))) { b = bv[w]; i0 = bi[w]; }
            out_val[r] = b;
            out_idx[r] = (i0 == 0x7fffffff ? 0 : i0) + col_offset;
        }
    }
}

// vals / idx: [parts, rows]; the largest value wins, ties go to the smallest column index
__global__ void ns_argmax_merge_kernel(const float* __restrict__ vals, const int32_t* __restrict__ idx, int parts, int rows, int32_t* __restrict__ ids)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float b = vals[r];
    int bi = idx[r];
    for (int pidx = 1; pidx < parts; pidx++) {
        const float v = vals[(size_t)pidx * rows + r];
        const int i = idx[(size_t)pidx * rows + r];
        if (v > b || (v == b && i < bi)) { b = v; bi = i; }
    }
    ids[r] = bi;
}

}  // namespace

extern "C" int ns_bias_residual(ns_device_t h, uint64_t partial, uint64_t bias, uint64_t residual, int residual_dtype, int64_t rows, int cols,
                                int out_dtype, uint64_t y)
{
    NS_ENTER(h);
    NS_REQUIRE(partial && y && rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_bias_residual: bad argument");
    NS_REQUIRE(out_dtype == NS_F32 || out_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_bias_residual: output must be NS_F32 or NS_BF16");
    const int64_t n = rows * cols;
    if (n == 0) return NS_OK;
    ns_launch_plain(ns_bias_residual_kernel, dim3(grid_elems(d, n, 256)), dim3(256), 0, d->stream, reinterpret_cast<const float*>(partial), reinterpret_cast<const float*>(bias),
                                                                         reinterpret_cast<const void*>(residual), residual_dtype, n, cols, out_dtype,
                                                                         reinterpret_cast<void*>(y));
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_argmax_partial(ns_device_t h, uint64_t x, int rows, int cols, int64_t row_stride, int col_offset, uint64_t out_val, uint64_t out_idx)
{
    NS_ENTER(h);
    NS_REQUIRE(x && out_val && out_idx && rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_argmax_partial: bad argument");
    if (rows == 0) return NS_OK;
    ns_launch_plain(ns_argmax_partial_kernel, dim3(grid_rows(d, rows)), dim3(ROW_THREADS), 0, d->stream, reinterpret_cast<const float*>(x), rows, cols, row_stride, col_offset,
                                                                               reinterpret_cast<float*>(out_val), reinterpret_cast<int32_t*>(out_idx));
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_argmax_merge(ns_device_t h, uint64_t vals, uint64_t idx, int parts, int rows, uint64_t ids)
{
    NS_ENTER(h);
    NS_REQUIRE(vals && idx && ids && parts >= 1 && rows >= 0, NS_ERR_ARGUMENT, "ns_argmax_merge: bad argument");
    if (rows == 0) return NS_OK;
    ns_launch_plain(ns_argmax_merge_kernel, dim3((rows + 127) / 128), dim3(128), 0, d->stream, reinterpret_cast<const float*>(vals), reinterpret_cast<const int32_t*>(idx), parts,
                                                                     rows, reinterpret_cast<int32_t*>(ids));
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}
