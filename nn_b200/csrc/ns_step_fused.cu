// Row kernels of the decoding step that take over a product's epilogue.
//
// With the few rows of a decoding step the cost of a step is the NUMBER of kernels (each launch costs about 5 us before
// its first useful byte), not their size.  A product whose K is split already needs a second kernel to add the partial
// sums; these kernels are that second kernel AND the row operator the reference runs next, in one launch:
//   ns_finish_norm_quant   partial sums -> dequantise + bias + residual -> bf16 residual stream -> LayerNorm -> bf16 ->
//                          int8 row quantisation (the next product's input).  Reference sequence: matmul_f32, add_rowvec_f32,
//                          add_f32 (x + Linear(...), src/NeuralSharp/Layers/Attention.cs:201-205), layernorm_fused_f32
//                          (Backends/Cuda/PtxKernels.Decoding.cs:61-90): four kernels.
//   ns_finish_kv_append    partial sums of the fused QKV product -> dequantise + bias -> bf16 [rows, 3 d] -> K and V thirds
//                          appended to the paged cache.  Reference: matmul_f32, add_rowvec_f32, three narrow + permute
//                          copies, kv_write_f32 twice (Layers/Attention.cs:98-118, PtxKernels.Decoding.cs:130-143).
// The arithmetic is the product epilogue's, operation for operation (ns_gemm_tc.cu: int -> float, * a_scale, * w_scale,
// + bias, + residual, each rounded to float; bf16 round to nearest even), followed by ns_layernorm's / ns_kv_append's, so
// results are bit-identical to the unfused sequence.
#include <math.h>

#include "ns_gemm.cuh"
#include "ns_rows.cuh"

struct NsKvCacheView {
    uint16_t* k_pool;
    uint16_t* v_pool;
    int page_size, heads, head_dim, num_pages;
};
int ns_kv_cache_view(ns_kv_cache_t cache, NsKvCacheView* out);   // ns_attention_decode.cu

namespace {

constexpr int FUSED_THREADS = 256;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < FUSED_THREADS / 32; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

__device__ __forceinline__ int8_t quant_one(float v, float scale)
{
    float q = rintf(__fdiv_rn(v, scale));
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return (int8_t)q;
}

// exact sum of the splits' accumulators of element (row, col)
__device__ __forceinline__ int32_t sum_splits(const int32_t* __restrict__ partial, int splits, size_t slab, size_t idx)
{
    int32_t s = 0;
    for (int sp = 0; sp < splits; sp++) s += partial[(size_t)sp * slab + idx];
    return s;
}

struct FinishNormParams {
    const int32_t* partial;
    int splits;
    const float* x_scale;     // per row, of the product's int8 input
    const float* w_scale;     // per column
    const float* bias;        // per column or null
    const uint16_t* residual; // bf16 [rows, cols] or null
    int64_t rows;
    int cols;
    uint16_t* x_out;          // bf16 [rows, cols]
    const float* gamma;       // null: no LayerNorm / quantisation
    const float* beta;
    float eps;
    int8_t* q;
    float* q_scale;
};

// One CTA per row; the row stays in shared memory between the passes, as in ns_layernorm_kernel.
__global__ void __launch_bounds__(FUSED_THREADS) ns_finish_norm_quant_kernel(const FinishNormParams p)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    extern __shared__ float rowbuf[];
    __shared__ float red[FUSED_THREADS / 32];
    const size_t slab = (size_t)p.rows * p.cols;
    for (int64_t r = blockIdx.x; r < p.rows; r += gridDim.x) {
        const size_t base = (size_t)r * p.cols;
        const float a_scale = p.x_scale[r];
        float s = 0.0f;
        for (int j = threadIdx.x; j < p.cols; j += FUSED_THREADS) {
            float v = __int2float_rn(sum_splits(p.partial, p.splits, slab, base + j));
            v = __fmul_rn(v, a_scale);
            v = __fmul_rn(v, p.w_scale[j]);
            if (p.bias != nullptr) v = __fadd_rn(v, p.bias[j]);
            if (p.residual != nullptr) v = __fadd_rn(v, ns_bf16_bits_to_f32(p.residual[base + j]));
            const uint16_t xb = ns_f32_to_bf16_bits(v);
            p.x_out[base + j] = xb;
            const float xr = ns_bf16_bits_to_f32(xb);
            rowbuf[j] = xr;
            s += xr;
        }
        if (p.gamma == nullptr) continue;   // same for every thread of the grid
        const float mean = block_reduce(s, false, red) / (float)p.cols;
        float v2 = 0.0f;
        for (int j = threadIdx.x; j < p.cols; j += FUSED_THREADS) { const float dlt = rowbuf[j] - mean; v2 += dlt * dlt; }
        const float var = block_reduce(v2, false, red);
        const float inv = 1.0f / sqrtf(var / (float)p.cols + p.eps);
        float amax = 0.0f;
        for (int j = threadIdx.x; j < p.cols; j += FUSED_THREADS) {
            const float h = __fadd_rn(__fmul_rn(__fmul_rn(rowbuf[j] - mean, inv), p.gamma[j]), p.beta[j]);
            const float hr = ns_bf16_bits_to_f32(ns_f32_to_bf16_bits(h));
            rowbuf[j] = hr;
            amax = fmaxf(amax, fabsf(hr));
        }
        amax = block_reduce(amax, true, red);
        const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
        __syncthreads();   // every thread has read x_scale[r] (it may be the same array as q_scale)
        if (threadIdx.x == 0) p.q_scale[r] = sc;
        for (int j = threadIdx.x; j < p.cols; j += FUSED_THREADS) p.q[base + j] = quant_one(rowbuf[j], sc);
        __syncthreads();
    }
}

// The same with the row in the registers of its CTA (cols % 256 == 0, at most 4 vectors per thread; see ns_rows.cuh).
template <int VPT>
__global__ void ns_finish_norm_quant_reg_kernel(const FinishNormParams p)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    __shared__ ns_rows::RowShared sh;
    const size_t slab = (size_t)p.rows * p.cols;
    for (int64_t r = blockIdx.x; r < p.rows; r += gridDim.x) {
        const float a_scale = p.x_scale[r];
        float v[VPT * 8];
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const int col = ns_rows::vec_col(j);
            const size_t idx = (size_t)r * p.cols + col;
            int32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int sp = 0; sp < p.splits; sp++) {
                const int4* src = reinterpret_cast<const int4*>(p.partial + (size_t)sp * slab + idx);
                const int4 a = src[0], b = src[1];
                acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
            }
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.w_scale + col)), w1 = __ldg(reinterpret_cast<const float4*>(p.w_scale + col + 4));
            const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float t[8];
#pragma unroll
            for (int i = 0; i < 8; i++) t[i] = __fmul_rn(__fmul_rn(__int2float_rn(acc[i]), a_scale), ws[i]);
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
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) w[i] = uint32_t(ns_f32_to_bf16_bits(t[2 * i])) | (uint32_t(ns_f32_to_bf16_bits(t[2 * i + 1])) << 16);
            const uint4 packed = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(p.x_out + idx) = packed;
            float xr[8];
            ns_rows::widen8(packed, xr);
#pragma unroll
            for (int i = 0; i < 8; i++) v[j * 8 + i] = xr[i];
        }
        // every thread has read x_scale[r] before the barriers of the reductions below, so q_scale may be the same array
        if (p.gamma != nullptr) ns_rows::layernorm_quantize_row<VPT>(v, p.gamma, p.beta, p.eps, p.cols, p.q + (size_t)r * p.cols, p.q_scale + r, sh);
    }
}

// Sum of the splits + dequantisation + bias + GELU, rounded to bf16 (what the product's own epilogue would have stored), then
// the int8 row quantisation of that: the input of FF2 straight from FF1's partial sums.  One CTA per row, the row in registers.
struct FinishGeluParams {
    const int32_t* partial;
    int splits;
    const float* x_scale;
    const float* w_scale;
    const float* bias;
    int64_t rows;
    int cols;
    int8_t* q;
    float* q_scale;
};

template <int VPT>
__global__ void ns_finish_gelu_quant_kernel(const FinishGeluParams p)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    __shared__ ns_rows::RowShared sh;
    const size_t slab = (size_t)p.rows * p.cols;
    int it = 0;
    for (int64_t r = blockIdx.x; r < p.rows; r += gridDim.x, it ^= 1) {
        const float a_scale = p.x_scale[r];
        float v[VPT * 8];
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const int col = ns_rows::vec_col(j);
            const size_t idx = (size_t)r * p.cols + col;
            int32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int sp = 0; sp < p.splits; sp++) {
                const int4* src = reinterpret_cast<const int4*>(p.partial + (size_t)sp * slab + idx);
                const int4 a = src[0], b = src[1];
                acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
            }
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.w_scale + col)), w1 = __ldg(reinterpret_cast<const float4*>(p.w_scale + col + 4));
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + col)), b1 = __ldg(reinterpret_cast<const float4*>(p.bias + col + 4));
            const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float t = ns_gelu_fast(__fadd_rn(__fmul_rn(__fmul_rn(__int2float_rn(acc[i]), a_scale), ws[i]), bs[i]));
                v[j * 8 + i] = ns_bf16_bits_to_f32(ns_f32_to_bf16_bits(t));
            }
        }
        // (x_scale[r] has been read by every thread before the barrier of the reduction: q_scale may be the same array)
        ns_rows::quantize_row<VPT>(v, p.q + (size_t)r * p.cols, p.q_scale + r, sh.red[it]);
    }
}

cudaError_t launch_finish_reg(NsDevice* d, unsigned threads, int vpt, const FinishNormParams& p)
{
    const int64_t cap = (int64_t)d->sm_count * 8;
    const dim3 grid((unsigned)(p.rows < cap ? p.rows : cap)), block(threads);
    switch (vpt) {
        case 1: return ns_launch_plain(ns_finish_norm_quant_reg_kernel<1>, grid, block, 0, d->stream, p);
        case 2: return ns_launch_plain(ns_finish_norm_quant_reg_kernel<2>, grid, block, 0, d->stream, p);
        default: return ns_launch_plain(ns_finish_norm_quant_reg_kernel<4>, grid, block, 0, d->stream, p);
    }
}

struct FinishKvParams {
    const int32_t* partial;
    int splits;
    const float* x_scale;
    const float* w_scale;
    const float* bias;
    int batch, steps;
    int d_loc;                // columns of each of the Q, K, V thirds
    uint16_t* qkv;            // bf16 [batch * steps, 3 * d_loc]
    uint16_t* k_pool;
    uint16_t* v_pool;
    const int32_t* page_table;
    int max_pages, page_size, heads, dh, num_pages;
    const int32_t* pos_dev;
    int* status;
};

// One thread per 8 consecutive columns of a row.
__global__ void ns_finish_kv_append_kernel(const FinishKvParams p)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    const int cols = 3 * p.d_loc;
    const int groups = cols / 8;
    const int64_t rows = (int64_t)p.batch * p.steps;
    const size_t slab = (size_t)rows * cols;
    const int pos0 = p.pos_dev[0];
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < rows * groups; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = e / groups;
        const int col0 = (int)(e % groups) * 8;
        const size_t idx0 = (size_t)row * cols + col0;
        const float a_scale = p.x_scale[row];
        int32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int sp = 0; sp < p.splits; sp++) {
            const int4* src = reinterpret_cast<const int4*>(p.partial + (size_t)sp * slab + idx0);
            const int4 a = src[0], b = src[1];
            acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
            acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float v0 = __fmul_rn(__fmul_rn(__int2float_rn(acc[2 * j]), a_scale), p.w_scale[col0 + 2 * j]);
            float v1 = __fmul_rn(__fmul_rn(__int2float_rn(acc[2 * j + 1]), a_scale), p.w_scale[col0 + 2 * j + 1]);
            if (p.bias != nullptr) { v0 = __fadd_rn(v0, p.bias[col0 + 2 * j]); v1 = __fadd_rn(v1, p.bias[col0 + 2 * j + 1]); }
            w[j] = uint32_t(ns_f32_to_bf16_bits(v0)) | (uint32_t(ns_f32_to_bf16_bits(v1)) << 16);
        }
        const uint4 out = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(p.qkv + idx0) = out;
        const int third = col0 / p.d_loc;          // 0 = Q, 1 = K, 2 = V
        if (third == 0) continue;
        const int in_third = col0 - third * p.d_loc;
        const int h = in_third / p.dh, c = in_third % p.dh;
        const int i = (int)(row % p.steps), b = (int)(row / p.steps);
        const int pos = pos0 + i;
        // an append outside the cache is skipped and reported (code 500), as in ns_kv_append
        if (pos < 0 || pos / p.page_size >= p.max_pages) { *reinterpret_cast<volatile int*>(p.status) = 500; continue; }
        const int page = p.page_table[(size_t)b * p.max_pages + pos / p.page_size];
        if (page < 0 || page >= p.num_pages) { *reinterpret_cast<volatile int*>(p.status) = 500; continue; }
        const size_t dst = (((size_t)page * p.heads + h) * p.page_size + pos % p.page_size) * p.dh + c;
        *reinterpret_cast<uint4*>((third == 1 ? p.k_pool : p.v_pool) + dst) = out;
    }
}

}  // namespace

extern "C" int ns_finish_norm_quant(ns_device_t h, uint64_t partial, int splits, ns_linear_t linear, uint64_t x_scale, uint64_t residual,
                                    int64_t rows, uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q, uint64_t q_scale)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    int n_loc = 0, mode = 0;
    uint64_t w_scale = 0, bias = 0;
    rc = ns_linear_info(linear, nullptr, &n_loc, &mode, nullptr, &w_scale, &bias);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(mode == NS_I8 && w_scale != 0, NS_ERR_ARGUMENT, "ns_finish_norm_quant: the layer must be an int8 layer");
    NS_REQUIRE(partial && x_scale && x_out && splits >= 1 && rows >= 0, NS_ERR_ARGUMENT, "ns_finish_norm_quant: bad argument");
    NS_REQUIRE(gamma == 0 || (beta != 0 && q != 0 && q_scale != 0), NS_ERR_ARGUMENT, "ns_finish_norm_quant: LayerNorm needs beta, q and q_scale");
    if (rows == 0) return NS_OK;
    const size_t smem = (size_t)n_loc * sizeof(float);
    NS_REQUIRE(smem <= 200 * 1024, NS_ERR_ARGUMENT, "ns_finish_norm_quant: rows of %d columns do not fit in shared memory", n_loc);
    static bool configured[64] = {false};
    if (smem > 48 * 1024 && !configured[d->ordinal]) {
        NS_CUDA(cudaFuncSetAttribute(ns_finish_norm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured[d->ordinal] = true;
    }
    FinishNormParams p;
    p.partial = reinterpret_cast<const int32_t*>(partial);
    p.splits = splits;
    p.x_scale = reinterpret_cast<const float*>(x_scale);
    p.w_scale = reinterpret_cast<const float*>(w_scale);
    p.bias = reinterpret_cast<const float*>(bias);
    p.residual = reinterpret_cast<const uint16_t*>(residual);
    p.rows = rows;
    p.cols = n_loc;
    p.x_out = reinterpret_cast<uint16_t*>(x_out);
    p.gamma = reinterpret_cast<const float*>(gamma);
    p.beta = reinterpret_cast<const float*>(beta);
    p.eps = eps;
    p.q = reinterpret_cast<int8_t*>(q);
    p.q_scale = reinterpret_cast<float*>(q_scale);
    const uint64_t all = partial | x_out | residual | gamma | beta | q | w_scale | bias;
    unsigned threads = 0;
    int vpt = 0;
    if ((all & 15) == 0 && ns_rows::row_shape(n_loc, &threads, &vpt)) {
        NS_CUDA(launch_finish_reg(d, threads, vpt, p));
        return NS_OK;
    }
    const int64_t cap = (int64_t)d->sm_count * 8;
    NS_CUDA(ns_launch_plain(ns_finish_norm_quant_kernel, dim3((unsigned)(rows < cap ? rows : cap)), dim3(FUSED_THREADS), smem, d->stream, p));
    return NS_OK;
}

extern "C" int ns_finish_gelu_quant(ns_device_t h, uint64_t partial, int splits, ns_linear_t linear, uint64_t x_scale, int64_t rows, uint64_t q,
                                    uint64_t q_scale)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    int n_loc = 0, mode = 0;
    uint64_t w_scale = 0, bias = 0;
    rc = ns_linear_info(linear, nullptr, &n_loc, &mode, nullptr, &w_scale, &bias);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(mode == NS_I8 && w_scale != 0 && bias != 0, NS_ERR_ARGUMENT, "ns_finish_gelu_quant: the layer must be an int8 layer with a bias");
    NS_REQUIRE(partial && x_scale && q && q_scale && splits >= 1 && rows >= 0, NS_ERR_ARGUMENT, "ns_finish_gelu_quant: bad argument");
    unsigned threads = 0;
    int vpt = 0;
    NS_REQUIRE(((partial | q | w_scale | bias) & 15) == 0 && ns_rows::row_shape(n_loc, &threads, &vpt), NS_ERR_ARGUMENT,
               "ns_finish_gelu_quant: rows of %d columns (a multiple of 256 up to 8192, buffers 16-byte aligned) expected", n_loc);
    if (rows == 0) return NS_OK;
    FinishGeluParams p;
    p.partial = reinterpret_cast<const int32_t*>(partial);
    p.splits = splits;
    p.x_scale = reinterpret_cast<const float*>(x_scale);
    p.w_scale = reinterpret_cast<const float*>(w_scale);
    p.bias = reinterpret_cast<const float*>(bias);
    p.rows = rows;
    p.cols = n_loc;
    p.q = reinterpret_cast<int8_t*>(q);
    p.q_scale = reinterpret_cast<float*>(q_scale);
    const int64_t cap = (int64_t)d->sm_count * 8;
    const dim3 grid((unsigned)(rows < cap ? rows : cap)), block(threads);
    switch (vpt) {
        case 1: NS_CUDA(ns_launch_plain(ns_finish_gelu_quant_kernel<1>, grid, block, 0, d->stream, p)); break;
        case 2: NS_CUDA(ns_launch_plain(ns_finish_gelu_quant_kernel<2>, grid, block, 0, d->stream, p)); break;
        default: NS_CUDA(ns_launch_plain(ns_finish_gelu_quant_kernel<4>, grid, block, 0, d->stream, p)); break;
    }
    return NS_OK;
}

extern "C" int ns_finish_kv_append(ns_device_t h, uint64_t partial, int splits, ns_linear_t linear, uint64_t x_scale, int batch, int steps,
                                   uint64_t qkv, ns_kv_cache_t cache, uint64_t page_table, int max_pages, uint64_t pos_dev)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    int n_loc = 0, mode = 0;
    uint64_t w_scale = 0, bias = 0;
    rc = ns_linear_info(linear, nullptr, &n_loc, &mode, nullptr, &w_scale, &bias);
    if (rc != NS_OK) return rc;
    NsKvCacheView c;
    rc = ns_kv_cache_view(cache, &c);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(mode == NS_I8 && w_scale != 0, NS_ERR_ARGUMENT, "ns_finish_kv_append: the layer must be an int8 layer");
    NS_REQUIRE(partial && x_scale && qkv && page_table && pos_dev && splits >= 1 && batch >= 0 && steps >= 0 && max_pages > 0, NS_ERR_ARGUMENT,
               "ns_finish_kv_append: bad argument");
    NS_REQUIRE(n_loc == 3 * c.heads * c.head_dim, NS_ERR_ARGUMENT, "ns_finish_kv_append: the layer has %d columns, the cache wants 3 x %d x %d", n_loc,
               c.heads, c.head_dim);
    NS_REQUIRE((qkv & 15) == 0 && (partial & 15) == 0, NS_ERR_ARGUMENT, "ns_finish_kv_append: buffers must be 16-byte aligned");
    const int64_t n = (int64_t)batch * steps * (n_loc / 8);
    if (n == 0) return NS_OK;
    FinishKvParams p;
    p.partial = reinterpret_cast<const int32_t*>(partial);
    p.splits = splits;
    p.x_scale = reinterpret_cast<const float*>(x_scale);
    p.w_scale = reinterpret_cast<const float*>(w_scale);
    p.bias = reinterpret_cast<const float*>(bias);
    p.batch = batch; p.steps = steps;
    p.d_loc = c.heads * c.head_dim;
    p.qkv = reinterpret_cast<uint16_t*>(qkv);
    p.k_pool = c.k_pool; p.v_pool = c.v_pool;
    p.page_table = reinterpret_cast<const int32_t*>(page_table);
    p.max_pages = max_pages; p.page_size = c.page_size; p.heads = c.heads; p.dh = c.head_dim; p.num_pages = c.num_pages;
    p.pos_dev = reinterpret_cast<const int32_t*>(pos_dev);
    p.status = d->status_dev;
    int64_t blocks = (n + 255) / 256;
    if (blocks > (int64_t)d->sm_count * 16) blocks = (int64_t)d->sm_count * 16;
    NS_CUDA(ns_launch_plain(ns_finish_kv_append_kernel, dim3((unsigned)blocks), dim3(256), 0, d->stream, p));
    return NS_OK;
}


// ---------------------------------------------------------------------------------------------------------
// One launch per Linear of the decoding step: the int8 product and, as its second phase, the row operator that
// follows it (ns_tail.cuh).  These replace the pairs ns_linear_forward_partial + ns_finish_* / ns_quantize_rows_i8 /
// ns_tp_reduce_norm_quant above; results are bit-identical to them.
// ---------------------------------------------------------------------------------------------------------
int ns_peer_fill_tail(ns_peer_group_t h, NsDevice* d, int slot, int64_t rows, int cols, NsTail* t, void** slot_ptr);   // ns_peer.cu

namespace {

struct LinearView {
    int k_loc, n_loc, mode;
    uint64_t w, w_scale, bias;
};

int view_linear(ns_linear_t linear, LinearView* v, const char* who)
{
    int rc = ns_linear_info(linear, &v->k_loc, &v->n_loc, &v->mode, &v->w, &v->w_scale, &v->bias);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(v->mode == NS_I8 && v->w_scale != 0, NS_ERR_ARGUMENT, "%s: the layer must be an int8 layer", who);
    return NS_OK;
}

// row shape of the second phase: `active` of its NS_TAIL_THREADS threads hold `vpt` vectors of 8 columns
int tail_row_shape(int cols, NsTail* t, const char* who)
{
    unsigned threads = 0;
    int vpt = 0;
    NS_REQUIRE(ns_rows::row_shape(cols, &threads, &vpt) && threads <= (unsigned)NS_TAIL_THREADS, NS_ERR_ARGUMENT,
               "%s: rows of %d columns (a multiple of 256 up to 8192 is needed)", who, cols);
    t->active = (int)threads;
    t->vpt = vpt;
    return NS_OK;
}

int run_with_tail(NsDevice* d, const LinearView& v, uint64_t x, int M, NsGemmParams p, NsTail* t)
{
    p.prefetch_b = 1;
    return ns_gemm_run(d, NS_KIND_I8, reinterpret_cast<const void*>(x), reinterpret_cast<const void*>(v.w), false, M, v.n_loc, v.k_loc, p, nullptr, 0,
                       nullptr, nullptr, t);
}

}  // namespace

extern "C" int ns_linear_forward_norm_quant(ns_device_t h, ns_linear_t linear, uint64_t x, uint64_t x_scale, uint64_t residual, int64_t rows,
                                            uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q, uint64_t q_scale)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    LinearView v;
    rc = view_linear(linear, &v, "ns_linear_forward_norm_quant");
    if (rc != NS_OK) return rc;
    NS_REQUIRE(x && x_scale && x_out && rows > 0 && rows <= NS_TAIL_MAX_ROWS, NS_ERR_ARGUMENT, "ns_linear_forward_norm_quant: bad argument (1..%d rows)",
               NS_TAIL_MAX_ROWS);
    NS_REQUIRE(gamma == 0 || (beta != 0 && q != 0 && q_scale != 0), NS_ERR_ARGUMENT, "ns_linear_forward_norm_quant: LayerNorm needs beta, q and q_scale");
    NS_REQUIRE(((x_out | residual | gamma | beta | q | v.w_scale | v.bias) & 15) == 0, NS_ERR_ARGUMENT, "ns_linear_forward_norm_quant: buffers must be 16-byte aligned");
    NsTail t = {};
    t.kind = NS_TAIL_NORM;
    rc = tail_row_shape(v.n_loc, &t, "ns_linear_forward_norm_quant");
    if (rc != NS_OK) return rc;
    t.x_scale = reinterpret_cast<const float*>(x_scale);
    t.w_scale = reinterpret_cast<const float*>(v.w_scale);
    t.bias = reinterpret_cast<const float*>(v.bias);
    t.rows = rows; t.cols = v.n_loc;
    t.residual = reinterpret_cast<const uint16_t*>(residual);
    t.x_out = reinterpret_cast<uint16_t*>(x_out);
    t.gamma = reinterpret_cast<const float*>(gamma);
    t.beta = reinterpret_cast<const float*>(beta);
    t.eps = eps;
    t.q = reinterpret_cast<int8_t*>(q);
    t.q_scale = reinterpret_cast<float*>(q_scale);
    NsGemmParams p = {};
    p.epilogue = NS_EPI_NONE; p.out_dtype = NS_F32; p.residual_dtype = NS_F32;
    return run_with_tail(d, v, x, (int)rows, p, &t);
}

extern "C" int ns_linear_forward_gelu_quant(ns_device_t h, ns_linear_t linear, uint64_t x, uint64_t x_scale, int64_t rows, uint64_t q, uint64_t q_scale)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    LinearView v;
    rc = view_linear(linear, &v, "ns_linear_forward_gelu_quant");
    if (rc != NS_OK) return rc;
    NS_REQUIRE(x && x_scale && q && q_scale && rows > 0 && rows <= NS_TAIL_MAX_ROWS, NS_ERR_ARGUMENT, "ns_linear_forward_gelu_quant: bad argument (1..%d rows)",
               NS_TAIL_MAX_ROWS);
    NS_REQUIRE(v.bias != 0, NS_ERR_ARGUMENT, "ns_linear_forward_gelu_quant: the layer has no bias");
    NS_REQUIRE(((q | v.w_scale | v.bias) & 15) == 0, NS_ERR_ARGUMENT, "ns_linear_forward_gelu_quant: buffers must be 16-byte aligned");
    NsTail t = {};
    t.kind = NS_TAIL_GELU;
    rc = tail_row_shape(v.n_loc, &t, "ns_linear_forward_gelu_quant");
    if (rc != NS_OK) return rc;
    t.x_scale = reinterpret_cast<const float*>(x_scale);
    t.w_scale = reinterpret_cast<const float*>(v.w_scale);
    t.bias = reinterpret_cast<const float*>(v.bias);
    t.rows = rows; t.cols = v.n_loc;
    t.q = reinterpret_cast<int8_t*>(q);
    t.q_scale = reinterpret_cast<float*>(q_scale);
    NsGemmParams p = {};
    p.epilogue = NS_EPI_NONE; p.out_dtype = NS_F32; p.residual_dtype = NS_F32;
    return run_with_tail(d, v, x, (int)rows, p, &t);
}

extern "C" int ns_linear_forward_kv_append(ns_device_t h, ns_linear_t linear, uint64_t x, uint64_t x_scale, int batch, int steps, uint64_t qkv,
                                           ns_kv_cache_t cache, uint64_t page_table, int max_pages, uint64_t pos_dev)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    LinearView v;
    rc = view_linear(linear, &v, "ns_linear_forward_kv_append");
    if (rc != NS_OK) return rc;
    NsKvCacheView c;
    rc = ns_kv_cache_view(cache, &c);
    if (rc != NS_OK) return rc;
    const int64_t rows = (int64_t)batch * steps;
    NS_REQUIRE(x && x_scale && qkv && page_table && pos_dev && batch > 0 && steps > 0 && max_pages > 0 && rows <= NS_TAIL_MAX_ROWS, NS_ERR_ARGUMENT,
               "ns_linear_forward_kv_append: bad argument (1..%d rows)", NS_TAIL_MAX_ROWS);
    NS_REQUIRE(v.n_loc == 3 * c.heads * c.head_dim, NS_ERR_ARGUMENT, "ns_linear_forward_kv_append: the layer has %d columns, the cache wants 3 x %d x %d",
               v.n_loc, c.heads, c.head_dim);
    NS_REQUIRE((qkv & 15) == 0, NS_ERR_ARGUMENT, "ns_linear_forward_kv_append: buffers must be 16-byte aligned");
    NsTail t = {};
    t.kind = NS_TAIL_KV;
    t.x_scale = reinterpret_cast<const float*>(x_scale);
    t.w_scale = reinterpret_cast<const float*>(v.w_scale);
    t.bias = reinterpret_cast<const float*>(v.bias);
    t.rows = rows; t.cols = v.n_loc;
    t.batch = batch; t.steps = steps;
    t.d_loc = c.heads * c.head_dim;
    t.qkv = reinterpret_cast<uint16_t*>(qkv);
    t.k_pool = c.k_pool; t.v_pool = c.v_pool;
    t.page_table = reinterpret_cast<const int32_t*>(page_table);
    t.max_pages = max_pages; t.page_size = c.page_size; t.heads = c.heads; t.dh = c.head_dim; t.num_pages = c.num_pages;
    t.pos_dev = reinterpret_cast<const int32_t*>(pos_dev);
    NsGemmParams p = {};
    p.epilogue = NS_EPI_NONE; p.out_dtype = NS_F32; p.residual_dtype = NS_F32;
    return run_with_tail(d, v, x, (int)rows, p, &t);
}

extern "C" int ns_linear_forward_tp_norm_quant(ns_device_t h, ns_linear_t linear, ns_peer_group_t group, int slot, uint64_t x, uint64_t x_scale,
                                               uint64_t residual, int64_t rows, uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q,
                                               uint64_t q_scale)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    LinearView v;
    rc = view_linear(linear, &v, "ns_linear_forward_tp_norm_quant");
    if (rc != NS_OK) return rc;
    NS_REQUIRE(x && x_scale && x_out && rows > 0 && rows <= NS_TAIL_MAX_ROWS && rows <= d->sm_count, NS_ERR_ARGUMENT,
               "ns_linear_forward_tp_norm_quant: bad argument (1..%d rows)", NS_TAIL_MAX_ROWS < d->sm_count ? NS_TAIL_MAX_ROWS : d->sm_count);
    NS_REQUIRE(gamma == 0 || (beta != 0 && q != 0 && q_scale != 0), NS_ERR_ARGUMENT, "ns_linear_forward_tp_norm_quant: LayerNorm needs beta, q and q_scale");
    NS_REQUIRE(((x_out | residual | gamma | beta | q | v.bias) & 15) == 0, NS_ERR_ARGUMENT, "ns_linear_forward_tp_norm_quant: buffers must be 16-byte aligned");
    NsTail t = {};
    t.kind = NS_TAIL_PEER;
    rc = tail_row_shape(v.n_loc, &t, "ns_linear_forward_tp_norm_quant");
    if (rc != NS_OK) return rc;
    void* slot_ptr = nullptr;
    rc = ns_peer_fill_tail(group, d, slot, rows, v.n_loc, &t, &slot_ptr);
    if (rc != NS_OK) return rc;
    // bias and residual are added once, after the ranks' partial rows are summed
    t.bias = reinterpret_cast<const float*>(v.bias);
    t.rows = rows; t.cols = v.n_loc;
    t.residual = reinterpret_cast<const uint16_t*>(residual);
    t.x_out = reinterpret_cast<uint16_t*>(x_out);
    t.gamma = reinterpret_cast<const float*>(gamma);
    t.beta = reinterpret_cast<const float*>(beta);
    t.eps = eps;
    t.q = reinterpret_cast<int8_t*>(q);
    t.q_scale = reinterpret_cast<float*>(q_scale);
    NsGemmParams p = {};
    p.epilogue = NS_EPI_NONE; p.out_dtype = NS_F32; p.residual_dtype = NS_F32;
    p.out = slot_ptr;
    p.a_scale = reinterpret_cast<const float*>(x_scale);
    p.w_scale = reinterpret_cast<const float*>(v.w_scale);
    return run_with_tail(d, v, x, (int)rows, p, &t);
}
