// float32 operator surface: the entry points of the reference's abstract Backend that one cached
// decoder step calls (src/NeuralSharp/Backends/Backend.cs:84-238), with the SAME argument lists, so a
// C# Backend subclass can forward to them one to one.  They keep float32 storage and the reference's
// arithmetic order where it is observable:
//   - every product element is one fused-multiply-add chain over k in ascending order, as in
//     matmul_f32 (Backends/Cuda/PtxKernels.cs:591-596) and CpuMatMul (Backends/Cpu/CpuMatMul.cs:102-175),
//     so results are bit-identical to the CPU backend's;
//   - ids, positions and counters are float-encoded integers in device memory, read with
//     truncation (PtxKernels.Decoding.cs:119-120,132-133), so a captured graph stays valid.
// What changes is the launch geometry: rows are handled by a warp or a CTA instead of one thread
// (the reference runs softmax, LayerNorm and argmax with one thread per row: PtxKernels.Decoding.cs:
// 24-90, PtxKernels.Advanced.cs:144-152).
#include <math.h>

#include "ns_common.cuh"

namespace {

// ------------------------------------------------------------------------------------------------
// C[b] = op(A[b]) * op(B[b]) + beta * C[b]
// 64 x 64 output tile per CTA of 256 threads, 4 x 4 outputs per thread, k consumed in ascending order.
// ------------------------------------------------------------------------------------------------
constexpr int FT = 64, FK = 16;

__global__ void __launch_bounds__(256) ns_f32_matmul_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                                            int m, int n, int k, int transA, int transB, float beta)
{
    __shared__ float As[FK][FT + 1];
    __shared__ float Bs[FK][FT + 1];
    const size_t bi = blockIdx.z;
    a += bi * (size_t)m * k;
    b += bi * (size_t)k * n;
    c += bi * (size_t)m * n;
    const int row0 = blockIdx.y * FT, col0 = blockIdx.x * FT;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < k; k0 += FK) {
        for (int e = threadIdx.x; e < FT * FK; e += 256) {
            // A tile: element (i, p)
            int i, p;
            if (transA) { i = e % FT; p = e / FT; } else { p = e % FK; i = e / FK; }
            int gi = row0 + i, gp = k0 + p;
            float v = 0.0f;
            if (gi < m && gp < k) v = transA ? a[(size_t)gp * m + gi] : a[(size_t)gi * k + gp];
            As[p][i] = v;
            // B tile: element (p, j)
            int j, q;
            if (transB) { q = e % FK; j = e / FK; } else { j = e % FT; q = e / FT; }
            int gj = col0 + j, gq = k0 + q;
            float w = 0.0f;
            if (gj < n && gq < k) w = transB ? b[(size_t)gj * k + gq] : b[(size_t)gq * n + gj];
            Bs[q][j] = w;
        }
        __syncthreads();
        const int kmax = min(FK, k - k0);
        for (int p = 0; p < kmax; p++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[p][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) bv[j] = Bs[p][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int gi = row0 + ty * 4 + i;
        if (gi >= m) continue;
        // columns the CPU backend writes with a vector store use fma(beta, c, acc); its scalar tail uses acc + beta*c
        int vec_end = (gi < (m / 4) * 4) ? (n / 16) * 16 : 0;
        vec_end += ((n - vec_end) / 8) * 8;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int gj = col0 + tx * 4 + j;
            if (gj >= n) continue;
            float* dst = &c[(size_t)gi * n + gj];
            if (beta == 0.0f) *dst = acc[i][j];
            else if (gj < vec_end) *dst = __fmaf_rn(beta, *dst, acc[i][j]);
            else *dst = __fadd_rn(acc[i][j], __fmul_rn(beta, *dst));
        }
    }
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int THREADS>
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red)
{
    v = is_max ? warp_max(v) : warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < THREADS / 32; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// y[r,:] = softmax(scale * x[r,:] + mask[r % maskRows,:]); one CTA of 128 threads per row.
__global__ void __launch_bounds__(128) ns_f32_scale_mask_softmax_kernel(const float* __restrict__ x, const float* __restrict__ mask,
                                                                        float* __restrict__ y, int rows, int cols, int maskRows, float scale)
{
    __shared__ float red[4];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xs = x + (size_t)r * cols;
        const float* ms = mask ? mask + (size_t)(r % maskRows) * cols : nullptr;
        float* ys = y + (size_t)r * cols;
        float mx = -INFINITY;
        for (int j = threadIdx.x; j < cols; j += 128) {
            float v = __fadd_rn(__fmul_rn(xs[j], scale), ms ? ms[j] : 0.0f);
            ys[j] = v;
            mx = fmaxf(mx, v);
        }
        mx = block_reduce<128>(mx, true, red);
        float sum = 0.0f;
        for (int j = threadIdx.x; j < cols; j += 128) {
            float e = expf(ys[j] - mx);
            ys[j] = e;
            sum += e;
        }
        sum = block_reduce<128>(sum, false, red);
        const float inv = 1.0f / sum;
        for (int j = threadIdx.x; j < cols; j += 128) ys[j] *= inv;
    }
}

// Two-pass LayerNorm over the last dimension, biased variance; one CTA of 128 threads per row.
__global__ void __launch_bounds__(128) ns_f32_layernorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                               const float* __restrict__ beta, float* __restrict__ y, int rows, int cols, float eps)
{
    __shared__ float red[4];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xs = x + (size_t)r * cols;
        float* ys = y + (size_t)r * cols;
        float s = 0.0f;
        for (int j = threadIdx.x; j < cols; j += 128) s += xs[j];
        const float mean = block_reduce<128>(s, false, red) / (float)cols;
        float v = 0.0f;
        for (int j = threadIdx.x; j < cols; j += 128) { float d = xs[j] - mean; v += d * d; }
        const float var = block_reduce<128>(v, false, red);
        const float inv = 1.0f / sqrtf(var / (float)cols + eps);
        for (int j = threadIdx.x; j < cols; j += 128)
            ys[j] = __fadd_rn(__fmul_rn(__fmul_rn(xs[j] - mean, inv), gamma[j]), beta[j]);
    }
}

__global__ void ns_f32_bias_gelu_kernel(const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y, int64_t n, int cols)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = ns_gelu_tanh(__fadd_rn(x[i], bias[i % cols]));
}

__global__ void ns_f32_add_rowvec_kernel(const float* __restrict__ a, const float* __restrict__ v, float* __restrict__ c, int64_t n, int cols)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        c[i] = __fadd_rn(a[i], v[i % cols]);
}

__global__ void ns_f32_add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        c[i] = __fadd_rn(a[i], b[i]);
}

__global__ void ns_f32_affine_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n, float alpha, float beta)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = __fmaf_rn(alpha, x[i], beta);
}

__global__ void ns_f32_add_broadcast_scalar_kernel(const float* __restrict__ s, float* __restrict__ y, int64_t n, float scale)
{
    const float v = scale * s[0];
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] += v;
}

__global__ void ns_f32_decoder_mask_kernel(const float* __restrict__ position, float* __restrict__ mask, int rows, int capacity)
{
    const int pos = (int)position[0];
    const int64_t n = (int64_t)rows * capacity;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        int i = (int)(e / capacity), j = (int)(e % capacity);
        mask[e] = j <= pos + i ? 0.0f : -1e9f;
    }
}

__global__ void ns_f32_kv_write_kernel(const float* __restrict__ source, float* __restrict__ cache, const float* __restrict__ position,
                                       int heads, int steps, int capacity, int dim)
{
    const int pos = (int)position[0];
    const int64_t n = (int64_t)heads * steps * dim;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        int d = (int)(e % dim);
        int t = (int)((e / dim) % steps);
        int h = (int)(e / ((int64_t)dim * steps));
        if (pos + t < capacity) cache[((size_t)h * capacity + pos + t) * dim + d] = source[e];
    }
}

// index = truncation of the float id, clamped to the table (the reference's GPU behaviour,
// Backends/Cuda/PtxKernels.Advanced.cs:504-514; its CPU backend throws instead).
__global__ void ns_f32_gather_kernel(const float* __restrict__ table, const float* __restrict__ indices, float* __restrict__ y,
                                     int count, int dim, int vocabulary)
{
    const int64_t n = (int64_t)count * dim;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        int i = (int)(e / dim), d = (int)(e % dim);
        float f = indices[i];
        int idx = f > 0.0f ? (int)f : 0;
        if (idx > vocabulary - 1) idx = vocabulary - 1;
        y[e] = table[(size_t)idx * dim + d];
    }
}

// First maximum per row (strict >), one CTA of 128 threads per row.
__global__ void __launch_bounds__(128) ns_f32_argmax_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols,
                                                            int64_t row_stride, int64_t row_offset)
{
    __shared__ float bv[4];
    __shared__ int bi[4];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xs = x + (size_t)r * row_stride + row_offset;
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int j = threadIdx.x; j < cols; j += 128) {
            float v = xs[j];
            if (idx == 0x7fffffff || v > best) { best = v; idx = j; }
        }
        // lexicographic (value desc, index asc) reduction
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
            for (int w = 1; w < 4; w++)
                if (bi[w] != 0x7fffffff && (i0 == 0x7fffffff || bv[w] > b || (bv[w] == b && bi[w] < i0))) { b = bv[w]; i0 = bi[w]; }
            y[r] = (float)(i0 == 0x7fffffff ? 0 : i0);
        }
    }
}

struct PermuteArgs {
    int rank;
    int shape[6];
    int strides[6];
};

__global__ void ns_f32_permute_kernel(const float* __restrict__ x, float* __restrict__ y, PermuteArgs pa, int64_t n, int accumulate)
{
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = e, off = 0;
        for (int d = pa.rank - 1; d >= 0; d--) {
            int cdim = (int)(rem % pa.shape[d]);
            rem /= pa.shape[d];
            off += (int64_t)cdim * pa.strides[d];
        }
        y[e] = accumulate ? y[e] + x[off] : x[off];
    }
}

__global__ void ns_f32_copy2d_kernel(const float* __restrict__ src, int64_t srcOffset, int srcStride, float* __restrict__ dst, int64_t dstOffset,
                                     int dstStride, int rows, int cols, int accumulate)
{
    const int64_t n = (int64_t)rows * cols;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        int r = (int)(e / cols), cc = (int)(e % cols);
        float v = src[srcOffset + (int64_t)r * srcStride + cc];
        float* d = &dst[dstOffset + (int64_t)r * dstStride + cc];
        *d = accumulate ? *d + v : v;
    }
}

inline unsigned grid_for(const NsDevice* d, int64_t n, int threads)
{
    int64_t blocks = (n + threads - 1) / threads;
    int64_t cap = (int64_t)d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

}  // namespace

#define NS_ENTER(h)                          \
    NsDevice* d = ns_dev(h);                 \
    {                                        \
        int _rc = ns_device_make_current(d); \
        if (_rc != NS_OK) return _rc;        \
    }
#define F32P(x) reinterpret_cast<float*>(x)
#define CF32P(x) reinterpret_cast<const float*>(x)

extern "C" int ns_f32_batched_matmul(ns_device_t h, uint64_t a, uint64_t b, uint64_t c, int batch, int m, int n, int k, int transA, int transB, float beta)
{
    NS_ENTER(h);
    NS_REQUIRE(a && b && c, NS_ERR_ARGUMENT, "ns_f32_batched_matmul: null operand");
    NS_REQUIRE(batch >= 0 && m >= 0 && n >= 0 && k >= 0, NS_ERR_ARGUMENT, "ns_f32_batched_matmul: negative dimension");
    if (batch == 0 || m == 0 || n == 0) return NS_OK;
    // gridDim.z is limited to 65535, as the reference's chunking (CudaBackend.cs:390-408)
    for (int b0 = 0; b0 < batch; b0 += 65535) {
        int nb = batch - b0 < 65535 ? batch - b0 : 65535;
        dim3 grid((n + FT - 1) / FT, (m + FT - 1) / FT, nb);
        ns_f32_matmul_kernel<<<grid, 256, 0, d->stream>>>(CF32P(a) + (size_t)b0 * m * k, CF32P(b) + (size_t)b0 * k * n,
                                                          F32P(c) + (size_t)b0 * m * n, m, n, k, transA, transB, beta);
        NS_CUDA(cudaGetLastError());
    }
    return NS_OK;
}

extern "C" int ns_f32_scale_mask_softmax(ns_device_t h, uint64_t x, uint64_t mask, uint64_t y, int rows, int cols, int maskRows, float scale)
{
    NS_ENTER(h);
    NS_REQUIRE(x && y && rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_f32_scale_mask_softmax: bad argument");
    NS_REQUIRE(mask == 0 || maskRows > 0, NS_ERR_ARGUMENT, "ns_f32_scale_mask_softmax: maskRows must be positive");
    if (rows == 0) return NS_OK;
    unsigned grid = rows < d->sm_count * 16 ? rows : d->sm_count * 16;
    ns_f32_scale_mask_softmax_kernel<<<grid, 128, 0, d->stream>>>(CF32P(x), CF32P(mask), F32P(y), rows, cols, maskRows > 0 ? maskRows : 1, scale);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_layernorm_fused(ns_device_t h, uint64_t x, uint64_t gamma, uint64_t beta, uint64_t y, int rows, int cols, float eps)
{
    NS_ENTER(h);
    NS_REQUIRE(x && gamma && beta && y && rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_f32_layernorm_fused: bad argument");
    if (rows == 0) return NS_OK;
    unsigned grid = rows < d->sm_count * 16 ? rows : d->sm_count * 16;
    ns_f32_layernorm_kernel<<<grid, 128, 0, d->stream>>>(CF32P(x), CF32P(gamma), CF32P(beta), F32P(y), rows, cols, eps);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_bias_gelu(ns_device_t h, uint64_t x, uint64_t bias, uint64_t y, int64_t n, int cols)
{
    NS_ENTER(h);
    NS_REQUIRE(x && bias && y && n >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_f32_bias_gelu: bad argument");
    if (n == 0) return NS_OK;
    ns_f32_bias_gelu_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(x), CF32P(bias), F32P(y), n, cols);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_add_row_vector(ns_device_t h, uint64_t a, uint64_t v, uint64_t c, int rows, int cols)
{
    NS_ENTER(h);
    NS_REQUIRE(a && v && c && rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_f32_add_row_vector: bad argument");
    int64_t n = (int64_t)rows * cols;
    if (n == 0) return NS_OK;
    ns_f32_add_rowvec_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(a), CF32P(v), F32P(c), n, cols);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_add(ns_device_t h, uint64_t a, uint64_t b, uint64_t c, int64_t n)
{
    NS_ENTER(h);
    NS_REQUIRE(a && b && c && n >= 0, NS_ERR_ARGUMENT, "ns_f32_add: bad argument");
    if (n == 0) return NS_OK;
    ns_f32_add_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(a), CF32P(b), F32P(c), n);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_affine(ns_device_t h, uint64_t x, uint64_t y, int64_t n, float alpha, float beta)
{
    NS_ENTER(h);
    NS_REQUIRE(x && y && n >= 0, NS_ERR_ARGUMENT, "ns_f32_affine: bad argument");
    if (n == 0) return NS_OK;
    ns_f32_affine_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(x), F32P(y), n, alpha, beta);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_add_broadcast_scalar(ns_device_t h, uint64_t s, uint64_t y, int64_t n, float scale)
{
    NS_ENTER(h);
    NS_REQUIRE(s && y && n >= 0, NS_ERR_ARGUMENT, "ns_f32_add_broadcast_scalar: bad argument");
    if (n == 0) return NS_OK;
    ns_f32_add_broadcast_scalar_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(s), F32P(y), n, scale);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_decoder_mask(ns_device_t h, uint64_t position, uint64_t mask, int rows, int capacity)
{
    NS_ENTER(h);
    NS_REQUIRE(position && mask && rows >= 0 && capacity > 0, NS_ERR_ARGUMENT, "ns_f32_decoder_mask: bad argument");
    if (rows == 0) return NS_OK;
    ns_f32_decoder_mask_kernel<<<grid_for(d, (int64_t)rows * capacity, 256), 256, 0, d->stream>>>(CF32P(position), F32P(mask), rows, capacity);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_key_value_write(ns_device_t h, uint64_t source, uint64_t cache, uint64_t position, int heads, int steps, int capacity, int dim)
{
    NS_ENTER(h);
    NS_REQUIRE(source && cache && position, NS_ERR_ARGUMENT, "ns_f32_key_value_write: null operand");
    NS_REQUIRE(heads >= 0 && steps >= 0 && dim > 0 && capacity >= steps, NS_ERR_ARGUMENT, "ns_f32_key_value_write: bad shape");
    int64_t n = (int64_t)heads * steps * dim;
    if (n == 0) return NS_OK;
    ns_f32_kv_write_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(source), F32P(cache), CF32P(position), heads, steps, capacity, dim);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_gather(ns_device_t h, uint64_t table, uint64_t indices, uint64_t y, int count, int dim, int vocabulary)
{
    NS_ENTER(h);
    NS_REQUIRE(table && indices && y && count >= 0 && dim > 0 && vocabulary > 0, NS_ERR_ARGUMENT, "ns_f32_gather: bad argument");
    if (count == 0) return NS_OK;
    ns_f32_gather_kernel<<<grid_for(d, (int64_t)count * dim, 256), 256, 0, d->stream>>>(CF32P(table), CF32P(indices), F32P(y), count, dim, vocabulary);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_argmax(ns_device_t h, uint64_t x, uint64_t y, int rows, int cols)
{
    NS_ENTER(h);
    NS_REQUIRE(x && y && rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_f32_argmax: bad argument");
    if (rows == 0) return NS_OK;
    unsigned grid = rows < d->sm_count * 16 ? rows : d->sm_count * 16;
    ns_f32_argmax_kernel<<<grid, 128, 0, d->stream>>>(CF32P(x), F32P(y), rows, cols, cols, 0);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_argmax_strided(ns_device_t h, uint64_t x, uint64_t y, int rows, int cols, int64_t row_stride, int64_t row_offset)
{
    NS_ENTER(h);
    NS_REQUIRE(x && y && rows >= 0 && cols > 0, NS_ERR_ARGUMENT, "ns_f32_argmax_strided: bad argument");
    if (rows == 0) return NS_OK;
    unsigned grid = rows < d->sm_count * 16 ? rows : d->sm_count * 16;
    ns_f32_argmax_kernel<<<grid, 128, 0, d->stream>>>(CF32P(x), F32P(y), rows, cols, row_stride, row_offset);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_permute(ns_device_t h, uint64_t x, uint64_t y, const int* outShape, const int* inStrides, int rank, int accumulate)
{
    NS_ENTER(h);
    NS_REQUIRE(x && y && outShape && inStrides, NS_ERR_ARGUMENT, "ns_f32_permute: null argument");
    NS_REQUIRE(rank >= 1 && rank <= 6, NS_ERR_ARGUMENT, "ns_f32_permute: rank %d not in [1, 6]", rank);
    PermuteArgs pa;
    pa.rank = rank;
    int64_t n = 1;
    for (int i = 0; i < rank; i++) { pa.shape[i] = outShape[i]; pa.strides[i] = inStrides[i]; n *= outShape[i]; }
    if (n == 0) return NS_OK;
    ns_f32_permute_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(x), F32P(y), pa, n, accumulate);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_copy2d(ns_device_t h, uint64_t src, int64_t srcOffset, int srcStride, uint64_t dst, int64_t dstOffset, int dstStride,
                             int rows, int cols, int accumulate)
{
    NS_ENTER(h);
    NS_REQUIRE(src && dst && rows >= 0 && cols >= 0, NS_ERR_ARGUMENT, "ns_f32_copy2d: bad argument");
    int64_t n = (int64_t)rows * cols;
    if (n == 0) return NS_OK;
    ns_f32_copy2d_kernel<<<grid_for(d, n, 256), 256, 0, d->stream>>>(CF32P(src), srcOffset, srcStride, F32P(dst), dstOffset, dstStride, rows, cols, accumulate);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}
