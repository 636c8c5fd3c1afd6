/*
 * ns_oracle.c -- CPU restatement of NeuralSharp's inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the GPU kernels are compared against and the
 * timed CPU baseline; no product code path may call it.  Every function names the reference source
 * it restates (paths inside the ahmedseada/NN project).
 *
 * Pinning status: the reference ships no golden vector files; its tests are literal known answers and
 * self-checking properties (fused == unfused, cached == full, first-max argmax, ...).  The known
 * answers are restated in tests/golden/kat.json and checked against this file.  The int8 / bf16 /
 * paged-attention rules have no counterpart in the (float32-only) reference: for those operations
 * parity is "unpinned" by the reference and the rules are the ones stated beside each function.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -mavx2 -mfma -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off keeps the compiler from fusing a*b+c; every fused multiply-add below is an
 * explicit fmaf / _mm256_fmadd_ps, exactly where the reference uses one.
 */
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------
 * Synthetic inputs: counter-based generator (hash of seed and element index -> uniform -> Box-Muller).
 * Same construction as the reference's CounterRandom (src/NeuralSharp/Backends/Backend.cs:285-298,
 * MurmurHash3 finalizer) and Tensor.Normal (src/NeuralSharp/Tensor.cs:148-165, cos branch).
 * ------------------------------------------------------------------------------------------------ */
static inline uint32_t orc_mix(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
    return h;
}

/* CounterRandom.Uniform(seed, step, row): Backend.cs:288-297. */
ORC_API float orc_counter_uniform(uint32_t seed, uint32_t step, uint32_t row)
{
    uint32_t h = seed ^ (step * 0x9E3779B9u) ^ (row * 0x85EBCA6Bu);
    return (float)(orc_mix(h) >> 8) * (1.0f / 16777216.0f);
}

static inline uint32_t orc_hash2(uint32_t seed, uint64_t index, uint32_t lane)
{
    uint32_t lo = (uint32_t)index, hi = (uint32_t)(index >> 32);
    uint32_t h = orc_mix(seed * 0x9E3779B9u + 0x7F4A7C15u + lane);
    h = orc_mix(h ^ (lo * 0x85EBCA6Bu));
    h = orc_mix(h ^ (hi * 0xC2B2AE35u) ^ 0x27D4EB2Fu);
    return h;
}

/* out[i] = mean + std * N(0,1), element i depends only on (seed, offset + i). */
ORC_API void orc_fill_normal(float *out, int64_t n, uint32_t seed, uint64_t offset, float mean, float std)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        uint64_t idx = offset + (uint64_t)i;
        double u1 = 1.0 - (double)(orc_hash2(seed, idx, 0) >> 8) * (1.0 / 16777216.0); /* (0,1] */
        double u2 = (double)(orc_hash2(seed, idx, 1) >> 8) * (1.0 / 16777216.0);       /* [0,1) */
        double r = sqrt(-2.0 * log(u1));
        out[i] = (float)((double)mean + (double)std * r * cos(2.0 * M_PI * u2));
    }
}

/* out[i] = uniform integer in [0, bound) stored as float (token ids are float-encoded in the reference:
 * src/NeuralSharp/Backends/Cuda/PtxKernels.Advanced.cs:504-514). */
ORC_API void orc_fill_ids(float *out, int64_t n, uint32_t seed, uint64_t offset, uint32_t bound)
{
    for (int64_t i = 0; i < n; i++) {
        out[i] = (float)(orc_hash2(seed, offset + (uint64_t)i, 2) % bound);
    }
}

/* ------------------------------------------------------------------------------------------------
 * float32 GEMM.  C = op(A) * op(B) + beta * C, row-major, every output element one sequential
 * fused-multiply-add chain over p = 0..k-1 (src/NeuralSharp/Backends/Cpu/CpuMatMul.cs:102-175; the
 * GPU kernel has the same chain, Backends/Cuda/PtxKernels.cs:591-596).  beta: vector columns use
 * fma(beta, c, acc) (CpuMatMul.cs:182-190), scalar tail columns acc + beta*c (CpuMatMul.cs:176-177).
 * orc_matmul_f32_scalar is the definition; orc_matmul_f32 is the blocked AVX2 + threads version used
 * as the timed CPU baseline (4 rows x 16 columns in registers, row blocks in parallel when
 * m*n*k >= 2^17: CpuMatMul.cs:19,42-54) and gives bit-identical results because SIMD lanes are
 * independent outputs.
 * ------------------------------------------------------------------------------------------------ */
static inline float orc_a_at(const float *a, int i, int p, int m, int k, int transA)
{
    return transA ? a[(size_t)p * m + i] : a[(size_t)i * k + p];
}

ORC_API void orc_matmul_f32_scalar(const float *a, const float *b, float *c, int batch, int m, int n, int k,
                                   int transA, int transB, float beta)
{
    for (int bi = 0; bi < batch; bi++) {
        const float *A = a + (size_t)bi * m * k, *B = b + (size_t)bi * k * n;
        float *C = c + (size_t)bi * m * n;
        for (int i = 0; i < m; i++) {
            /* which columns the reference computes with vector stores */
            int vec_end = (i < (m / 4) * 4) ? (n / 16) * 16 : 0;
            vec_end = vec_end + ((n - vec_end) / 8) * 8;
            for (int j = 0; j < n; j++) {
                float acc = 0.0f;
                for (int p = 0; p < k; p++) {
                    float bv = transB ? B[(size_t)j * k + p] : B[(size_t)p * n + j];
                    acc = fmaf(orc_a_at(A, i, p, m, k, transA), bv, acc);
                }
                float *dst = &C[(size_t)i * n + j];
                if (beta == 0.0f) *dst = acc;
                else if (j < vec_end) *dst = fmaf(beta, *dst, acc);
                else *dst = acc + beta * *dst;
            }
        }
    }
}

static void orc_transpose(const float *src, float *dst, int rows, int cols)
{
    /* CpuMatMul.Transpose, CpuMatMul.cs:62-81: dst[col*rows + r] = src[r*cols + col] */
    for (int r0 = 0; r0 < rows; r0 += 32)
        for (int c0 = 0; c0 < cols; c0 += 32)
            for (int r = r0; r < rows && r < r0 + 32; r++)
                for (int cc = c0; cc < cols && cc < c0 + 32; cc++)
                    dst[(size_t)cc * rows + r] = src[(size_t)r * cols + cc];
}

static inline void orc_store8(float *dst, __m256 v, float beta)
{
    if (beta != 0.0f) v = _mm256_fmadd_ps(_mm256_set1_ps(beta), _mm256_loadu_ps(dst), v);
    _mm256_storeu_ps(dst, v);
}

static void orc_row_tail(const float *a, const float *b, float *c, int i, int j, int n, int k,
                         ptrdiff_t rs, ptrdiff_t cs, float beta)
{
    /* CpuMatMul.Row, CpuMatMul.cs:150-179 */
    const float *ai = a + i * rs;
    float *ci = c + (size_t)i * n;
    for (; j + 8 <= n; j += 8) {
        __m256 acc = _mm256_setzero_ps();
        for (int p = 0; p < k; p++)
            acc = _mm256_fmadd_ps(_mm256_set1_ps(ai[p * cs]), _mm256_loadu_ps(b + (size_t)p * n + j), acc);
        orc_store8(ci + j, acc, beta);
    }
    for (; j < n; j++) {
        float acc = 0.0f;
        for (int p = 0; p < k; p++) acc = fmaf(ai[p * cs], b[(size_t)p * n + j], acc);
        ci[j] = beta == 0.0f ? acc : acc + beta * ci[j];
    }
}

static void orc_run_block(const float *a, const float *b, float *c, int block, int m, int n, int k,
                          ptrdiff_t rs, ptrdiff_t cs, float beta)
{
    /* CpuMatMul.RunBlock + Block4, CpuMatMul.cs:83-148 */
    int i0 = block * 4, rows = m - i0 < 4 ? m - i0 : 4, j = 0;
    if (rows == 4) {
        const float *a0 = a + i0 * rs, *a1 = a0 + rs, *a2 = a1 + rs, *a3 = a2 + rs;
        for (; j + 16 <= n; j += 16) {
            __m256 c00 = _mm256_setzero_ps(), c01 = c00, c10 = c00, c11 = c00, c20 = c00, c21 = c00, c30 = c00, c31 = c00;
            const float *bj = b + j;
            for (int p = 0; p < k; p++) {
                __m256 b0 = _mm256_loadu_ps(bj + (size_t)p * n), b1 = _mm256_loadu_ps(bj + (size_t)p * n + 8);
                __m256 x = _mm256_set1_ps(a0[p * cs]);
                c00 = _mm256_fmadd_ps(x, b0, c00); c01 = _mm256_fmadd_ps(x, b1, c01);
                x = _mm256_set1_ps(a1[p * cs]);
                c10 = _mm256_fmadd_ps(x, b0, c10); c11 = _mm256_fmadd_ps(x, b1, c11);
                x = _mm256_set1_ps(a2[p * cs]);
                c20 = _mm256_fmadd_ps(x, b0, c20); c21 = _mm256_fmadd_ps(x, b1, c21);
                x = _mm256_set1_ps(a3[p * cs]);
                c30 = _mm256_fmadd_ps(x, b0, c30); c31 = _mm256_fmadd_ps(x, b1, c31);
            }
            float *c0 = c + (size_t)i0 * n + j, *c1 = c0 + n, *c2 = c1 + n, *c3 = c2 + n;
            orc_store8(c0, c00, beta); orc_store8(c0 + 8, c01, beta);
            orc_store8(c1, c10, beta); orc_store8(c1 + 8, c11, beta);
            orc_store8(c2, c20, beta); orc_store8(c2 + 8, c21, beta);
            orc_store8(c3, c30, beta); orc_store8(c3 + 8, c31, beta);
        }
    }
    for (int r = 0; r < rows; r++) orc_row_tail(a, b, c, i0 + r, j, n, k, rs, cs, beta);
}

static void orc_multiply(const float *a, const float *b, float *c, int m, int n, int k, int transA, int transB,
                         float beta, int allow_parallel)
{
    /* CpuMatMul.Multiply, CpuMatMul.cs:25-60 */
    float *rented = NULL;
    if (transB) {
        rented = (float *)malloc(sizeof(float) * (size_t)k * n);
        orc_transpose(b, rented, n, k);
        b = rented;
    }
    ptrdiff_t rs = transA ? 1 : k, cs = transA ? m : 1;
    int blocks = (m + 3) / 4;
    if ((long long)m * n * k < (1LL << 17) || blocks == 1 || !allow_parallel) {
        for (int bl = 0; bl < blocks; bl++) orc_run_block(a, b, c, bl, m, n, k, rs, cs, beta);
    } else {
#pragma omp parallel for schedule(dynamic, 4)
        for (int bl = 0; bl < blocks; bl++) orc_run_block(a, b, c, bl, m, n, k, rs, cs, beta);
    }
    free(rented);
}

/* CpuBackend.BatchedMatMul, src/NeuralSharp/Backends/Cpu/CpuBackend.Advanced.cs:31-49: batch == 1 ->
 * row-block parallel; batch > 1 -> parallel over the batch, each product single-threaded. */
ORC_API void orc_matmul_f32(const float *a, const float *b, float *c, int batch, int m, int n, int k,
                            int transA, int transB, float beta)
{
    if (batch == 1) { orc_multiply(a, b, c, m, n, k, transA, transB, beta, 1); return; }
#pragma omp parallel for schedule(dynamic, 1)
    for (int bi = 0; bi < batch; bi++)
        orc_multiply(a + (size_t)bi * m * k, b + (size_t)bi * k * n, c + (size_t)bi * m * n, m, n, k, transA, transB, beta, 0);
}

ORC_API void orc_set_threads(int n)
{
#ifdef _OPENMP
    omp_set_num_threads(n > 0 ? n : omp_get_num_procs());
#else
    (void)n;
#endif
}

ORC_API int orc_get_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------------------------
 * Row-wise inference operators (src/NeuralSharp/Backends/Cpu/CpuBackend.Decoding.cs).
 * ------------------------------------------------------------------------------------------------ */

/* ScaleMaskSoftmax, CpuBackend.Decoding.cs:9-41: y = x*scale + mask[r % maskRows]; max; exp(y-max)
 * summed in float; multiply by 1/sum. */
ORC_API void orc_scale_mask_softmax(const float *x, const float *mask, float *y, int rows, int cols, int maskRows, float scale)
{
#pragma omp parallel for schedule(static) if ((long long)rows * cols > 65536)
    for (int r = 0; r < rows; r++) {
        const float *xs = x + (size_t)r * cols;
        float *ys = y + (size_t)r * cols;
        const float *ms = mask ? mask + (size_t)(r % maskRows) * cols : NULL;
        float max = -INFINITY;
        for (int j = 0; j < cols; j++) {
            ys[j] = xs[j] * scale + (ms ? ms[j] : 0.0f);
            max = fmaxf(max, ys[j]);
        }
        float sum = 0.0f;
        for (int j = 0; j < cols; j++) { ys[j] = expf(ys[j] - max); sum += ys[j]; }
        float inv = 1.0f / sum;
        for (int j = 0; j < cols; j++) ys[j] *= inv;
    }
}

/* Unfused softmax (double sum), CpuBackend.Advanced.cs:51-80; used to restate the reference's
 * FusedKernels test (tests/NeuralSharp.Tests/DecodingTests.cs:34-67). */
ORC_API void orc_softmax(const float *x, float *y, int rows, int cols)
{
    for (int r = 0; r < rows; r++) {
        const float *xs = x + (size_t)r * cols;
        float *ys = y + (size_t)r * cols;
        float max = -INFINITY;
        for (int j = 0; j < cols; j++) max = fmaxf(max, xs[j]);
        double sum = 0.0;
        for (int j = 0; j < cols; j++) sum += exp((double)(xs[j] - max));
        for (int j = 0; j < cols; j++) ys[j] = (float)(exp((double)(xs[j] - max)) / sum);
    }
}

/* LayerNormFused, CpuBackend.Decoding.cs:43-72: two passes, float sums, biased variance. */
ORC_API void orc_layernorm_fused(const float *x, const float *gamma, const float *beta, float *y, int rows, int cols, float eps)
{
#pragma omp parallel for schedule(static) if ((long long)rows * cols > 65536)
    for (int r = 0; r < rows; r++) {
        const float *xs = x + (size_t)r * cols;
        float *ys = y + (size_t)r * cols;
        float mean = 0.0f;
        for (int j = 0; j < cols; j++) mean += xs[j];
        mean /= (float)cols;
        float var = 0.0f;
        for (int j = 0; j < cols; j++) var += (xs[j] - mean) * (xs[j] - mean);
        float inv = 1.0f / sqrtf(var / (float)cols + eps);
        for (int j = 0; j < cols; j++) ys[j] = (xs[j] - mean) * inv * gamma[j] + beta[j];
    }
}

static inline float orc_gelu(float v)
{
    /* constants: CpuBackend.Advanced.cs:770-772 */
    const float GeluK = 0.7978845608f, GeluC = 0.044715f;
    return 0.5f * v * (1.0f + tanhf(GeluK * (v + GeluC * v * v * v)));
}

/* BiasGelu, CpuBackend.Decoding.cs:74-89. */
ORC_API void orc_bias_gelu(const float *x, const float *bias, float *y, int64_t n, int cols)
{
    int64_t rows = n / cols;
#pragma omp parallel for schedule(static) if (n > 65536)
    for (int64_t r = 0; r < rows; r++)
        for (int j = 0; j < cols; j++) y[r * cols + j] = orc_gelu(x[r * cols + j] + bias[j]);
}

/* AddRowVector (bias add after every Linear): c[i] = a[i] + v[i % cols], CpuBackend.cs; GPU
 * add_rowvec_f32 PtxKernels.cs:225-234. */
ORC_API void orc_add_rowvec(const float *a, const float *v, float *c, int64_t rows, int cols)
{
    for (int64_t r = 0; r < rows; r++)
        for (int j = 0; j < cols; j++) c[r * cols + j] = a[r * cols + j] + v[j];
}

ORC_API void orc_add(const float *a, const float *b, float *c, int64_t n)
{
    for (int64_t i = 0; i < n; i++) c[i] = a[i] + b[i];
}

/* DecoderMask, CpuBackend.Decoding.cs:91-102. */
ORC_API void orc_decoder_mask(const float *position, float *mask, int rows, int capacity)
{
    int pos = (int)position[0];
    for (int i = 0; i < rows; i++)
        for (int j = 0; j < capacity; j++) mask[(size_t)i * capacity + j] = j <= pos + i ? 0.0f : -1e9f;
}

/* KeyValueWrite, CpuBackend.Decoding.cs:104-112: cache[h, pos + t, :] = source[h, t, :]. */
ORC_API void orc_kv_write(const float *source, float *cache, const float *position, int heads, int steps, int capacity, int dim)
{
    int pos = (int)position[0];
    for (int h = 0; h < heads; h++)
        memcpy(cache + ((size_t)h * capacity + pos) * dim, source + (size_t)h * steps * dim, sizeof(float) * (size_t)steps * dim);
}

/* Gather, CpuBackend.Advanced.cs:399-429.  Returns -1 when an index is not an integer in
 * [0, vocabulary) (the reference throws IndexOutOfRangeException there). */
ORC_API int orc_gather(const float *table, const float *indices, float *y, int count, int dim, int vocabulary)
{
    for (int i = 0; i < count; i++) {
        int index = (int)indices[i];
        if ((unsigned)index >= (unsigned)vocabulary || (float)index != indices[i]) return -1;
        memcpy(y + (size_t)i * dim, table + (size_t)index * dim, sizeof(float) * dim);
    }
    return 0;
}

/* ArgMax, CpuBackend.Advanced.cs:117-138: first maximum wins (strict >). */
ORC_API void orc_argmax(const float *x, float *y, int rows, int cols)
{
    for (int r = 0; r < rows; r++) {
        const float *row = x + (size_t)r * cols;
        int best = 0;
        for (int j = 1; j < cols; j++) if (row[j] > row[best]) best = j;
        y[r] = (float)best;
    }
}

/* Sinusoidal position table, src/NeuralSharp/Layers/Attention.cs:236-246. */
ORC_API void orc_sinusoid_table(float *table, int maxLength, int dim)
{
    for (int pos = 0; pos < maxLength; pos++)
        for (int i = 0; i < dim; i++) {
            double angle = pos / pow(10000.0, 2 * (i / 2) / (double)dim);
            table[(size_t)pos * dim + i] = (float)(i % 2 == 0 ? sin(angle) : cos(angle));
        }
}

/* ------------------------------------------------------------------------------------------------
 * Rules the float32-only reference does not have (parity unpinned by the reference; these are the
 * definitions the CUDA kernels are held to).
 * ------------------------------------------------------------------------------------------------ */

/* bf16 <-> f32, round to nearest even. */
ORC_API uint16_t orc_f32_to_bf16(float f)
{
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
ORC_API float orc_bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f;
}
ORC_API void orc_round_bf16(const float *x, uint16_t *y, int64_t n)
{
#pragma omp parallel for schedule(static) if (n > 65536)
    for (int64_t i = 0; i < n; i++) y[i] = orc_f32_to_bf16(x[i]);
}
ORC_API void orc_widen_bf16(const uint16_t *x, float *y, int64_t n)
{
#pragma omp parallel for schedule(static) if (n > 65536)
    for (int64_t i = 0; i < n; i++) y[i] = orc_bf16_to_f32(x[i]);
}

/* Symmetric absmax int8 per row: scale = absmax / 127 (absmax == 0 -> 1); q = clamp(rint(x / scale),
 * -127, 127), round half to even.  Rows of A [M,K] for activations; rows of W [N,K] (= one output
 * channel, a column of the reference's [K,N] Linear.Weight, src/NeuralSharp/Layers/Linear.cs:25-27). */
ORC_API void orc_quantize_rows_i8(const float *x, int64_t rows, int cols, int8_t *q, float *scale)
{
#pragma omp parallel for schedule(static) if (rows * cols > 65536)
    for (int64_t r = 0; r < rows; r++) {
        const float *xs = x + r * cols;
        float amax = 0.0f;
        for (int j = 0; j < cols; j++) amax = fmaxf(amax, fabsf(xs[j]));
        float s = amax == 0.0f ? 1.0f : amax / 127.0f;
        scale[r] = s;
        for (int j = 0; j < cols; j++) {
            float v = rintf(xs[j] / s);
            v = v > 127.0f ? 127.0f : (v < -127.0f ? -127.0f : v);
            q[r * cols + j] = (int8_t)v;
        }
    }
}

/* Same rule with bf16 input (activations of the W8A8 decoder are bf16). */
ORC_API void orc_quantize_rows_i8_bf16(const uint16_t *x, int64_t rows, int cols, int8_t *q, float *scale)
{
#pragma omp parallel for schedule(static) if (rows * cols > 65536)
    for (int64_t r = 0; r < rows; r++) {
        const uint16_t *xs = x + r * cols;
        float amax = 0.0f;
        for (int j = 0; j < cols; j++) amax = fmaxf(amax, fabsf(orc_bf16_to_f32(xs[j])));
        float s = amax == 0.0f ? 1.0f : amax / 127.0f;
        scale[r] = s;
        for (int j = 0; j < cols; j++) {
            float v = rintf(orc_bf16_to_f32(xs[j]) / s);
            v = v > 127.0f ? 127.0f : (v < -127.0f ? -127.0f : v);
            q[r * cols + j] = (int8_t)v;
        }
    }
}

/* int8 x int8 -> exact int32: acc[m,n] = sum_k aq[m,k] * wq[n,k]  (W stored [N,K]).
 * Rows [row0, row0+nrows) only, so large M can be sampled. */
ORC_API void orc_qmatmul_i8_acc(const int8_t *aq, const int8_t *wq, int32_t *acc, int row0, int nrows, int N, int K)
{
#pragma omp parallel for schedule(static) collapse(2)
    for (int i = 0; i < nrows; i++)
        for (int j = 0; j < N; j++) {
            const int8_t *ar = aq + (size_t)(row0 + i) * K, *wr = wq + (size_t)j * K;
            int32_t s = 0;
            for (int p = 0; p < K; p++) s += (int32_t)ar[p] * (int32_t)wr[p];
            acc[(size_t)i * N + j] = s;
        }
}

/* Dequant epilogue: y = ((float)acc * a_scale[m]) * w_scale[n] + bias[n], each step rounded to
 * float (no fused multiply-add); act: 0 none, 1 tanh-GELU (constants as orc_gelu); optional residual
 * added last. a_scale is indexed from row0. */
ORC_API void orc_dequant_epilogue(const int32_t *acc, const float *a_scale, const float *w_scale, const float *bias,
                                  const float *residual, float *y, int row0, int nrows, int N, int act)
{
    for (int i = 0; i < nrows; i++)
        for (int j = 0; j < N; j++) {
            float v = ((float)acc[(size_t)i * N + j] * a_scale[row0 + i]) * w_scale[j];
            if (bias) v = v + bias[j];
            if (act == 1) v = orc_gelu(v);
            if (residual) v = v + residual[(size_t)i * N + j];
            y[(size_t)i * N + j] = v;
        }
}

/* bf16 GEMM: inputs already rounded to bf16, products accumulated in float in k order (fmaf chain),
 * C[i,j] for rows [row0,row0+nrows).  b_is_nk: B stored [N,K] (else [K,N]).  The result is returned as
 * float; the caller rounds to bf16 when the kernel under test writes bf16.  The tolerance (1e-2
 * relative, |e-a| <= tol*max(1,|e|)) absorbs the accumulation-order difference of the tensor cores. */
ORC_API void orc_matmul_bf16(const uint16_t *a, const uint16_t *b, float *c, int row0, int nrows, int N, int K, int b_is_nk)
{
    float *bt = NULL;
    /* widen B once to [N,K] float */
    bt = (float *)malloc(sizeof(float) * (size_t)N * K);
#pragma omp parallel for schedule(static)
    for (int j = 0; j < N; j++)
        for (int p = 0; p < K; p++)
            bt[(size_t)j * K + p] = orc_bf16_to_f32(b_is_nk ? b[(size_t)j * K + p] : b[(size_t)p * N + j]);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < nrows; i++) {
        float *ar = (float *)malloc(sizeof(float) * K);
        for (int p = 0; p < K; p++) ar[p] = orc_bf16_to_f32(a[(size_t)(row0 + i) * K + p]);
        for (int j = 0; j < N; j++) {
            const float *br = bt + (size_t)j * K;
            float acc = 0.0f;
            for (int p = 0; p < K; p++) acc = fmaf(ar[p], br[p], acc);
            c[(size_t)i * N + j] = acc;
        }
        free(ar);
    }
    free(bt);
}

/* Causal attention for one (batch, head) slice, reference order (src/NeuralSharp/Layers/Attention.cs:
 * 54-90 and 98-118): s = (q . k) * scale + mask, mask = 0 if j <= q_pos0 + i else -1e9; softmax with
 * float sum (CpuBackend.Decoding.cs:9-41); o = p . v.  q: [tq, dh] rows; k, v: [tk, dh] (tk = cache
 * capacity or sequence length); strides in elements.  Row i of q sits at absolute position
 * q_pos0 + i.  All inputs float (bf16 inputs are widened by the caller). */
ORC_API void orc_attention_slice(const float *q, const float *k, const float *v, float *o, int tq, int tk, int dh,
                                 int64_t q_stride, int64_t k_stride, int64_t v_stride, int64_t o_stride,
                                 int q_pos0, float scale, int causal)
{
#pragma omp parallel
    {
        float *s = (float *)malloc(sizeof(float) * tk);
#pragma omp for schedule(dynamic, 4)
        for (int i = 0; i < tq; i++) {
            const float *qi = q + i * q_stride;
            float max = -INFINITY;
            for (int j = 0; j < tk; j++) {
                const float *kj = k + j * k_stride;
                float acc = 0.0f;
                for (int d = 0; d < dh; d++) acc = fmaf(qi[d], kj[d], acc);
                float m = (causal && j > q_pos0 + i) ? -1e9f : 0.0f;
                s[j] = acc * scale + m;
                max = fmaxf(max, s[j]);
            }
            float sum = 0.0f;
            for (int j = 0; j < tk; j++) { s[j] = expf(s[j] - max); sum += s[j]; }
            float inv = 1.0f / sum;
            for (int j = 0; j < tk; j++) s[j] *= inv;
            float *oi = o + i * o_stride;
            for (int d = 0; d < dh; d++) oi[d] = 0.0f;
            for (int j = 0; j < tk; j++) {
                if (s[j] == 0.0f) continue; /* exact: adds +0 */
                const float *vj = v + j * v_stride;
                for (int d = 0; d < dh; d++) oi[d] = fmaf(s[j], vj[d], oi[d]);
            }
        }
        free(s);
    }
}

/* ------------------------------------------------------------------------------------------------
 * Token sampler (src/NeuralSharp/Backends/Cpu/CpuBackend.Decoding.cs:114-292), float32, restated
 * pass for pass: scaled scores s = z / max(T, 1e-3); top-k threshold = k-th largest distinct score;
 * min-p threshold max + ln(minP); top-p by 24 bisection steps on the score; e = exp(s - max) above the
 * threshold; first index whose running sum exceeds u * sum with u = CounterRandom.Uniform(seed, step,
 * row); 13 statistics per token: id, probability, entropy in bits, five (alternative id, probability)
 * pairs (-1, 0 when fewer exist).
 * ------------------------------------------------------------------------------------------------ */
ORC_API void orc_sample_rows(const float *logits, float *ids, float *stats, const float *step, int rows, int vocabulary,
                             int rowStride, int rowOffset, float temperature, int topK, float topP, float minP, uint32_t seed)
{
    uint32_t stepNumber = (uint32_t)step[0];
    float invT = 1.0f / fmaxf(temperature, 1e-3f);
    float *e = (float *)malloc(sizeof(float) * vocabulary);
    for (int r = 0; r < rows; r++) {
        const float *z = logits + (size_t)r * rowStride + rowOffset;
        float max = -INFINITY;
        for (int j = 0; j < vocabulary; j++) max = fmaxf(max, z[j] * invT);
        float threshold = -INFINITY;
        if (topK > 0 && topK < vocabulary) {
            threshold = INFINITY;
            for (int k = 0; k < topK; k++) {
                float next = -INFINITY;
                for (int j = 0; j < vocabulary; j++) {
                    float s = z[j] * invT;
                    if (s < threshold && s > next) next = s;
                }
                threshold = next;
            }
        }
        if (minP > 0.0f) threshold = fmaxf(threshold, max + logf(minP));
        if (topP > 0.0f && topP < 1.0f) {
            float total = 0.0f;
            for (int j = 0; j < vocabulary; j++) {
                float s = z[j] * invT;
                total += s >= threshold ? expf(s - max) : 0.0f;
            }
            float goal = total * topP, lo = fmaxf(max - 40.0f, threshold), hi = max;
            for (int it = 0; it < 24; it++) {
                float mid = (lo + hi) * 0.5f, mass = 0.0f;
                for (int j = 0; j < vocabulary; j++) {
                    float s = z[j] * invT;
                    mass += (s >= threshold && s >= mid) ? expf(s - max) : 0.0f;
                }
                if (mass >= goal) lo = mid; else hi = mid;
            }
            threshold = lo;
        }
        float sum = 0.0f;
        for (int j = 0; j < vocabulary; j++) {
            float s = z[j] * invT;
            e[j] = s >= threshold ? expf(s - max) : 0.0f;
            sum += e[j];
        }
        float target = orc_counter_uniform(seed, stepNumber, (uint32_t)r) * sum;
        int chosen = -1;
        float cumulative = 0.0f;
        for (int j = 0; j < vocabulary; j++) {
            if (e[j] > 0.0f) {
                chosen = j;
                cumulative += e[j];
                if (cumulative > target) break;
            }
        }
        float entropy = 0.0f;
        for (int j = 0; j < vocabulary; j++)
            if (e[j] > 0.0f) { float p = e[j] / sum; entropy -= p * log2f(p); }
        ids[r] = (float)chosen;
        size_t o = ((size_t)stepNumber * rows + r) * 13;
        stats[o] = (float)chosen;
        stats[o + 1] = e[chosen] / sum;
        stats[o + 2] = entropy;
        int taken[5];
        for (int a = 0; a < 5; a++) {
            int best = -1;
            for (int j = 0; j < vocabulary; j++) {
                if (e[j] > 0.0f && (best < 0 || e[j] > e[best])) {
                    int used = 0;
                    for (int t = 0; t < a; t++) used |= taken[t] == j;
                    if (!used) best = j;
                }
            }
            taken[a] = best;
            stats[o + 3 + 2 * a] = (float)best;
            stats[o + 4 + 2 * a] = best < 0 ? 0.0f : e[best] / sum;
        }
    }
    free(e);
}

/* PenalizeRows, CpuBackend.Decoding.cs:247-282. */
ORC_API void orc_penalize_rows(const float *logits, float *work, const float *history, const float *length, int rows, int vocabulary,
                               int rowStride, int rowOffset, int capacity, int lastN, float repeat, float presence, float frequency)
{
    uint32_t len = (uint32_t)length[0];
    uint32_t lim = (uint32_t)(lastN < capacity ? lastN : capacity);
    int n = (int)(len < lim ? len : lim);
    for (int r = 0; r < rows; r++) {
        float *w = work + (size_t)r * vocabulary;
        memcpy(w, logits + (size_t)r * rowStride + rowOffset, sizeof(float) * vocabulary);
        for (int k = 0; k < n; k++) {
            int id = (int)history[(size_t)r * capacity + (int)((len - 1 - (uint32_t)k) % (uint32_t)capacity)];
            int seenMoreRecently = 0, count = 0;
            for (int q = 0; q < n; q++) {
                int other = (int)history[(size_t)r * capacity + (int)((len - 1 - (uint32_t)q) % (uint32_t)capacity)];
                if (other == id) { count++; seenMoreRecently |= q < k; }
            }
            if (seenMoreRecently || (unsigned)id >= (unsigned)vocabulary) continue;
            float x = w[id];
            x = x > 0.0f ? x / repeat : x * repeat;
            w[id] = x - presence - frequency * count;
        }
    }
}

/* HistoryPush, CpuBackend.Decoding.cs:284-292. */
ORC_API void orc_history_push(const float *ids, float *history, const float *length, int rows, int capacity)
{
    uint32_t len = (uint32_t)length[0];
    for (int r = 0; r < rows; r++) history[(size_t)r * capacity + (int)(len % (uint32_t)capacity)] = ids[r];
}
