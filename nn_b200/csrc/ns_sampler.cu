// On-device token sampler of the float32 operator surface: SampleRows, PenalizeRows, HistoryPush with the
// reference's argument lists (src/NeuralSharp/Backends/Backend.cs:240-261) and its algorithm, pass for pass
// (Backends/Cpu/CpuBackend.Decoding.cs:114-292, mirrored there by the kernel sample_rows_f32,
// Backends/Cuda/PtxKernels.Decoding.cs:170-447): scaled scores s = z / max(T, 1e-3); top-k cut-off = k-th largest
// distinct score; min-p cut-off max + ln(minP); top-p by 24 bisection steps on the score; e = exp(s - max) above the
// cut-off; the first index whose running sum exceeds u * sum, u = CounterRandom.Uniform(seed, step, row)
// (Backend.cs:288-297); 13 statistics per token.  The step number, history length and ids are float-encoded
// values in device memory, so a recorded graph stays valid.
//
// The reference runs ONE THREAD per row and makes k + 30-odd serial passes over the vocabulary; here a CTA of 256
// threads handles a row and every pass is a block reduction.  Sums are therefore added in another order than the
// CPU's sequential float sum; the reference accepts up to 0.5 % differing draws between its own CPU and GPU
// backends for the same reason (tests/NeuralSharp.Tests/DecodingTests.cs:232-243).
#include <math.h>

#include "ns_common.cuh"

namespace {

constexpr int SAMP_THREADS = 256;

__device__ __forceinline__ float block_max(float v, float* red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < SAMP_THREADS / 32; w++) r = fmaxf(r, red[w]);
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < SAMP_THREADS / 32; w++) r += red[w];
    return r;
}

__device__ __forceinline__ uint32_t mix32(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
    return h;
}
__device__ __forceinline__ float counter_uniform(uint32_t seed, uint32_t step, uint32_t row)
{
    const uint32_t h = seed ^ (step * 0x9E3779B9u) ^ (row * 0x85EBCA6Bu);
    return (float)(mix32(h) >> 8) * (1.0f / 16777216.0f);
}

// (value, index) reduction: larger value wins, ties go to the smaller index; index -1 = nothing.
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* redv, int* redi)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi >= 0 && (idx < 0 || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { redv[threadIdx.x >> 5] = v; redi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    v = redv[0]; idx = redi[0];
    for (int w = 1; w < SAMP_THREADS / 32; w++) {
        const float ov = redv[w];
        const int oi = redi[w];
        if (oi >= 0 && (idx < 0 || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
    }
}

__global__ void __launch_bounds__(SAMP_THREADS) ns_sample_rows_kernel(const float* __restrict__ logits, float* __restrict__ ids,
                                                                      float* __restrict__ stats, const float* __restrict__ step, int rows,
                                                                      int vocabulary, int rowStride, int rowOffset, float temperature, int topK,
                                                                      float topP, float minP, uint32_t seed)
{
    __shared__ float red[SAMP_THREADS / 32];
    __shared__ int redi[SAMP_THREADS / 32];
    __shared__ float seg_sum[SAMP_THREADS];
    __shared__ int s_chosen;
    const int tid = threadIdx.x;
    const uint32_t stepNumber = (uint32_t)step[0];
    const float invT = 1.0f / fmaxf(temperature, 1e-3f);
    // contiguous segment of the vocabulary per thread, so that prefix sums follow the index order
    const int seg = (vocabulary + SAMP_THREADS - 1) / SAMP_THREADS;
    const int j0 = min(tid * seg, vocabulary), j1 = min(j0 + seg, vocabulary);

    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* z = logits + (size_t)r * rowStride + rowOffset;
        float mx = -INFINITY;
        for (int j = tid; j < vocabulary; j += SAMP_THREADS) mx = fmaxf(mx, __fmul_rn(z[j], invT));
        const float max = block_max(mx, red);

        float threshold = -INFINITY;
        if (topK > 0 && topK < vocabulary) {
            threshold = INFINITY;
            for (int k = 0; k < topK; k++) {
                float next = -INFINITY;
                for (int j = tid; j < vocabulary; j += SAMP_THREADS) {
                    const float s = __fmul_rn(z[j], invT);
                    if (s < threshold && s > next) next = s;
                }
                threshold = block_max(next, red);
            }
        }
        if (minP > 0.0f) threshold = fmaxf(threshold, max + logf(minP));
        if (topP > 0.0f && topP < 1.0f) {
            float part = 0.0f;
            for (int j = tid; j < vocabulary; j += SAMP_THREADS) {
                const float s = __fmul_rn(z[j], invT);
                part += s >= threshold ? expf(s - max) : 0.0f;
            }
            const float total = block_sum(part, red);
            const float goal = total * topP;
            float lo = fmaxf(max - 40.0f, threshold), hi = max;
            for (int it = 0; it < 24; it++) {
                const float mid = (lo + hi) * 0.5f;
                float m = 0.0f;
                for (int j = tid; j < vocabulary; j += SAMP_THREADS) {
                    const float s = __fmul_rn(z[j], invT);
                    m += (s >= threshold && s >= mid) ? expf(s - max) : 0.0f;
                }
                const float mass = block_sum(m, red);
                if (mass >= goal) lo = mid; else hi = mid;
            }
            threshold = lo;
        }
        // e_j over this thread's segment, in index order
        float local = 0.0f;
        for (int j = j0; j < j1; j++) {
            const float s = __fmul_rn(z[j], invT);
            local += s >= threshold ? expf(s - max) : 0.0f;
        }
        seg_sum[tid] = local;
        const float sum = block_sum(local, red);   // also orders seg_sum for the reads below
        const float target = counter_uniform(seed, stepNumber, (uint32_t)r) * sum;
        // the first index whose running sum exceeds the target; the last kept index when none does
        float before = 0.0f;
        for (int t = 0; t < tid; t++) before += seg_sum[t];
        if (tid == 0) s_chosen = -1;
        __syncthreads();
        int cross = -1, last_kept = -1;
        {
            float cum = before;
            for (int j = j0; j < j1; j++) {
                const float s = __fmul_rn(z[j], invT);
                const float e = s >= threshold ? expf(s - max) : 0.0f;
                if (e > 0.0f) {
                    last_kept = j;
                    cum += e;
                    if (cum > target && cross < 0) cross = j;
                }
            }
        }
        // smallest crossing index over the block, else the largest kept index
        {
            float v = cross >= 0 ? -(float)cross : -INFINITY;   // larger value = smaller index
            int idx = cross;
            block_argmax(v, idx, red, redi);
            if (idx >= 0) {
                if (tid == 0) s_chosen = idx;
            } else {
                float v2 = last_kept >= 0 ? (float)last_kept : -INFINITY;
                int i2 = last_kept;
                block_argmax(v2, i2, red, redi);
                if (tid == 0) s_chosen = i2;
            }
        }
        __syncthreads();
        const int chosen = s_chosen;
        // entropy in bits
        float ent = 0.0f;
        for (int j = tid; j < vocabulary; j += SAMP_THREADS) {
            const float s = __fmul_rn(z[j], invT);
            if (s >= threshold) {
                const float e = expf(s - max);
                if (e > 0.0f) { const float pr = e / sum; ent = __fsub_rn(ent, __fmul_rn(pr, log2f(pr))); }
            }
        }
        const float entropy = block_sum(ent, red);
        const size_t o = ((size_t)stepNumber * rows + r) * 13;
        if (tid == 0) {
            ids[r] = (float)chosen;
            stats[o] = (float)chosen;
            const float sc = __fmul_rn(z[chosen], invT);
            stats[o + 1] = (sc >= threshold ? expf(sc - max) : 0.0f) / sum;
            stats[o + 2] = entropy;
        }
        // five most likely kept tokens, first maximum wins, none twice
        int taken[5] = {-1, -1, -1, -1, -1};
        for (int a = 0; a < 5; a++) {
            float bv = -INFINITY;
            int bi = -1;
            for (int j = tid; j < vocabulary; j += SAMP_THREADS) {
                const float s = __fmul_rn(z[j], invT);
                const float e = s >= threshold ? expf(s - max) : 0.0f;
                if (e > 0.0f && j != taken[0] && j != taken[1] && j != taken[2] && j != taken[3] && j != taken[4] &&
                    (bi < 0 || e > bv)) { bv = e; bi = j; }
            }
            block_argmax(bv, bi, red, redi);
            taken[a] = bi;
            if (tid == 0) {
                stats[o + 3 + 2 * a] = (float)bi;
                stats[o + 4 + 2 * a] = bi < 0 ? 0.0f : bv / sum;
            }
        }
        __syncthreads();
    }
}

// work[r, :] = logits row r, then the repetition penalties of the last min(length, lastN, capacity) history entries;
// each distinct token once.  One CTA per row: the copy is spread over the CTA, thread k owns history entry k.
__global__ void __launch_bounds__(SAMP_THREADS) ns_penalize_rows_kernel(const float* __restrict__ logits, float* __restrict__ work,
                                                                        const float* __restrict__ history, const float* __restrict__ length,
                                                                        int rows, int vocabulary, int rowStride, int rowOffset, int capacity,
                                                                        int lastN, float repeat, float presence, float frequency)
{
    const uint32_t len = (uint32_t)length[0];
    const uint32_t lim = (uint32_t)min(lastN, capacity);
    const int n = (int)min(len, lim);
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        float* w = work + (size_t)r * vocabulary;
        const float* z = logits + (size_t)r * rowStride + rowOffset;
        for (int j = threadIdx.x; j < vocabulary; j += SAMP_THREADS) w[j] = z[j];
        __syncthreads();
        const float* h = history + (size_t)r * capacity;
        for (int k = threadIdx.x; k < n; k += SAMP_THREADS) {
            const int id = (int)h[(len - 1 - (uint32_t)k) % (uint32_t)capacity];
            bool seen_more_recently = false;
            int count = 0;
            for (int q = 0; q < n; q++) {
                const int other = (int)h[(len - 1 - (uint32_t)q) % (uint32_t)capacity];
                if (other == id) { count++; seen_more_recently |= q < k; }
            }
            if (seen_more_recently || (unsigned)id >= (unsigned)vocabulary) continue;
            float x = w[id];   // distinct ids: no two threads touch the same element
            x = x > 0.0f ? x / repeat : x * repeat;
            w[id] = __fsub_rn(__fsub_rn(x, presence), __fmul_rn(frequency, (float)count));
        }
        __syncthreads();
    }
}

__global__ void ns_history_push_kernel(const float* __restrict__ ids, float* __restrict__ history, const float* __restrict__ length, int rows,
                                       int capacity)
{
    const uint32_t len = (uint32_t)length[0];
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x)
        history[(size_t)r * capacity + (len % (uint32_t)capacity)] = ids[r];
}

}  // namespace

#define NS_ENTER(h)                          \
    NsDevice* d = ns_dev(h);                 \
    {                                        \
        int _rc = ns_device_make_current(d); \
        if (_rc != NS_OK) return _rc;        \
    }

extern "C" int ns_f32_sample_rows(ns_device_t h, uint64_t logits, uint64_t ids, uint64_t stats, uint64_t step, int rows, int vocabulary,
                                  int rowStride, int rowOffset, float temperature, int topK, float topP, float minP, uint32_t seed)
{
    NS_ENTER(h);
    NS_REQUIRE(logits && ids && stats && step, NS_ERR_ARGUMENT, "ns_f32_sample_rows: null operand");
    NS_REQUIRE(rows >= 0 && vocabulary > 0 && rowStride >= 0 && rowOffset >= 0, NS_ERR_ARGUMENT, "ns_f32_sample_rows: bad shape");
    if (rows == 0) return NS_OK;
    const int grid = rows < d->sm_count * 8 ? rows : d->sm_count * 8;
    ns_sample_rows_kernel<<<grid, SAMP_THREADS, 0, d->stream>>>(reinterpret_cast<const float*>(logits), reinterpret_cast<float*>(ids),
                                                               reinterpret_cast<float*>(stats), reinterpret_cast<const float*>(step), rows, vocabulary,
                                                               rowStride, rowOffset, temperature, topK, topP, minP, seed);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_penalize_rows(ns_device_t h, uint64_t logits, uint64_t work, uint64_t history, uint64_t length, int rows, int vocabulary,
                                    int rowStride, int rowOffset, int capacity, int lastN, float repeat, float presence, float frequency)
{
    NS_ENTER(h);
    NS_REQUIRE(logits && work && history && length, NS_ERR_ARGUMENT, "ns_f32_penalize_rows: null operand");
    NS_REQUIRE(rows >= 0 && vocabulary > 0 && capacity > 0 && lastN >= 0, NS_ERR_ARGUMENT, "ns_f32_penalize_rows: bad shape");
    if (rows == 0) return NS_OK;
    const int grid = rows < d->sm_count * 8 ? rows : d->sm_count * 8;
    ns_penalize_rows_kernel<<<grid, SAMP_THREADS, 0, d->stream>>>(reinterpret_cast<const float*>(logits), reinterpret_cast<float*>(work),
                                                                 reinterpret_cast<const float*>(history), reinterpret_cast<const float*>(length), rows,
                                                                 vocabulary, rowStride, rowOffset, capacity, lastN, repeat, presence, frequency);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}

extern "C" int ns_f32_history_push(ns_device_t h, uint64_t ids, uint64_t history, uint64_t length, int rows, int capacity)
{
    NS_ENTER(h);
    NS_REQUIRE(ids && history && length && rows >= 0 && capacity > 0, NS_ERR_ARGUMENT, "ns_f32_history_push: bad argument");
    if (rows == 0) return NS_OK;
    ns_history_push_kernel<<<(rows + 127) / 128, 128, 0, d->stream>>>(reinterpret_cast<const float*>(ids), reinterpret_cast<float*>(history),
                                                                     reinterpret_cast<const float*>(length), rows, capacity);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}
