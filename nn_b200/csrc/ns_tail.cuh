// Second phase of a decode-step product: the row operator that follows a Linear, run by the SAME kernel launch.
//
// With the few rows of a decoding step every launch costs a few microseconds before its first useful byte, and a step
// is a chain of some ten dependent launches per layer.  The product kernel (ns_gemm_tc.cu) therefore ends with a second
// phase: every CTA leaves its exact int32 partial sums in the scratch block, arrives on a device-wide counter, and the
// CTAs that own rows wait for the counter and run the row operator -- the one the reference runs as separate kernels
// after matmul_f32 (src/NeuralSharp/Layers/Attention.cs:201-211: add_rowvec_f32, add_f32, layernorm_fused_f32,
// bias_gelu_f32, kv_write_f32; Backends/Cuda/PtxKernels.Decoding.cs:61-143).  Kinds:
//   NS_TAIL_KV    fused QKV product: dequantise + bias -> bf16 [rows, 3 d], K and V thirds appended to the paged cache
//   NS_TAIL_NORM  out-projection / FF2: dequantise + bias + residual -> bf16 stream -> LayerNorm -> int8 rows
//   NS_TAIL_GELU  FF1: dequantise + bias + GELU -> bf16 -> int8 rows
//   NS_TAIL_PEER  row-parallel shard on several GPUs: the product's float partial rows are in this rank's peer slot;
//                 the ranks' rows are summed over NVLink, then bias + residual + LayerNorm + int8 rows (ns_peer.cu)
// The arithmetic of each is, operation for operation, that of the separate kernels (ns_step_fused.cu, ns_glue.cu,
// ns_peer.cu), so results are bit-identical to the unfused sequence.
//
// All CTAs of the grid are resident at once (one per SM, grid <= SM count), which the waits below rely on; every
// wait is bounded and reports through the device status word.
#pragma once

#include "ns_common.cuh"
#include "ns_rows.cuh"

enum { NS_TAIL_NONE = 0, NS_TAIL_KV = 1, NS_TAIL_NORM = 2, NS_TAIL_GELU = 3, NS_TAIL_PEER = 4 };
constexpr int NS_TAIL_THREADS = 256;
constexpr int NS_TAIL_PEER_MAX = 8;

struct NsTail {
    int kind;
    int vpt, active;          // row shape of NORM / GELU / PEER: `active` threads hold vpt vectors of 8 columns each
    uint32_t* sync;           // [0] arrivals of this launch, [1] departures; both zero between launches
    int* status;
    // the product's exact partial sums (filled in by the launcher)
    const int32_t* partial;
    int splits;
    const float* x_scale;     // per row, of the product's int8 input
    const float* w_scale;     // per column
    const float* bias;        // per column or null
    int64_t rows;
    int cols;
    // NORM / PEER / GELU
    const uint16_t* residual; // bf16 [rows, cols] or null
    uint16_t* x_out;          // bf16 [rows, cols]
    const float* gamma;       // null: no LayerNorm / quantisation
    const float* beta;
    float eps;
    int8_t* q;
    float* q_scale;
    // KV
    int batch, steps, d_loc;
    uint16_t* qkv;
    uint16_t* k_pool;
    uint16_t* v_pool;
    const int32_t* page_table;
    int max_pages, page_size, heads, dh, num_pages;
    const int32_t* pos_dev;
    // PEER
    const float* part[NS_TAIL_PEER_MAX];
    uint32_t* remote_flag[NS_TAIL_PEER_MAX];
    const uint32_t* local_flags;
    uint32_t* epoch;
    int rank, world;
    // test hook: when non-null, CTA b writes the time (ns) of four points of its second phase to times[4 b ..]
    unsigned long long* times;
};

// The device code is compiled into the one source file that defines NS_TAIL_DEVICE_CODE before including this header
// (ns_gemm_tc.cu); the others only need the struct.
#if defined(__CUDACC__) && defined(NS_TAIL_DEVICE_CODE)
namespace ns_tail {

__device__ __forceinline__ void stamp(const NsTail& t, int slot)
{
    if (t.times != nullptr && threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        t.times[4 * blockIdx.x + slot] = now;
    }
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Every thread of the CTA calls this after its own writes of the first phase are complete.  The CTA arrives on
// sync[0]; when `waits`, it then waits (bounded) until all gridDim.x CTAs have arrived.  Returns false when the wait
// was given up (status code written).
__device__ __forceinline__ bool arrive_and_wait(uint32_t* sync, bool waits, int* status, int code, int* flag_smem)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(&sync[0], 1u);
        int ok = 1;
        if (waits) {
            const long long t0 = clock64();
            while (ld_acquire_gpu(&sync[0]) < gridDim.x) {
                if (clock64() - t0 > NS_WAIT_LIMIT_CYCLES) {
                    *reinterpret_cast<volatile int*>(status) = code;
                    ok = 0;
                    break;
                }
                __nanosleep(20);
            }
            __threadfence();
        }
        *flag_smem = ok;
    }
    __syncthreads();
    return *flag_smem != 0;
}

// The CTAs that waited leave through here; the last of `waiters` clears the two words for the next launch.
__device__ __forceinline__ void depart(uint32_t* sync, unsigned waiters)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(&sync[1], 1u);
        if (t == waiters - 1) {
            sync[1] = 0u;
            sync[0] = 0u;
            __threadfence();
        }
    }
}

// first column of vector j of this thread (threads >= active hold nothing)
__device__ __forceinline__ int vec_col(int j, int active) { return (j * active + (int)threadIdx.x) * 8; }

// Block reduction over all NS_TAIL_THREADS threads; threads outside the active range contribute the identity (0), so
// the value equals the reduction of a CTA of `active` threads (ns_rows::block_reduce): x + 0 and max(x, 0) are exact.
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < NS_TAIL_THREADS / 32; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// ns_rows::block_sum_pieces over all NS_TAIL_THREADS threads: the pieces of the warps outside the active range are zero, and
// adding zero is exact, so the value is the one a CTA of `active` threads gets.
template <int VPT>
__device__ __forceinline__ float block_sum_pieces(const float (&part)[VPT], int active, float* red)
{
    const int warps = active >> 5, warp = threadIdx.x >> 5;
    float t[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        float v = part[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        t[j] = v;
    }
    if ((threadIdx.x & 31) == 0 && warp < warps) {
#pragma unroll
        for (int j = 0; j < VPT; j++) red[j * warps + warp] = t[j];
    }
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < VPT * warps; w++) r += red[w];
    return r;
}

template <int VPT>
__device__ __forceinline__ void quantize_row(const float (&x)[VPT * 8], bool on, int active, int8_t* __restrict__ q_row, float* __restrict__ scale_out,
                                             float* red)
{
    float amax = 0.0f;
    if (on) {
#pragma unroll
        for (int i = 0; i < VPT * 8; i++) amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = block_reduce(amax, true, red);
    const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) *scale_out = sc;
    if (!on) return;
    const float rcp = __frcp_rn(sc);
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        uint32_t lo, hi;
        ns_rows::quant8<true>(x + j * 8, sc, rcp, lo, hi);
        *reinterpret_cast<uint2*>(q_row + vec_col(j, active)) = make_uint2(lo, hi);
    }
}

// ns_rows::layernorm_quantize_row for `active` of the CTA's threads.
template <int VPT>
__device__ __forceinline__ void layernorm_quantize_row(float (&x)[VPT * 8], bool on, int active, const float* __restrict__ gamma,
                                                       const float* __restrict__ beta, float eps, int cols, int8_t* __restrict__ q_row,
                                                       float* __restrict__ scale_out, ns_rows::RowShared& sh)
{
    float4 g[VPT][2], b[VPT][2];
    if (on) {
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const int col = vec_col(j, active);
            g[j][0] = __ldg(reinterpret_cast<const float4*>(gamma + col)); g[j][1] = __ldg(reinterpret_cast<const float4*>(gamma + col + 4));
            b[j][0] = __ldg(reinterpret_cast<const float4*>(beta + col)); b[j][1] = __ldg(reinterpret_cast<const float4*>(beta + col + 4));
        }
    }
    float part[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        float s = 0.0f;
        if (on) {
#pragma unroll
            for (int i = 0; i < 8; i++) s += x[j * 8 + i];
        }
        part[j] = s;
    }
    const float mean = block_sum_pieces<VPT>(part, active, sh.red[0]) / (float)cols;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        float v2 = 0.0f;
        if (on) {
#pragma unroll
            for (int i = 0; i < 8; i++) { const float d = x[j * 8 + i] - mean; v2 = fmaf(d, d, v2); }
        }
        part[j] = v2;
    }
    const float inv = 1.0f / sqrtf(block_sum_pieces<VPT>(part, active, sh.red[1]) / (float)cols + eps);
    if (on) {
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
    }
    quantize_row<VPT>(x, on, active, q_row, scale_out, sh.red[2]);
}

// exact sum of the splits' accumulators of 8 consecutive columns, read past L1 (other SMs wrote them in this launch)
__device__ __forceinline__ void sum_splits8(const int32_t* __restrict__ partial, int splits, size_t slab, size_t idx, int32_t (&acc)[8])
{
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0;
    for (int sp = 0; sp < splits; sp++) {
        const int4* src = reinterpret_cast<const int4*>(partial + (size_t)sp * slab + idx);
        const int4 a = __ldcg(src), b = __ldcg(src + 1);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
}

// dequantised value of 8 columns: ((float)acc * a_scale) * w_scale (+ bias), each step rounded to float
__device__ __forceinline__ void dequant8(const NsTail& t, const int32_t (&acc)[8], float a_scale, int col, float (&v)[8])
{
    const float4 w0 = __ldg(reinterpret_cast<const float4*>(t.w_scale + col)), w1 = __ldg(reinterpret_cast<const float4*>(t.w_scale + col + 4));
    const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fmul_rn(__fmul_rn(__int2float_rn(acc[i]), a_scale), ws[i]);
    if (t.bias != nullptr) {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(t.bias + col)), b1 = __ldg(reinterpret_cast<const float4*>(t.bias + col + 4));
        const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fadd_rn(v[i], bs[i]);
    }
}

// ---- NS_TAIL_NORM: ns_finish_norm_quant_reg_kernel's row pass
template <int VPT>
__device__ __forceinline__ void norm_rows(const NsTail& t, ns_rows::RowShared& sh)
{
    const bool on = (int)threadIdx.x < t.active;
    const size_t slab = (size_t)t.rows * t.cols;
    for (int64_t r = blockIdx.x; r < t.rows; r += gridDim.x) {
        const float a_scale = t.x_scale[r];
        float v[VPT * 8];
        if (on) {
#pragma unroll
            for (int j = 0; j < VPT; j++) {
                const int col = vec_col(j, t.active);
                const size_t idx = (size_t)r * t.cols + col;
                int32_t acc[8];
                sum_splits8(t.partial, t.splits, slab, idx, acc);
                float f[8];
                dequant8(t, acc, a_scale, col, f);
                if (t.residual != nullptr) {
                    float rs[8];
                    ns_rows::widen8(*reinterpret_cast<const uint4*>(t.residual + idx), rs);
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = __fadd_rn(f[i], rs[i]);
                }
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; i++) w[i] = uint32_t(ns_f32_to_bf16_bits(f[2 * i])) | (uint32_t(ns_f32_to_bf16_bits(f[2 * i + 1])) << 16);
                const uint4 packed = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(t.x_out + idx) = packed;
                float xr[8];
                ns_rows::widen8(packed, xr);
#pragma unroll
                for (int i = 0; i < 8; i++) v[j * 8 + i] = xr[i];
            }
        }
        // every thread has read x_scale[r] before the barriers of the reductions below, so q_scale may be the same array
        if (t.gamma != nullptr)
            layernorm_quantize_row<VPT>(v, on, t.active, t.gamma, t.beta, t.eps, t.cols, t.q + (size_t)r * t.cols, t.q_scale + r, sh);
    }
}

// ---- NS_TAIL_GELU: the product's bias + GELU epilogue (bf16 output) followed by ns_quantize_rows_i8
template <int VPT>
__device__ __forceinline__ void gelu_rows(const NsTail& t, ns_rows::RowShared& sh)
{
    const bool on = (int)threadIdx.x < t.active;
    const size_t slab = (size_t)t.rows * t.cols;
    for (int64_t r = blockIdx.x; r < t.rows; r += gridDim.x) {
        const float a_scale = t.x_scale[r];
        float v[VPT * 8];
        if (on) {
#pragma unroll
            for (int j = 0; j < VPT; j++) {
                const int col = vec_col(j, t.active);
                const size_t idx = (size_t)r * t.cols + col;
                int32_t acc[8];
                sum_splits8(t.partial, t.splits, slab, idx, acc);
                float f[8];
                dequant8(t, acc, a_scale, col, f);
#pragma unroll
                for (int i = 0; i < 8; i++) v[j * 8 + i] = ns_bf16_bits_to_f32(ns_f32_to_bf16_bits(ns_gelu_fast(f[i])));
            }
        }
        __syncthreads();   // x_scale[r] has been read by every thread before thread 0 overwrites it (q_scale may be the same array)
        quantize_row<VPT>(v, on, t.active, t.q + (size_t)r * t.cols, t.q_scale + r, sh.red[0]);
        __syncthreads();   // red[0] is reused by the next row
    }
}

// ---- NS_TAIL_KV: ns_finish_kv_append_kernel's pass, all CTAs of the grid
__device__ __forceinline__ void kv_rows(const NsTail& t)
{
    const int cols = 3 * t.d_loc;
    const int groups = cols / 8;
    const int64_t rows = (int64_t)t.batch * t.steps;
    const size_t slab = (size_t)rows * cols;
    const int pos0 = t.pos_dev[0];
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < rows * groups; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = e / groups;
        const int col0 = (int)(e % groups) * 8;
        const size_t idx0 = (size_t)row * cols + col0;
        const float a_scale = t.x_scale[row];
        int32_t acc[8];
        sum_splits8(t.partial, t.splits, slab, idx0, acc);
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float v0 = __fmul_rn(__fmul_rn(__int2float_rn(acc[2 * j]), a_scale), t.w_scale[col0 + 2 * j]);
            float v1 = __fmul_rn(__fmul_rn(__int2float_rn(acc[2 * j + 1]), a_scale), t.w_scale[col0 + 2 * j + 1]);
            if (t.bias != nullptr) { v0 = __fadd_rn(v0, t.bias[col0 + 2 * j]); v1 = __fadd_rn(v1, t.bias[col0 + 2 * j + 1]); }
            w[j] = uint32_t(ns_f32_to_bf16_bits(v0)) | (uint32_t(ns_f32_to_bf16_bits(v1)) << 16);
        }
        const uint4 out = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(t.qkv + idx0) = out;
        const int third = col0 / t.d_loc;          // 0 = Q, 1 = K, 2 = V
        if (third == 0) continue;
        const int in_third = col0 - third * t.d_loc;
        const int h = in_third / t.dh, c = in_third % t.dh;
        const int i = (int)(row % t.steps), b = (int)(row / t.steps);
        const int pos = pos0 + i;
        if (pos < 0 || pos / t.page_size >= t.max_pages) { *reinterpret_cast<volatile int*>(t.status) = 500; continue; }
        const int page = t.page_table[(size_t)b * t.max_pages + pos / t.page_size];
        if (page < 0 || page >= t.num_pages) { *reinterpret_cast<volatile int*>(t.status) = 500; continue; }
        const size_t dst = (((size_t)page * t.heads + h) * t.page_size + pos % t.page_size) * t.dh + c;
        *reinterpret_cast<uint4*>((third == 1 ? t.k_pool : t.v_pool) + dst) = out;
    }
}

__device__ __forceinline__ float4 peer_load4(const float* ptr)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr) : "memory");
    return v;
}

// ---- NS_TAIL_PEER: ns_tp_reduce_norm_quant_kernel's pass.  `e` is the epoch this exchange carries.
template <int VPT>
__device__ __forceinline__ void peer_rows(const NsTail& t, ns_rows::RowShared& sh)
{
    const bool on = (int)threadIdx.x < t.active;
    for (int64_t r = blockIdx.x; r < t.rows; r += gridDim.x) {
        float v[VPT * 8];
        if (on) {
#pragma unroll
            for (int j = 0; j < VPT; j++) {
                const int col = vec_col(j, t.active);
                const size_t idx = (size_t)r * t.cols + col;
                // every rank's vectors are requested before the first is used: one NVLink round trip, not one per rank
                float4 va[NS_TAIL_PEER_MAX], vb[NS_TAIL_PEER_MAX];
#pragma unroll
                for (int k = 0; k < NS_TAIL_PEER_MAX; k++) {
                    if (k < t.world) {
                        va[k] = peer_load4(t.part[k] + idx);
                        vb[k] = peer_load4(t.part[k] + idx + 4);
                    }
                }
                float f[8] = {va[0].x, va[0].y, va[0].z, va[0].w, vb[0].x, vb[0].y, vb[0].z, vb[0].w};
#pragma unroll
                for (int k = 1; k < NS_TAIL_PEER_MAX; k++) {
                    if (k < t.world) {
                        f[0] = __fadd_rn(f[0], va[k].x); f[1] = __fadd_rn(f[1], va[k].y); f[2] = __fadd_rn(f[2], va[k].z); f[3] = __fadd_rn(f[3], va[k].w);
                        f[4] = __fadd_rn(f[4], vb[k].x); f[5] = __fadd_rn(f[5], vb[k].y); f[6] = __fadd_rn(f[6], vb[k].z); f[7] = __fadd_rn(f[7], vb[k].w);
                    }
                }
                if (t.bias != nullptr) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(t.bias + col)), b1 = __ldg(reinterpret_cast<const float4*>(t.bias + col + 4));
                    const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = __fadd_rn(f[i], bs[i]);
                }
                if (t.residual != nullptr) {
                    float rs[8];
                    ns_rows::widen8(*reinterpret_cast<const uint4*>(t.residual + idx), rs);
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = __fadd_rn(f[i], rs[i]);
                }
                const uint4 packed = make_uint4(ns_pack_bf16x2(f[0], f[1]), ns_pack_bf16x2(f[2], f[3]), ns_pack_bf16x2(f[4], f[5]), ns_pack_bf16x2(f[6], f[7]));
                *reinterpret_cast<uint4*>(t.x_out + idx) = packed;
                float xr[8];
                ns_rows::widen8(packed, xr);
#pragma unroll
                for (int i = 0; i < 8; i++) v[j * 8 + i] = xr[i];
            }
        }
        if (t.gamma != nullptr)
            layernorm_quantize_row<VPT>(v, on, t.active, t.gamma, t.beta, t.eps, t.cols, t.q + (size_t)r * t.cols, t.q_scale + r, sh);
        __syncthreads();
    }
}

// The second phase.  Called by all NS_TAIL_THREADS threads of every CTA after the product's own teardown, when the stores
// each thread queued in the first phase are complete.
__device__ __noinline__ void run(const NsTail& t)
{
    __shared__ ns_rows::RowShared sh;
    __shared__ int flag, flag2;
    ns_pdl_wait();   // every thread, before it reads what the kernel before this launch wrote (residual, row scales)
    if (t.kind == NS_TAIL_PEER) {
        // Every CTA arrives; CTA 0 waits for all arrivals (this rank's partial rows are then complete in its slot) and
        // tells every rank, itself included, by storing the epoch into their flag words; CTAs that own rows wait for
        // every rank's flag.  The last CTA through advances the epoch and clears the counters.
        const uint32_t e = *reinterpret_cast<volatile uint32_t*>(t.epoch) + 1u;
        const bool ok0 = arrive_and_wait(t.sync, blockIdx.x == 0, t.status, 410, &flag);
        if (blockIdx.x == 0 && (int)threadIdx.x < t.world && ok0) {
            __threadfence_system();
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(t.remote_flag[threadIdx.x]), "r"(e) : "memory");
        }
        const bool has_rows = (int64_t)blockIdx.x < t.rows;
        if (threadIdx.x == 0) flag2 = 1;
        __syncthreads();
        if (has_rows && (int)threadIdx.x < t.world) {
            const long long t0 = clock64();
            uint32_t seen = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(t.local_flags + threadIdx.x) : "memory");
                if ((int32_t)(seen - e) >= 0) break;
                if (clock64() - t0 > NS_WAIT_LIMIT_CYCLES) {
                    *reinterpret_cast<volatile int*>(t.status) = 400 + (int)threadIdx.x;
                    flag2 = 0;
                    break;
                }
                __nanosleep(32);
            }
        }
        __syncthreads();
        if (has_rows && flag2 != 0) {
            switch (t.vpt) {
                case 1: peer_rows<1>(t, sh); break;
                case 2: peer_rows<2>(t, sh); break;
                default: peer_rows<4>(t, sh); break;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t ticket = atomicAdd(&t.sync[1], 1u);
            if (ticket == gridDim.x - 1) {
                // every CTA has arrived and left: the epoch advances whether or not a wait ran out, so the ranks stay in step
                t.sync[1] = 0u;
                t.sync[0] = 0u;
                __threadfence();
                *reinterpret_cast<volatile uint32_t*>(t.epoch) = e;
            }
        }
        return;
    }
    const bool all_wait = t.kind == NS_TAIL_KV;
    const bool waits = all_wait || (int64_t)blockIdx.x < t.rows;
    const unsigned waiters = all_wait ? gridDim.x : (unsigned)(t.rows < (int64_t)gridDim.x ? t.rows : (int64_t)gridDim.x);
    stamp(t, 1);
    const bool ok = arrive_and_wait(t.sync, waits, t.status, 420 + t.kind, &flag);
    stamp(t, 2);
    if (!waits) return;
    if (ok) {
        if (t.kind == NS_TAIL_KV) {
            kv_rows(t);
        } else if (t.kind == NS_TAIL_NORM) {
            switch (t.vpt) {
                case 1: norm_rows<1>(t, sh); break;
                case 2: norm_rows<2>(t, sh); break;
                default: norm_rows<4>(t, sh); break;
            }
        } else {
            switch (t.vpt) {
                case 1: gelu_rows<1>(t, sh); break;
                case 2: gelu_rows<2>(t, sh); break;
                default: gelu_rows<4>(t, sh); break;
            }
        }
    }
    stamp(t, 3);
    depart(t.sync, waiters);
}

}  // namespace ns_tail
#endif  // __CUDACC__ && NS_TAIL_DEVICE_CODE
