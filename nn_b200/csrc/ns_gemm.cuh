// Interface of the tensor-core product shared by ns_qmatmul_i8, ns_matmul_bf16 and the Linear objects.
#pragma once

#include "ns_common.cuh"
#include "ns_tail.cuh"

enum { NS_KIND_I8 = 0, NS_KIND_BF16 = 1 };

struct NsGemmParams {
    int M, N, K;        // K in elements
    int k_blocks;       // ceil(K * elsize / 128)
    int k_splits;       // >= 1
    int kb_per_split;   // k-blocks per split
    int tiles_m, tiles_n;
    int a_rows;         // rows of A fetched per tile (64 when M <= 64, else 128)
    int epilogue;       // NS_EPI_*
    int out_dtype;      // NS_F32 / NS_BF16
    int residual_dtype;
    int vec_cols;       // 1: w_scale and bias are 16-byte aligned (vector loads in the epilogue)
    int tma_store;      // 1: outputs leave through shared memory and TMA stores; 0: direct stores (odd N)
    int prefetch_b;     // 1: B is a weight no kernel on the stream writes (Linear objects): its first tiles may be
                        //    requested before the previous kernel has finished; 0: every load waits for that kernel
    void* out;          // [M, N] or null
    int32_t* raw;       // optional exact accumulators (int8 kind only)
    const float* a_scale;
    const float* w_scale;
    const float* bias;
    const void* residual;
    void* partial;      // [k_splits, M, N] 32-bit words when k_splits > 1
    // CTA-pair kernel with its tiles' k-blocks dealt out evenly to the clusters (see ns_gemm_pair_kernel): total k-block
    // units = tiles * k_blocks; a tile that straddles two clusters leaves one part's accumulators in sk_work
    // [clusters, 256, 256] 32-bit words and a count of finished epilogue warps in sk_flags [clusters]
    int streamk;
    uint32_t* sk_work;
    uint32_t* sk_flags;
    int* status;
    int status_base;    // code = status_base + role
};

// Fills the shape-derived fields of `p`, builds the tensor maps and launches on d->stream.
// a: [M, K]; b: [N, K] (b_is_kn = false) or [K, N] (b_is_kn = true, bf16 only).
// partial_override: when non-null, split-K partial sums go there (it must hold
// k_splits * M * N 32-bit words) instead of the device object's scratch block.
// deferred_partial / deferred_splits: when non-null (int8 kind only) the epilogue is left to a later kernel: exact
// int32 partial sums [splits, M, N] stay in the device object's scratch block (one slab when K is not split) and the
// two out-parameters describe them; no second kernel is launched.
// tail: when non-null (int8 kind, [N, K] weights, M <= NS_TAIL_MAX_ROWS) the launch continues with the row operator
// the struct describes (ns_tail.cuh).  For NS_TAIL_PEER the product writes its float partial rows to p.out (K is not
// split); for the other kinds the epilogue is deferred as above and the launcher fills tail->partial / tail->splits.
int ns_gemm_run(NsDevice* d, int kind, const void* a, const void* b, bool b_is_kn, int M, int N, int K, NsGemmParams p,
                void* partial_override = nullptr, size_t partial_override_bytes = 0, void** deferred_partial = nullptr,
                int* deferred_splits = nullptr, NsTail* tail = nullptr);
constexpr int NS_TAIL_MAX_ROWS = 256;

// The row-streaming int8 kernel for 1..8 activation rows (ns_gemv_i8.cu).  `p` must hold M, N, K, the epilogue
// fields, out / raw and the scale, bias and residual pointers.
bool ns_gemv_i8_fits(int M, int K);
int ns_gemv_i8_run(NsDevice* d, const NsGemmParams& p, const void* a, const void* w);
// The streaming int8 kernel for 9..64 activation rows (ns_stream_i8.cu): one launch, K summed inside the CTA.  Same fields of `p`.
bool ns_stream_i8_fits(int M, int K);
int ns_stream_i8_run(NsDevice* d, const NsGemmParams& p, const void* a, const void* w);

#ifdef __CUDACC__
__device__ __forceinline__ float ns_gemm_residual(const NsGemmParams& p, size_t idx)
{
    if (p.residual_dtype == NS_BF16) return ns_bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p.residual)[idx]);
    return reinterpret_cast<const float*>(p.residual)[idx];
}

// exact int32 sum -> output value (without the residual): ((float)acc * a_scale) * w_scale (+ bias (, GELU))
__device__ __forceinline__ float ns_gemm_finish_i8(const NsGemmParams& p, int32_t acc, float a_scale, float w_scale, float bias)
{
    float v = __int2float_rn(acc);
    v = __fmul_rn(v, a_scale);
    v = __fmul_rn(v, w_scale);
    if (p.epilogue != NS_EPI_NONE) v = __fadd_rn(v, bias);
    if (p.epilogue == NS_EPI_BIAS_GELU) v = ns_gelu_fast(v);
    return v;
}
#endif

// Tile width / split count the launcher would pick for a shape (also used to size scratch memory).
void ns_gemm_choose_tiling(const NsDevice* d, int M, int N, int k_blocks, int* tile_n, int* k_splits, bool b_is_kn = false);
