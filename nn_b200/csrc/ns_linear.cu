// Linear objects: device-resident weights of one Linear layer prepared for the tensor-core products,
// optionally one tensor-parallel shard of it.
//
// Reference: Linear (src/NeuralSharp/Layers/Linear.cs:25-47) keeps Weight as float [in, out] = [K, N] and
// Bias as float [N], computes x . W with matmul_f32 and adds the bias with a second kernel.  Here the
// weight is transposed once to [N, K] (one row per output channel), converted to bf16 or quantised to
// int8 with one scale per output channel, and the bias / GELU / residual are applied in the product's
// epilogue.  The reference has no tensor parallelism; the column / row split follows the usual
// scheme: a column shard owns a slice of the outputs (and of the bias), a row shard owns a slice of
// the inputs and produces a partial sum that the caller reduces across ranks.
#include <stdlib.h>
#include <string.h>

#include "ns_gemm.cuh"

struct NsLinear {
    int ordinal;
    int mode;        // NS_BF16 or NS_I8
    int K, N;        // full layer
    int K_loc, N_loc;
    int split, tp_rank, tp_size;
    void* w;         // [N_loc, K_loc] bf16 or int8
    float* w_scale;  // [N_loc] (int8 mode)
    float* bias;     // [N_loc] or null
};

extern "C" int ns_linear_create(ns_device_t h, int K, int N, int mode, const float* w_kn, const float* bias, int split, int col_groups,
                                int tp_rank, int tp_size, ns_linear_t* out)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(out && w_kn, NS_ERR_ARGUMENT, "ns_linear_create: null argument");
    NS_REQUIRE(mode == NS_BF16 || mode == NS_I8, NS_ERR_ARGUMENT, "ns_linear_create: mode must be NS_BF16 or NS_I8");
    NS_REQUIRE(split >= NS_SPLIT_NONE && split <= NS_SPLIT_ROW, NS_ERR_ARGUMENT, "ns_linear_create: unknown split %d", split);
    NS_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, NS_ERR_ARGUMENT, "ns_linear_create: bad rank %d of %d", tp_rank, tp_size);
    NS_REQUIRE(K > 0 && N > 0 && col_groups >= 1, NS_ERR_ARGUMENT, "ns_linear_create: bad shape");
    NS_REQUIRE(!d->capturing, NS_ERR_STATE, "ns_linear_create: not allowed while the stream is being captured");
    if (split == NS_SPLIT_NONE) { tp_rank = 0; tp_size = 1; }
    int K_loc = K, N_loc = N;
    if (split == NS_SPLIT_COLUMN) {
        NS_REQUIRE(N % (col_groups * tp_size) == 0, NS_ERR_ARGUMENT, "ns_linear_create: N=%d does not split into %d groups x %d ranks", N, col_groups, tp_size);
        N_loc = N / tp_size;
    } else if (split == NS_SPLIT_ROW) {
        NS_REQUIRE(K % tp_size == 0, NS_ERR_ARGUMENT, "ns_linear_create: K=%d does not split into %d ranks", K, tp_size);
        K_loc = K / tp_size;
    }
    NS_REQUIRE((K_loc * (mode == NS_I8 ? 1 : 2)) % 16 == 0, NS_ERR_ARGUMENT, "ns_linear_create: local K=%d gives rows that are not multiples of 16 bytes", K_loc);

    // local slice, transposed to [N_loc, K_loc], on the host
    std::vector<float> wt((size_t)N_loc * K_loc);
    std::vector<float> bl(bias ? N_loc : 0);
    const int group_full = N / col_groups;         // columns per group of the full layer
    const int group_loc = N_loc / col_groups;      // columns per group of this shard (column split)
    auto src_col = [&](int n) {
        if (split != NS_SPLIT_COLUMN) return n;
        const int g = n / group_loc, c = n % group_loc;
        return g * group_full + tp_rank * group_loc + c;
    };
    const int k0 = split == NS_SPLIT_ROW ? tp_rank * K_loc : 0;
    // blocked transpose: both arrays are walked in 32 x 32 tiles so neither side strides through memory
    for (int nb = 0; nb < N_loc; nb += 32)
        for (int kb = 0; kb < K_loc; kb += 32)
            for (int n = nb; n < N_loc && n < nb + 32; n++) {
                const int sn = src_col(n);
                for (int k = kb; k < K_loc && k < kb + 32; k++) wt[(size_t)n * K_loc + k] = w_kn[(size_t)(k0 + k) * N + sn];
            }
    if (bias)
        for (int n = 0; n < N_loc; n++) bl[n] = bias[src_col(n)];

    NsLinear* L = new NsLinear();
    memset(L, 0, sizeof(*L));
    L->ordinal = d->ordinal; L->mode = mode; L->K = K; L->N = N; L->K_loc = K_loc; L->N_loc = N_loc;
    L->split = split; L->tp_rank = tp_rank; L->tp_size = tp_size;
    float* staging = nullptr;
    const size_t n_el = (size_t)N_loc * K_loc;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&staging), n_el * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&L->w, n_el * (mode == NS_I8 ? 1 : 2));
    if (e == cudaSuccess && mode == NS_I8) e = cudaMalloc(reinterpret_cast<void**>(&L->w_scale), N_loc * sizeof(float));
    if (e == cudaSuccess && bias) e = cudaMalloc(reinterpret_cast<void**>(&L->bias), N_loc * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpyAsync(staging, wt.data(), n_el * sizeof(float), cudaMemcpyHostToDevice, d->stream);
    if (e == cudaSuccess && bias) e = cudaMemcpyAsync(L->bias, bl.data(), N_loc * sizeof(float), cudaMemcpyHostToDevice, d->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (staging) cudaFree(staging);
        if (L->w) cudaFree(L->w);
        if (L->w_scale) cudaFree(L->w_scale);
        if (L->bias) cudaFree(L->bias);
        delete L;
        return ns_fail(NS_ERR_MEMORY, "ns_linear_create: %s (%d)", cudaGetErrorName(e), (int)e);
    }
    if (mode == NS_I8)
        rc = ns_quantize_rows_i8(h, reinterpret_cast<uint64_t>(staging), NS_F32, N_loc, K_loc, reinterpret_cast<uint64_t>(L->w),
                                 reinterpret_cast<uint64_t>(L->w_scale));
    else
        rc = ns_convert(h, reinterpret_cast<uint64_t>(staging), NS_F32, reinterpret_cast<uint64_t>(L->w), NS_BF16, (int64_t)n_el);
    cudaStreamSynchronize(d->stream);
    cudaFree(staging);
    if (rc != NS_OK) { ns_linear_destroy(reinterpret_cast<ns_linear_t>(L)); return rc; }
    *out = reinterpret_cast<ns_linear_t>(L);
    return NS_OK;
}

extern "C" int ns_linear_destroy(ns_linear_t lh)
{
    NsLinear* L = reinterpret_cast<NsLinear*>(lh);
    if (!L) return NS_OK;
    cudaSetDevice(L->ordinal);
    if (L->w) cudaFree(L->w);
    if (L->w_scale) cudaFree(L->w_scale);
    if (L->bias) cudaFree(L->bias);
    delete L;
    return NS_OK;
}

extern "C" int ns_linear_info(ns_linear_t lh, int* k_local, int* n_local, int* mode, uint64_t* w, uint64_t* w_scale, uint64_t* bias)
{
    NsLinear* L = reinterpret_cast<NsLinear*>(lh);
    NS_REQUIRE(L != nullptr, NS_ERR_ARGUMENT, "ns_linear_info: linear is null");
    if (k_local) *k_local = L->K_loc;
    if (n_local) *n_local = L->N_loc;
    if (mode) *mode = L->mode;
    if (w) *w = reinterpret_cast<uint64_t>(L->w);
    if (w_scale) *w_scale = reinterpret_cast<uint64_t>(L->w_scale);
    if (bias) *bias = reinterpret_cast<uint64_t>(L->bias);
    return NS_OK;
}

extern "C" int ns_linear_forward(ns_device_t h, ns_linear_t lh, uint64_t x, uint64_t x_scale, int M, int epilogue, uint64_t residual,
                                 int residual_dtype, int out_dtype, uint64_t y)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsLinear* L = reinterpret_cast<NsLinear*>(lh);
    NS_REQUIRE(L && x && y, NS_ERR_ARGUMENT, "ns_linear_forward: null argument");
    NS_REQUIRE(L->mode != NS_I8 || x_scale != 0, NS_ERR_ARGUMENT, "ns_linear_forward: an int8 layer needs the row scales of its input");
    NS_REQUIRE(epilogue >= NS_EPI_NONE && epilogue <= NS_EPI_BIAS_RESIDUAL, NS_ERR_ARGUMENT, "ns_linear_forward: unknown epilogue %d", epilogue);
    NS_REQUIRE(epilogue == NS_EPI_NONE || L->bias != nullptr, NS_ERR_ARGUMENT, "ns_linear_forward: the layer has no bias for epilogue %d", epilogue);
    NS_REQUIRE(epilogue != NS_EPI_BIAS_RESIDUAL || residual != 0, NS_ERR_ARGUMENT, "ns_linear_forward: NS_EPI_BIAS_RESIDUAL needs a residual");
    NS_REQUIRE(out_dtype == NS_F32 || out_dtype == NS_BF16, NS_ERR_ARGUMENT, "ns_linear_forward: output must be NS_F32 or NS_BF16");
    // a row shard yields a partial sum: bias and residual are added once, after the ranks' partials are reduced
    NS_REQUIRE(!(L->split == NS_SPLIT_ROW && L->tp_size > 1 && epilogue != NS_EPI_NONE), NS_ERR_ARGUMENT,
               "ns_linear_forward: a row shard must use NS_EPI_NONE; add bias and residual after the reduction (ns_bias_residual)");
    NsGemmParams p = {};
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.residual_dtype = residual_dtype == NS_BF16 ? NS_BF16 : NS_F32;
    p.out = reinterpret_cast<void*>(y);
    p.a_scale = reinterpret_cast<const float*>(x_scale);
    p.w_scale = L->w_scale;
    p.bias = epilogue == NS_EPI_NONE ? nullptr : L->bias;
    p.prefetch_b = 1;   // the layer's weights were written before a synchronisation (ns_linear_create)
    p.residual = reinterpret_cast<const void*>(residual);
    return ns_gemm_run(d, L->mode == NS_I8 ? NS_KIND_I8 : NS_KIND_BF16, reinterpret_cast<const void*>(x), L->w, false, M, L->N_loc, L->K_loc, p);
}

// Internal entry points for the host-to-host pipeline (ns_host_pipeline.cu).
int ns_linear_shape(NsLinear* L, int* K, int* N, int* mode, int* split_ranks)
{
    NS_REQUIRE(L != nullptr, NS_ERR_ARGUMENT, "linear is null");
    *K = L->K_loc; *N = L->N_loc; *mode = L->mode; *split_ranks = L->split == NS_SPLIT_NONE ? 1 : L->tp_size;
    return NS_OK;
}

int ns_linear_forward_on(NsDevice* d, NsLinear* L, const void* x, const float* x_scale, int M, int epilogue, void* y)
{
    NS_REQUIRE(epilogue == NS_EPI_NONE || L->bias != nullptr, NS_ERR_ARGUMENT, "the layer has no bias for epilogue %d", epilogue);
    NsGemmParams p = {};
    p.epilogue = epilogue;
    p.out_dtype = NS_F32;
    p.residual_dtype = NS_F32;
    p.out = y;
    p.a_scale = x_scale;
    p.w_scale = L->w_scale;
    p.bias = epilogue == NS_EPI_NONE ? nullptr : L->bias;
    p.prefetch_b = 1;   // the layer's weights were written before a synchronisation (ns_linear_create)
    return ns_gemm_run(d, L->mode == NS_I8 ? NS_KIND_I8 : NS_KIND_BF16, x, L->w, false, M, L->N_loc, L->K_loc, p);
}

// The int8 product of a layer without its epilogue: exact int32 partial sums [splits, M, N_local] stay in the device
// object's scratch block for the row kernel that follows (ns_finish_norm_quant, ns_finish_kv_append).
extern "C" int ns_linear_forward_partial(ns_device_t h, ns_linear_t lh, uint64_t x, int M, uint64_t* partial, int* splits)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsLinear* L = reinterpret_cast<NsLinear*>(lh);
    NS_REQUIRE(L && x && partial && splits, NS_ERR_ARGUMENT, "ns_linear_forward_partial: null argument");
    NS_REQUIRE(L->mode == NS_I8, NS_ERR_ARGUMENT, "ns_linear_forward_partial: int8 layers only");
    NS_REQUIRE(M > 0 && (int64_t)M * L->N_loc <= (int64_t)1 << 24, NS_ERR_ARGUMENT,
               "ns_linear_forward_partial: meant for the few rows of a decoding step (M * N <= 2^24), got M=%d N=%d", M, L->N_loc);
    NsGemmParams p = {};
    p.epilogue = NS_EPI_NONE;
    p.out_dtype = NS_F32;
    p.residual_dtype = NS_F32;
    p.prefetch_b = 1;
    void* ptr = nullptr;
    int s = 0;
    rc = ns_gemm_run(d, NS_KIND_I8, reinterpret_cast<const void*>(x), L->w, false, M, L->N_loc, L->K_loc, p, nullptr, 0, &ptr, &s);
    if (rc != NS_OK) return rc;
    *partial = reinterpret_cast<uint64_t>(ptr);
    *splits = s;
    return NS_OK;
}
