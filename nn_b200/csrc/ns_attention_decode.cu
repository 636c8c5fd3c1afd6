// Paged key/value cache and attention for cached decoding (new queries against the cache).
//
// Reference path: MultiHeadAttention.ForwardCached (src/NeuralSharp/Layers/Attention.cs:98-118) with
// KeyValueCache (Layers/Decoding.cs:14-35): kv_write_f32 appends the new keys/values at a device-side
// position, then matmul_f32 (Q.K^T over the WHOLE capacity), scale_mask_softmax_f32 with a -1e9 mask
// and matmul_f32 (P.V) run as three kernels with the score tensor in memory.  Here one kernel reads
// only positions [0, pos + i] (exactly equivalent: exp(-1e9 - max) is 0 in float and unwritten rows
// are always masked), keeps scores in shared memory and never writes them out.  The work is
// HBM-bound (every cached key and value is read once per step), so it runs on the CUDA cores with
// 16-byte loads; there is no contraction large enough for the tensor cores at one query per head.
//
// Cache layout: two pools (keys, values) of bf16 [num_pages, heads, page_size, head_dim]; a page table
// int32 [batch, max_pages] maps (sequence, position / page_size) to a page.  A contiguous cache is the
// identity table.  One (page, head) slab is page_size * head_dim * 2 bytes of contiguous memory.
#include <math.h>
#include <string.h>

#include "ns_common.cuh"

struct NsKvCache {
    int ordinal;
    int num_pages, page_size, heads, head_dim;
    uint16_t* k_pool;
    uint16_t* v_pool;
    bool owns_pools;
};

namespace {

constexpr int DEC_THREADS = 128;
// The cache of a row is walked in CHUNKS of `chunk` positions, [chunk k, chunk (k + 1)), whatever the batch, the grid or the
// split of the work: every chunk yields its own (maximum, sum, weighted values) triple, computed from the chunk alone, and a
// row's result is the fold of its chunks' triples in chunk order with one fixed formula (fold_chunk).  One CTA that owns the
// whole row folds in registers; several CTAs per row write their chunks' triples to scratch memory and
// ns_attention_combine_kernel folds them -- the same operations in the same order, so a row's output bits do not depend on how
// many sequences share the GPU (a sequence decoded in a batch equals the sequence decoded alone: DecodingTests.cs:100-142
// holds the reference to that).  The chunk length is a function of the cache's capacity alone (decode_chunk): two chunks up
// to 2048 positions, about 1024 positions each beyond (a chunk costs a block-wide reduction of the weighted values; with
// 256-position chunks a 64-sequence step lost 8 % to them).
constexpr int DEC_MAX_CHUNK = 1024;      // scores of a chunk are kept in shared memory

struct DecodeParams {
    const uint16_t* q;  // element (b, i, h, d) at q[(b * steps + i) * q_stride + h * dh + d]
    int64_t q_stride;
    uint16_t* o;
    int64_t o_stride;
    const uint16_t* k_pool;
    const uint16_t* v_pool;
    const int32_t* page_table;
    int max_pages, page_size, page_shift, heads;
    const int32_t* pos_dev;
    int batch, steps, splits;
    int chunk;              // positions per chunk (a multiple of 64, at most DEC_MAX_CHUNK)
    int max_chunks;         // chunks of the longest possible context: triple slots per row in `partial`
    int chunks_per_split;   // consecutive chunks one CTA owns
    float scale;
    float* partial;  // [rows, max_chunks, 2 + dh] when splits > 1
    // optional: int8 row quantisation of the output (the next product's input) by the last CTA to finish a row
    int8_t* q_out;          // [batch * steps, heads * dh] or null
    float* q_scale;         // [batch * steps]
    uint32_t* row_tickets;  // one word per output row, zero between launches
};

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

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8])
{
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int t = 0; t < 4; t++) {
        f[2 * t] = __uint_as_float(w[t] << 16);
        f[2 * t + 1] = __uint_as_float(w[t] & 0xFFFF0000u);
    }
}

// (M, L, O) <- (M, L, O) folded with the triple (m, l, o) of the next chunk; every product and sum rounded on its own so that
// the kernels that fold give the same bits.  The first chunk of a row is taken as it is.
__device__ __forceinline__ void fold_chunk(bool first, float& M, float& L, float& O, float m, float l, float o)
{
    if (first) { M = m; L = l; O = o; return; }
    const float M2 = fmaxf(M, m);
    const float a = expf(M - M2), b = expf(m - M2);
    L = __fadd_rn(__fmul_rn(L, a), __fmul_rn(l, b));
    O = __fadd_rn(__fmul_rn(O, a), __fmul_rn(o, b));
    M = M2;
}

// The output row (b, i) -- all heads of one token -- is complete when `heads` CTAs have stored their 128 (or 64, 32)
// columns.  Each CTA takes a ticket of its row after its store; the one that draws the last ticket quantises the row:
// scale = absmax / 127 (1 for a zero row), q = clamp(rint(x / scale)), exactly ns_quantize_rows_i8 on the bf16 values,
// and clears the ticket word.  This folds a launch of the decoding step into the attention kernel.
template <int THREADS>
__device__ __forceinline__ void quantize_row_if_last(const DecodeParams& p, int b, int i, int dh, float* red, int* last_smem)
{
    const int row = b * p.steps + i;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(&p.row_tickets[row], 1u);
        *last_smem = (t == (uint32_t)p.heads - 1u) ? 1 : 0;
        if (*last_smem) p.row_tickets[row] = 0u;
    }
    __syncthreads();
    if (*last_smem == 0) return;
    __threadfence();
    const int cols = p.heads * dh;
    const uint16_t* src = p.o + (size_t)row * p.o_stride;
    float amax = 0.0f;
    for (int v = threadIdx.x; v < cols / 8; v += THREADS) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(src + v * 8));
        float f[8];
        unpack8(raw, f);
#pragma unroll
        for (int d = 0; d < 8; d++) amax = fmaxf(amax, fabsf(f[d]));
    }
    amax = warp_max_f(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
    for (int w = 1; w < THREADS / 32; w++) amax = fmaxf(amax, red[w]);
    const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) p.q_scale[row] = sc;
    int8_t* dst = p.q_out + (size_t)row * cols;
    for (int v = threadIdx.x; v < cols / 8; v += THREADS) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(src + v * 8));
        float f[8];
        unpack8(raw, f);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int d = 0; d < 4; d++) {
            float q0 = fminf(fmaxf(rintf(__fdiv_rn(f[d], sc)), -127.0f), 127.0f);
            float q1 = fminf(fmaxf(rintf(__fdiv_rn(f[4 + d], sc)), -127.0f), 127.0f);
            lo |= (uint32_t)(uint8_t)(int8_t)q0 << (8 * d);
            hi |= (uint32_t)(uint8_t)(int8_t)q1 << (8 * d);
        }
        *reinterpret_cast<uint2*>(dst + v * 8) = make_uint2(lo, hi);
    }
}

// One CTA per (batch, head, new position, split).  DH = head_dim.  LPR = DH / 32 lanes share one cached row, each
// lane owning four 16-byte pieces of it (piece i of lane `sub` is piece sub + LPR * i of the row, so the lanes of a
// row read contiguous 16 * LPR bytes per load).
template <int DH, int U>
__global__ void __launch_bounds__(DEC_THREADS) ns_attention_decode_kernel(const DecodeParams p)
{
    constexpr int LPR = DH / 32;               // lanes per cached row
    constexpr int RPW = 32 / LPR;              // rows per warp per load round
    constexpr int GROUPS = DEC_THREADS / LPR;  // rows in flight per CTA
    // U = load rounds in flight per lane (a round = one cached row per lane group): two when thousands of CTAs share the
    // SMs, four when the grid is small and a CTA's own chain of loads is what its time consists of
    __shared__ float s_scores[DEC_MAX_CHUNK];
    __shared__ float s_red[DEC_THREADS / 32], s_red2[DEC_THREADS / 32];
    __shared__ float s_acc[GROUPS][DH];

    ns_pdl_wait();
    ns_pdl_trigger();
    int idx = blockIdx.x;
    const int split = idx % p.splits; idx /= p.splits;
    const int i = idx % p.steps; idx /= p.steps;
    const int h = idx % p.heads;
    const int b = idx / p.heads;
    const int kv_len = p.pos_dev[0] + i + 1;
    const int n_chunks = (kv_len + p.chunk - 1) / p.chunk;
    const int k0 = split * p.chunks_per_split;
    const int k1 = min(n_chunks, k0 + p.chunks_per_split);
    const int row_id = (b * p.heads + h) * p.steps + i;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = threadIdx.x % LPR;       // which pieces of a row this lane owns
    const int grp = threadIdx.x / LPR;       // row slot of this lane inside the CTA
    const int page_mask = p.page_size - 1;

    // running fold of this CTA's chunks (one CTA per row): thread d < DH holds column d of the weighted values
    float M_run = 0.0f, L_run = 0.0f, O_run = 0.0f;

    float qf[4][8];
    {
        const uint16_t* qrow = p.q + (size_t)(b * p.steps + i) * p.q_stride + h * DH;
#pragma unroll
        for (int c = 0; c < 4; c++) unpack8(*reinterpret_cast<const uint4*>(qrow + (sub + LPR * c) * 8), qf[c]);
    }
    const int32_t* pt = p.page_table + (size_t)b * p.max_pages;
    const size_t slab = (size_t)p.page_size * DH;
    const size_t head_off = (size_t)h * slab + sub * 8;
    auto row_ptr = [&](const uint16_t* pool, int j) {
        const int page = __ldg(&pt[j >> p.page_shift]);
        return pool + (size_t)page * p.heads * slab + head_off + (size_t)(j & page_mask) * DH;
    };

    for (int k = k0; k < k1; k++) {
        const int c0 = k * p.chunk;
        const int c1 = min(kv_len, c0 + p.chunk);
        float acc[4][8];
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int d = 0; d < 8; d++) acc[c][d] = 0.0f;
        // ---- scores: s_j = (q . k_j) * scale; U rounds of four loads per lane are in flight before any is used.
        // Loop bounds are uniform per warp because the reduction shuffles need every lane.
        for (int jb = c0 + warp * RPW; jb < c1; jb += (DEC_THREADS / 32) * RPW * U) {
            uint4 kv[U][4];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int j = jb + u * (DEC_THREADS / 32) * RPW + lane / LPR;
                if (j < c1) {
                    const uint16_t* kr = row_ptr(p.k_pool, j);
#pragma unroll
                    for (int c = 0; c < 4; c++) kv[u][c] = __ldg(reinterpret_cast<const uint4*>(kr + LPR * c * 8));
                } else {
#pragma unroll
                    for (int c = 0; c < 4; c++) kv[u][c] = make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int j = jb + u * (DEC_THREADS / 32) * RPW + lane / LPR;
                float dot = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float kf[8];
                    unpack8(kv[u][c], kf);
#pragma unroll
                    for (int d = 0; d < 8; d++) dot = fmaf(qf[c][d], kf[d], dot);
                }
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (sub == 0 && j < c1) s_scores[j - c0] = dot * p.scale;
            }
        }
        __syncthreads();
        // ---- the chunk's own maximum and exponentials
        float mx = -INFINITY;
        for (int j = threadIdx.x; j < c1 - c0; j += DEC_THREADS) mx = fmaxf(mx, s_scores[j]);
        mx = warp_max_f(mx);
        if (lane == 0) s_red[warp] = mx;
        __syncthreads();
        mx = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
        float sum = 0.0f;
        for (int j = threadIdx.x; j < c1 - c0; j += DEC_THREADS) {
            const float e = expf(s_scores[j] - mx);
            s_scores[j] = e;
            sum += e;
        }
        sum = warp_sum_f(sum);
        if (lane == 0) s_red2[warp] = sum;      // (its own words: the maxima may still be being read)
        __syncthreads();
        sum = s_red2[0] + s_red2[1] + s_red2[2] + s_red2[3];
        // ---- o_g = sum of p_j * v_j over the rows of slot `grp`: rows grp, grp + GROUPS, ... of the chunk
        for (int jb = c0 + grp; jb < c1; jb += GROUPS * U) {
            uint4 vv[U][4];
            float pj[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int j = jb + u * GROUPS;
                pj[u] = 0.0f;
                if (j < c1) {
                    const uint16_t* vr = row_ptr(p.v_pool, j);
#pragma unroll
                    for (int c = 0; c < 4; c++) vv[u][c] = __ldg(reinterpret_cast<const uint4*>(vr + LPR * c * 8));
                    pj[u] = s_scores[j - c0];
                } else {
#pragma unroll
                    for (int c = 0; c < 4; c++) vv[u][c] = make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float vf[8];
                    unpack8(vv[u][c], vf);
#pragma unroll
                    for (int d = 0; d < 8; d++) acc[c][d] = fmaf(pj[u], vf[d], acc[c][d]);
                }
        }
        // ---- the chunk's weighted values: the GROUPS slots summed in slot order
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int d = 0; d < 8; d++) s_acc[grp][(sub + LPR * c) * 8 + d] = acc[c][d];
        __syncthreads();
        for (int d = threadIdx.x; d < DH; d += DEC_THREADS) {
            float t = 0.0f;
#pragma unroll 8
            for (int gg = 0; gg < GROUPS; gg++) t += s_acc[gg][d];
            if (p.splits == 1) {
                fold_chunk(k == k0, M_run, L_run, O_run, mx, sum, t);
            } else {
                float* dst = p.partial + ((size_t)row_id * p.max_chunks + k) * (2 + DH);
                dst[2 + d] = t;
                if (d == 0) { dst[0] = mx; dst[1] = sum; }
            }
        }
        // (no barrier here: the next chunk writes s_scores and s_red only after this one's last reads of them, which precede
        // the barrier above, and s_acc only after three more barriers)
    }
    if (p.splits == 1) {
        for (int d = threadIdx.x; d < DH; d += DEC_THREADS)
            p.o[(size_t)(b * p.steps + i) * p.o_stride + h * DH + d] = ns_f32_to_bf16_bits(O_run / L_run);
    }
    if (p.q_out != nullptr && p.splits == 1) {
        __shared__ int last_cta;
        quantize_row_if_last<DEC_THREADS>(p, b, i, DH, s_red, &last_cta);
    }
}

// Merges the per-split (max, sum, unnormalised output) triples of one row.
template <int DH>
__global__ void ns_attention_combine_kernel(const DecodeParams p)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    const int row_id = blockIdx.x;
    const int i = row_id % p.steps;
    const int h = (row_id / p.steps) % p.heads;
    const int b = row_id / (p.steps * p.heads);
    const int n_chunks = (p.pos_dev[0] + i + 1 + p.chunk - 1) / p.chunk;
    const float* src = p.partial + (size_t)row_id * p.max_chunks * (2 + DH);
    for (int d = threadIdx.x; d < DH; d += blockDim.x) {
        float M = 0.0f, L = 0.0f, O = 0.0f;
        for (int k = 0; k < n_chunks; k++) {
            const float* t = src + (size_t)k * (2 + DH);
            fold_chunk(k == 0, M, L, O, t[0], t[1], t[2 + d]);
        }
        p.o[(size_t)(b * p.steps + i) * p.o_stride + h * DH + d] = ns_f32_to_bf16_bits(O / L);
    }
    if (p.q_out != nullptr) {
        __shared__ int last_cta;
        __shared__ float red[2];
        if (DH < 64) quantize_row_if_last<32>(p, b, i, DH, red, &last_cta);
        else quantize_row_if_last<64>(p, b, i, DH, red, &last_cta);
    }
}

// cache[page(b, pos + i), h, (pos + i) % page_size, :] = src[(b, i), h, :]
// A negative position, a position beyond the page table or a table entry that names no page of the pool is not written:
// the store is skipped and code 500 goes to the device status word (the reference throws for positions beyond the
// capacity, DecodingContext.BeginStep, src/NeuralSharp/Layers/Decoding.cs:96-99).
__global__ void ns_kv_append_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v, int64_t src_stride, uint16_t* k_pool,
                                    uint16_t* v_pool, const int32_t* __restrict__ page_table, int max_pages, int page_size, int heads, int dh,
                                    const int32_t* pos_dev, int batch, int steps, int num_pages, int* status)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    const int pos0 = pos_dev[0];
    const int vec = dh / 8;
    const int64_t n = (int64_t)batch * steps * heads * vec;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(e % vec);
        const int h = (int)((e / vec) % heads);
        const int64_t tok = e / ((int64_t)vec * heads);
        const int i = (int)(tok % steps), b = (int)(tok / steps);
        const int pos = pos0 + i;
        if (pos < 0 || pos / page_size >= max_pages) { *reinterpret_cast<volatile int*>(status) = 500; continue; }
        const int page = page_table[(size_t)b * max_pages + pos / page_size];
        if (page < 0 || page >= num_pages) { *reinterpret_cast<volatile int*>(status) = 500; continue; }
        const size_t dst = (((size_t)page * heads + h) * page_size + pos % page_size) * dh + c * 8;
        const size_t src = (size_t)tok * src_stride + h * dh + c * 8;
        *reinterpret_cast<uint4*>(k_pool + dst) = *reinterpret_cast<const uint4*>(k + src);
        *reinterpret_cast<uint4*>(v_pool + dst) = *reinterpret_cast<const uint4*>(v + src);
    }
}

template <int DH>
int launch_decode(NsDevice* d, const DecodeParams& p)
{
    const int rows = p.batch * p.heads * p.steps;
    if ((int64_t)rows * p.splits < 3 * (int64_t)d->sm_count)   // measured: 384 CTAs gain 9 %, 512 CTAs lose 30 % with four rounds
        NS_CUDA(ns_launch_plain(ns_attention_decode_kernel<DH, 4>, dim3(rows * p.splits), dim3(DEC_THREADS), 0, d->stream, p));
    else
        NS_CUDA(ns_launch_plain(ns_attention_decode_kernel<DH, 2>, dim3(rows * p.splits), dim3(DEC_THREADS), 0, d->stream, p));
    if (p.splits > 1) {
        NS_CUDA(ns_launch_plain(ns_attention_combine_kernel<DH>, dim3(rows), dim3(DH < 64 ? 32 : 64), 0, d->stream, p));
    }
    return NS_OK;
}

}  // namespace

extern "C" int ns_kv_cache_create(ns_device_t h, int num_pages, int page_size, int heads, int head_dim, ns_kv_cache_t* out)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(out != nullptr, NS_ERR_ARGUMENT, "ns_kv_cache_create: out handle is null");
    NS_REQUIRE(num_pages > 0 && page_size > 0 && heads > 0, NS_ERR_ARGUMENT, "ns_kv_cache_create: bad shape");
    NS_REQUIRE((page_size & (page_size - 1)) == 0, NS_ERR_ARGUMENT, "ns_kv_cache_create: page_size must be a power of two (got %d)", page_size);
    NS_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128, NS_ERR_ARGUMENT, "ns_kv_cache_create: head_dim must be 32, 64 or 128");
    NS_REQUIRE(!d->capturing, NS_ERR_STATE, "ns_kv_cache_create: not allowed while the stream is being captured");
    NsKvCache* c = new NsKvCache();
    c->ordinal = d->ordinal;
    c->num_pages = num_pages; c->page_size = page_size; c->heads = heads; c->head_dim = head_dim;
    c->owns_pools = true;
    const size_t bytes = (size_t)num_pages * heads * page_size * head_dim * 2;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->k_pool), bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&c->v_pool), bytes);
    if (e != cudaSuccess) {
        if (c->k_pool) cudaFree(c->k_pool);
        delete c;
        cudaGetLastError();
        return ns_fail(NS_ERR_MEMORY, "key/value pools of 2 x %zu bytes: %s (%d)", bytes, cudaGetErrorName(e), (int)e);
    }
    // the reference's cache is zero-initialised (Layers/Decoding.cs:19-20)
    NS_CUDA(cudaMemsetAsync(c->k_pool, 0, bytes, d->stream));
    NS_CUDA(cudaMemsetAsync(c->v_pool, 0, bytes, d->stream));
    *out = reinterpret_cast<ns_kv_cache_t>(c);
    return NS_OK;
}

extern "C" int ns_kv_cache_destroy(ns_kv_cache_t ch)
{
    NsKvCache* c = reinterpret_cast<NsKvCache*>(ch);
    if (!c) return NS_OK;
    cudaSetDevice(c->ordinal);
    if (c->owns_pools) {
        cudaFree(c->k_pool);
        cudaFree(c->v_pool);
    }
    delete c;
    return NS_OK;
}

// A cache over pools the caller allocated (and keeps): one device allocation can then hold the pools of every layer, which
// is what lets another process map them (ns_ipc_handle) and write prompt keys / values straight into them.
extern "C" int ns_kv_cache_create_in(ns_device_t h, int num_pages, int page_size, int heads, int head_dim, uint64_t k_pool, uint64_t v_pool,
                                     ns_kv_cache_t* out)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(out != nullptr && k_pool != 0 && v_pool != 0, NS_ERR_ARGUMENT, "ns_kv_cache_create_in: null argument");
    NS_REQUIRE(num_pages > 0 && page_size > 0 && heads > 0, NS_ERR_ARGUMENT, "ns_kv_cache_create_in: bad shape");
    NS_REQUIRE((page_size & (page_size - 1)) == 0, NS_ERR_ARGUMENT, "ns_kv_cache_create_in: page_size must be a power of two (got %d)", page_size);
    NS_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128, NS_ERR_ARGUMENT, "ns_kv_cache_create_in: head_dim must be 32, 64 or 128");
    NS_REQUIRE(((k_pool | v_pool) & 255) == 0, NS_ERR_ARGUMENT, "ns_kv_cache_create_in: pools must be 256-byte aligned");
    NsKvCache* c = new NsKvCache();
    c->ordinal = d->ordinal;
    c->num_pages = num_pages; c->page_size = page_size; c->heads = heads; c->head_dim = head_dim;
    c->k_pool = reinterpret_cast<uint16_t*>(k_pool);
    c->v_pool = reinterpret_cast<uint16_t*>(v_pool);
    c->owns_pools = false;
    const size_t bytes = (size_t)num_pages * heads * page_size * head_dim * 2;
    NS_CUDA(cudaMemsetAsync(c->k_pool, 0, bytes, d->stream));
    NS_CUDA(cudaMemsetAsync(c->v_pool, 0, bytes, d->stream));
    *out = reinterpret_cast<ns_kv_cache_t>(c);
    return NS_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Prompt keys / values from a batch-sharded prefill into head-sharded caches.
//
// On several GPUs the prompt is read by batch sharding (every GPU holds a full copy of the weights and reads batch / ranks
// sequences with no collective), while decoding is tensor-parallel: each GPU's cache holds heads / ranks heads of ALL
// sequences.  The one exchange step in between: every GPU copies, for each of its sequences, the (page, head) slabs of
// its full-head cache into the cache of the rank that owns the head -- plain 16-byte stores into peer-mapped memory
// (NVLink), the local share included.  A slab (page_size x head_dim bf16) is contiguous on both sides.  The reference is
// single-device; the caller it serves is the prompt read of CharGpt.Generate (samples/Shared/Gpt/CharGpt.cs:261-270).
// ---------------------------------------------------------------------------------------------------------
namespace {
struct KvScatterParams {
    const uint16_t* src_k;
    const uint16_t* src_v;
    const int32_t* src_table;     // [n_seqs, src_max_pages]
    int src_max_pages, src_heads;
    uint16_t* dst_k[8];
    uint16_t* dst_v[8];
    const int32_t* dst_table;     // [batch, dst_max_pages], this rank's copy
    int dst_max_pages, dst_heads, dst_num_pages;
    int n_seqs, seq0, pages_used, world;
    int slab_vec;                 // 16-byte vectors per slab
    int layers;                   // the pools of layer l sit l * src_layer_vec / dst_layer_vec 16-byte vectors after layer 0's
    size_t src_layer_vec, dst_layer_vec;
    int* status;
};

__global__ void __launch_bounds__(256) ns_kv_scatter_heads_kernel(const KvScatterParams p)
{
    ns_pdl_wait();
    ns_pdl_trigger();
    const int slabs = p.n_seqs * p.pages_used * p.src_heads;
    const long long total = (long long)slabs * p.layers;
    for (long long w = blockIdx.x; w < total; w += gridDim.x) {
        const int layer = (int)(w / slabs);
        const int s = (int)(w % slabs);
        const int h = s % p.src_heads;
        const int j = (s / p.src_heads) % p.pages_used;
        const int b = s / (p.src_heads * p.pages_used);
        const int sp = p.src_table[(size_t)b * p.src_max_pages + j];
        const int dp = p.dst_table[(size_t)(p.seq0 + b) * p.dst_max_pages + j];
        const int r = h / p.dst_heads, hl = h % p.dst_heads;
        if (dp < 0 || dp >= p.dst_num_pages || r >= p.world) {
            if (threadIdx.x == 0) *reinterpret_cast<volatile int*>(p.status) = 510;
            continue;
        }
        const size_t so = ((size_t)sp * p.src_heads + h) * p.slab_vec + (size_t)layer * p.src_layer_vec;
        const size_t dofs = ((size_t)dp * p.dst_heads + hl) * p.slab_vec + (size_t)layer * p.dst_layer_vec;
        const uint4* sk = reinterpret_cast<const uint4*>(p.src_k) + so;
        const uint4* sv = reinterpret_cast<const uint4*>(p.src_v) + so;
        uint4* dk = reinterpret_cast<uint4*>(p.dst_k[r]) + dofs;
        uint4* dv = reinterpret_cast<uint4*>(p.dst_v[r]) + dofs;
        for (int i = threadIdx.x; i < p.slab_vec; i += blockDim.x) {
            const uint4 a = __ldg(sk + i), c = __ldg(sv + i);
            dk[i] = a;
            dv[i] = c;
        }
    }
}
}  // namespace

extern "C" int ns_kv_scatter_heads(ns_device_t h, ns_kv_cache_t src, uint64_t src_table, int src_max_pages, int n_seqs, int seq0, int pages_used,
                                   const uint64_t* dst_k_pools, const uint64_t* dst_v_pools, int world, int dst_heads, int dst_num_pages,
                                   uint64_t dst_table, int dst_max_pages, int layers, uint64_t src_layer_stride, uint64_t dst_layer_stride)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsKvCache* c = reinterpret_cast<NsKvCache*>(src);
    NS_REQUIRE(c && src_table && dst_table && dst_k_pools && dst_v_pools, NS_ERR_ARGUMENT, "ns_kv_scatter_heads: null argument");
    NS_REQUIRE(world >= 1 && world <= 8 && dst_heads >= 1 && dst_heads * world == c->heads, NS_ERR_ARGUMENT,
               "ns_kv_scatter_heads: %d ranks x %d heads do not make the source's %d heads", world, dst_heads, c->heads);
    NS_REQUIRE(n_seqs >= 0 && seq0 >= 0 && pages_used >= 0 && pages_used <= src_max_pages && pages_used <= dst_max_pages, NS_ERR_ARGUMENT,
               "ns_kv_scatter_heads: bad shape");
    NS_REQUIRE(layers >= 1 && (layers == 1 || (src_layer_stride % 16 == 0 && dst_layer_stride % 16 == 0 && src_layer_stride > 0 && dst_layer_stride > 0)),
               NS_ERR_ARGUMENT, "ns_kv_scatter_heads: layer strides must be positive multiples of 16 bytes");
    if (n_seqs == 0 || pages_used == 0) return NS_OK;
    KvScatterParams p;
    memset(&p, 0, sizeof(p));
    p.src_k = c->k_pool; p.src_v = c->v_pool;
    p.src_table = reinterpret_cast<const int32_t*>(src_table);
    p.src_max_pages = src_max_pages; p.src_heads = c->heads;
    for (int r = 0; r < world; r++) {
        NS_REQUIRE(dst_k_pools[r] != 0 && dst_v_pools[r] != 0 && ((dst_k_pools[r] | dst_v_pools[r]) & 15) == 0, NS_ERR_ARGUMENT,
                   "ns_kv_scatter_heads: pool of rank %d is null or misaligned", r);
        p.dst_k[r] = reinterpret_cast<uint16_t*>(dst_k_pools[r]);
        p.dst_v[r] = reinterpret_cast<uint16_t*>(dst_v_pools[r]);
    }
    p.dst_table = reinterpret_cast<const int32_t*>(dst_table);
    p.dst_max_pages = dst_max_pages; p.dst_heads = dst_heads; p.dst_num_pages = dst_num_pages;
    p.n_seqs = n_seqs; p.seq0 = seq0; p.pages_used = pages_used; p.world = world;
    p.slab_vec = c->page_size * c->head_dim * 2 / 16;
    p.layers = layers;
    p.src_layer_vec = src_layer_stride / 16;
    p.dst_layer_vec = dst_layer_stride / 16;
    p.status = d->status_dev;
    const int64_t slabs = (int64_t)n_seqs * pages_used * c->heads * layers;
    const int64_t cap = (int64_t)d->sm_count * 8;
    NS_CUDA(ns_launch_plain(ns_kv_scatter_heads_kernel, dim3((unsigned)(slabs < cap ? slabs : cap)), dim3(256), 0, d->stream, p));
    return NS_OK;
}


extern "C" int ns_kv_cache_pools(ns_kv_cache_t ch, uint64_t* k_pool, uint64_t* v_pool, uint64_t* bytes_each)
{
    NsKvCache* c = reinterpret_cast<NsKvCache*>(ch);
    NS_REQUIRE(c != nullptr, NS_ERR_ARGUMENT, "ns_kv_cache_pools: cache is null");
    if (k_pool) *k_pool = reinterpret_cast<uint64_t>(c->k_pool);
    if (v_pool) *v_pool = reinterpret_cast<uint64_t>(c->v_pool);
    if (bytes_each) *bytes_each = (uint64_t)c->num_pages * c->heads * c->page_size * c->head_dim * 2;
    return NS_OK;
}

extern "C" int ns_kv_append(ns_device_t h, ns_kv_cache_t ch, uint64_t k, uint64_t v, int64_t src_stride, uint64_t page_table, int max_pages,
                            uint64_t pos_dev, int batch, int steps)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsKvCache* c = reinterpret_cast<NsKvCache*>(ch);
    NS_REQUIRE(c && k && v && page_table && pos_dev, NS_ERR_ARGUMENT, "ns_kv_append: null argument");
    NS_REQUIRE(batch >= 0 && steps >= 0 && max_pages > 0, NS_ERR_ARGUMENT, "ns_kv_append: bad shape");
    NS_REQUIRE(src_stride % 8 == 0 && (k & 15) == 0 && (v & 15) == 0, NS_ERR_ARGUMENT, "ns_kv_append: source rows must be 16-byte aligned");
    const int64_t n = (int64_t)batch * steps * c->heads * (c->head_dim / 8);
    if (n == 0) return NS_OK;
    int64_t blocks = (n + 255) / 256;
    if (blocks > (int64_t)d->sm_count * 16) blocks = (int64_t)d->sm_count * 16;
    NS_CUDA(ns_launch_plain(ns_kv_append_kernel, dim3((unsigned)blocks), dim3(256), 0, d->stream, reinterpret_cast<const uint16_t*>(k), reinterpret_cast<const uint16_t*>(v), src_stride,
                                                                c->k_pool, c->v_pool, reinterpret_cast<const int32_t*>(page_table), max_pages,
                                                                c->page_size, c->heads, c->head_dim, reinterpret_cast<const int32_t*>(pos_dev), batch,
                                                                steps, c->num_pages, d->status_dev));
    return NS_OK;
}

// The pools and geometry of a cache, for kernels in other files that write to it (ns_step_fused.cu).
struct NsKvCacheView {
    uint16_t* k_pool;
    uint16_t* v_pool;
    int page_size, heads, head_dim, num_pages;
};
int ns_kv_cache_view(ns_kv_cache_t ch, NsKvCacheView* out)
{
    NsKvCache* c = reinterpret_cast<NsKvCache*>(ch);
    NS_REQUIRE(c != nullptr && out != nullptr, NS_ERR_ARGUMENT, "cache is null");
    out->k_pool = c->k_pool; out->v_pool = c->v_pool;
    out->page_size = c->page_size; out->heads = c->heads; out->head_dim = c->head_dim; out->num_pages = c->num_pages;
    return NS_OK;
}

// Scratch bytes ns_attention_decode needs for `rows` = batch * heads * steps query rows split `splits` ways.
static size_t decode_scratch_bytes(int rows, int max_chunks, int dh) { return (size_t)rows * max_chunks * (2 + dh) * sizeof(float); }

// Positions per chunk for a cache of `max_len` positions: a function of the capacity alone, so that every launch on that
// cache -- whatever its batch -- cuts a row the same way.
static int decode_chunk(int max_len)
{
    int n = (max_len + DEC_MAX_CHUNK - 1) / DEC_MAX_CHUNK;
    if (n < 2) n = 2;
    int c = ((max_len + n - 1) / n + 63) / 64 * 64;
    return c > DEC_MAX_CHUNK ? DEC_MAX_CHUNK : c;
}

// CTAs per row: one per chunk when the rows alone do not fill the SMs twice, else one.
static int choose_splits(const NsDevice* d, int rows, int max_chunks)
{
    if (rows >= 2 * d->sm_count) return 1;
    return max_chunks > 32 ? 32 : max_chunks;
}

int ns_attention_decode_impl(NsDevice* d, NsKvCache* c, uint64_t q, int64_t q_stride, uint64_t o, int64_t o_stride, uint64_t page_table,
                             int max_pages, uint64_t pos_dev, int batch, int steps, float scale, float* scratch, size_t scratch_bytes,
                             bool own_scratch, uint64_t q_out = 0, uint64_t q_scale = 0)
{
    NS_REQUIRE(c && q && o && page_table && pos_dev, NS_ERR_ARGUMENT, "ns_attention_decode: null argument");
    NS_REQUIRE(batch > 0 && steps > 0 && max_pages > 0, NS_ERR_ARGUMENT, "ns_attention_decode: bad shape");
    NS_REQUIRE(q_stride % 8 == 0 && (q & 15) == 0, NS_ERR_ARGUMENT, "ns_attention_decode: query rows must be 16-byte aligned");
    DecodeParams p;
    p.q = reinterpret_cast<const uint16_t*>(q); p.q_stride = q_stride;
    p.o = reinterpret_cast<uint16_t*>(o); p.o_stride = o_stride;
    p.k_pool = c->k_pool; p.v_pool = c->v_pool;
    p.page_table = reinterpret_cast<const int32_t*>(page_table);
    p.max_pages = max_pages; p.page_size = c->page_size; p.heads = c->heads;
    p.page_shift = 0;
    while ((1 << p.page_shift) < c->page_size) p.page_shift++;
    p.pos_dev = reinterpret_cast<const int32_t*>(pos_dev);
    p.batch = batch; p.steps = steps; p.scale = scale;
    p.q_out = reinterpret_cast<int8_t*>(q_out);
    p.q_scale = reinterpret_cast<float*>(q_scale);
    p.row_tickets = d->sync_words + NS_SYNC_ROW_TICKETS;
    if (q_out != 0) {
        NS_REQUIRE(q_scale != 0 && (q_out & 7) == 0 && (o & 15) == 0 && o_stride % 8 == 0, NS_ERR_ARGUMENT,
                   "ns_attention_decode_quant: q_scale missing or buffers misaligned");
        NS_REQUIRE((int64_t)batch * steps <= NS_SYNC_MAX_ROWS, NS_ERR_ARGUMENT, "ns_attention_decode_quant: at most %d output rows", (int)NS_SYNC_MAX_ROWS);
    }
    const int rows = batch * c->heads * steps;
    // the context length lives on the device; the split count is sized for the longest possible context
    p.chunk = decode_chunk(max_pages * c->page_size);
    p.max_chunks = (max_pages * c->page_size + p.chunk - 1) / p.chunk;
    p.splits = choose_splits(d, rows, p.max_chunks);
    p.chunks_per_split = (p.max_chunks + p.splits - 1) / p.splits;
    p.splits = (p.max_chunks + p.chunks_per_split - 1) / p.chunks_per_split;      // no CTA without a chunk
    p.partial = nullptr;
    if (p.splits > 1) {
        const size_t need = decode_scratch_bytes(rows, p.max_chunks, c->head_dim);
        if (own_scratch) {
            void* s = nullptr;
            int rc = ns_scratch_reserve(d, need, &s);
            if (rc != NS_OK) return rc;
            p.partial = reinterpret_cast<float*>(s);
        } else {
            NS_REQUIRE(need <= scratch_bytes, NS_ERR_MEMORY, "attention partials need %zu bytes, the fixed scratch block holds %zu", need, scratch_bytes);
            p.partial = scratch;
        }
    }
    switch (c->head_dim) {
        case 32: return launch_decode<32>(d, p);
        case 64: return launch_decode<64>(d, p);
        default: return launch_decode<128>(d, p);
    }
}

extern "C" int ns_attention_decode(ns_device_t h, ns_kv_cache_t ch, uint64_t q, int64_t q_stride, uint64_t o, int64_t o_stride,
                                   uint64_t page_table, int max_pages, uint64_t pos_dev, int batch, int steps, float scale)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    return ns_attention_decode_impl(d, reinterpret_cast<NsKvCache*>(ch), q, q_stride, o, o_stride, page_table, max_pages, pos_dev, batch, steps,
                                    scale, nullptr, 0, true);
}

// The same, and the output rows [batch * steps, heads * head_dim] also leave as int8 rows with one scale per row (the
// input of the attention output projection): the row quantisation the decoding step would otherwise launch next.
extern "C" int ns_attention_decode_quant(ns_device_t h, ns_kv_cache_t ch, uint64_t q, int64_t q_stride, uint64_t o, int64_t o_stride,
                                         uint64_t page_table, int max_pages, uint64_t pos_dev, int batch, int steps, float scale, uint64_t q_out,
                                         uint64_t q_scale)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(q_out != 0 && q_scale != 0, NS_ERR_ARGUMENT, "ns_attention_decode_quant: q_out and q_scale are required");
    NsKvCache* c = reinterpret_cast<NsKvCache*>(ch);
    NS_REQUIRE(c != nullptr && o_stride == (int64_t)c->heads * c->head_dim, NS_ERR_ARGUMENT,
               "ns_attention_decode_quant: the output rows must be contiguous (stride = heads x head_dim)");
    return ns_attention_decode_impl(d, c, q, q_stride, o, o_stride, page_table, max_pages, pos_dev, batch, steps, scale, nullptr, 0, true, q_out, q_scale);
}
