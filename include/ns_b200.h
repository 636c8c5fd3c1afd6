/*
 * ns_b200.h -- C ABI of libns_b200.so, the sm_100a implementation of NeuralSharp's CUDA inference hot
 * path (the products behind Linear, causal attention behind MultiHeadAttention, and the small
 * operators of one cached decoder step).
 *
 * Conventions (they follow the reference's P/Invoke layer, src/NeuralSharp/Backends/Cuda/CudaDriver.cs:
 * 63-77,86-179, so a C# `LibraryImport` binding reads like CudaDriver.cs):
 *   - every function returns int: 0 = success, otherwise an NS_ERR_* code; ns_last_error() gives the
 *     text of the calling thread's last failure ("<call> failed: <name> (<code>)" for CUDA errors);
 *   - device addresses are uint64_t (the reference's CUdeviceptr, CudaBackend.cs:7-10); handles are
 *     opaque pointers; out-parameters come last;
 *   - sizes of raw memory calls are BYTES (the reference counts floats; int8 and bf16 buffers exist
 *     here);
 *   - all work is queued on the device object's stream; nothing synchronises unless it says so;
 *   - matrices are row-major and contiguous unless a leading dimension is passed.
 * There is no CPU fallback: without a CUDA device every compute entry point fails with NS_ERR_CUDA.
 */
#ifndef NS_B200_H
#define NS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NS_API __attribute__((visibility("default")))

enum {
    NS_OK = 0,
    NS_ERR_CUDA = 1,        /* a CUDA runtime/driver call failed (text has the CUDA error name) */
    NS_ERR_ARGUMENT = 2,    /* bad shape, null pointer, misaligned buffer, unsupported combination */
    NS_ERR_MEMORY = 3,      /* allocation failed or a stated maximum was exceeded */
    NS_ERR_KERNEL = 4,      /* a kernel's bounded wait ran out; see ns_device_status */
    NS_ERR_COMM = 5,        /* NCCL reported an error or is not available */
    NS_ERR_STATE = 6        /* call not valid now (e.g. allocation during stream capture) */
};

enum { NS_F32 = 0, NS_BF16 = 1, NS_I8 = 2, NS_I32 = 3 };

/* Epilogue of a product: what happens to each accumulator before it is stored. */
enum {
    NS_EPI_NONE = 0,        /* + nothing */
    NS_EPI_BIAS = 1,        /* + bias[n]                        (Linear.ForwardCore, Layers/Linear.cs:43-47) */
    NS_EPI_BIAS_GELU = 2,   /* gelu_tanh(. + bias[n])           (Tensor.BiasGelu, Tensor.Decoding.cs:44-51) */
    NS_EPI_BIAS_RESIDUAL = 3 /* . + bias[n] + residual[m,n]      (x + Linear(...), Layers/Attention.cs:201-205) */
};

/* How a Linear layer is divided among tensor-parallel ranks. */
enum { NS_SPLIT_NONE = 0, NS_SPLIT_COLUMN = 1, NS_SPLIT_ROW = 2 };

typedef struct ns_device_s* ns_device_t;
typedef struct ns_graph_s* ns_graph_t;
typedef struct ns_linear_s* ns_linear_t;
typedef struct ns_kv_cache_s* ns_kv_cache_t;
typedef struct ns_comm_s* ns_comm_t;
typedef struct ns_peer_group_s* ns_peer_group_t;

/* ------------------------------------------------------------------------------------------------
 * Runtime.  Replaces CudaBackend's constructor and CudaDriver's cuInit, cuDeviceGet, cuCtx.. and cuStream..
 * imports (Backends/Cuda/CudaBackend.cs:48-100,112-139; CudaDriver.cs:86-120).
 * ------------------------------------------------------------------------------------------------ */
NS_API const char* ns_last_error(void);
NS_API const char* ns_error_name(int code);
NS_API int ns_version(void);
NS_API int ns_device_count(int* count);
/* Opens device `ordinal` with a stream of its own. */
NS_API int ns_device_open(int ordinal, ns_device_t* dev);
/* Opens device `ordinal` on a stream the caller owns (cudaStream_t as an integer; 0 = legacy default). */
NS_API int ns_device_open_on_stream(int ordinal, uint64_t stream, ns_device_t* dev);
NS_API int ns_device_close(ns_device_t dev);
/* name: at least 128 bytes.  Backend info of CudaBackend.cs:56-60. */
NS_API int ns_device_info(ns_device_t dev, char* name, int* sm_count, uint64_t* total_bytes, uint64_t* free_bytes);
NS_API int ns_device_stream(ns_device_t dev, uint64_t* stream);
/* Backend.Synchronize (Backends/Backend.cs:219). Also reports a kernel whose bounded wait ran out. */
NS_API int ns_stream_sync(ns_device_t dev);
/* Reads and clears the device status word: 0 = no kernel gave up a wait. */
NS_API int ns_device_status(ns_device_t dev, int* status);
/* TEST HOOK, not for hosts: overrides the products' tiling heuristic so that tests and profiler cases can reach
 * every kernel variant on one shape.  tile_n: 0 = heuristic, 64 / 128 / 256 = that tile width with the single-CTA
 * kernel, NS_TUNE_NARROW = the narrowest tile, NS_TUNE_PAIR = the CTA-pair kernel wherever a shape allows it.
 * k_splits: 0 = heuristic, otherwise the split-K count; with NS_TUNE_PAIR, 2 = the pair kernel with its tiles' k-blocks dealt
 * out to the clusters in equal shares (the form large products take when their last wave of tiles would leave many clusters
 * idle), on any shape of at least four tiles.  tile_n = NS_TUNE_DROP_ROW: the many-row kernels (ns_quantize_rows_i8 and
 * ns_layernorm from 2048 rows on) leave out the copy of row k_splits, so that the bounded wait of that row's warps runs out
 * (status 600 + warps per row) without anything faulting; any other call of ns_device_tune ends it.  A host binding has no
 * reason to import this. */
/* TEST HOOK, not for hosts: while `buffer` (device memory, 4 x 8 bytes per SM) is non-zero, every CTA of a product with a
 * second phase (ns_linear_forward_norm_quant and its siblings) records four times in nanoseconds there: kernel start,
 * product done, all CTAs arrived, rows done.  0 turns it off. */
NS_API int ns_debug_tail_times(ns_device_t dev, uint64_t buffer);
#define NS_TUNE_NARROW 32
#define NS_TUNE_PAIR 512
#define NS_TUNE_DROP_ROW 600
NS_API int ns_device_tune(ns_device_t dev, int tile_n, int k_splits);

/* ------------------------------------------------------------------------------------------------
 * Memory.  Replaces Backend.Allocate/Return/Upload/Download/DownloadRange/Fill/Copy
 * (Backends/Backend.cs:68-86; CudaBackend.cs:185-301).
 * ------------------------------------------------------------------------------------------------ */
NS_API int ns_alloc(ns_device_t dev, uint64_t bytes, int zeroed, uint64_t* ptr);
NS_API int ns_free(ns_device_t dev, uint64_t ptr);
NS_API int ns_h2d(ns_device_t dev, uint64_t dst, const void* src, uint64_t bytes);        /* synchronous */
NS_API int ns_d2h(ns_device_t dev, void* dst, uint64_t src, uint64_t bytes);              /* synchronous */
NS_API int ns_h2d_async(ns_device_t dev, uint64_t dst, const void* src, uint64_t bytes);  /* src should be pinned */
NS_API int ns_d2h_async(ns_device_t dev, void* dst, uint64_t src, uint64_t bytes);
NS_API int ns_d2d_async(ns_device_t dev, uint64_t dst, uint64_t src, uint64_t bytes);
/* `rows` rows of width_bytes, pitches in bytes (Backend.Copy2D for raw bytes, Backends/Backend.cs:199). */
NS_API int ns_d2d_2d_async(ns_device_t dev, uint64_t dst, uint64_t dst_pitch, uint64_t src, uint64_t src_pitch, uint64_t width_bytes, uint64_t rows);
NS_API int ns_memset32_async(ns_device_t dev, uint64_t dst, uint32_t value, uint64_t count);
NS_API int ns_host_alloc(uint64_t bytes, void** ptr);   /* pinned host memory */
NS_API int ns_host_free(void* ptr);
/* One process per GPU: a block from ns_alloc made reachable from the other processes of the machine.  The owner exports a
 * 64-byte handle, hands it over by its own means, a peer maps it (peer access over NVLink) and unmaps it before the owner
 * frees the block.  No counterpart in the single-process reference (its cross-device move is a host round trip,
 * Tensor.cs:244-253). */
NS_API int ns_ipc_handle(ns_device_t dev, uint64_t ptr, void* handle64);
NS_API int ns_ipc_open(ns_device_t dev, const void* handle64, uint64_t* ptr);
NS_API int ns_ipc_close(ns_device_t dev, uint64_t ptr);

/* ------------------------------------------------------------------------------------------------
 * CUDA graphs.  Replaces Backend.BeginCapture/EndCapture/AbortCapture/ReplayGraph/DestroyGraph
 * (Backends/Backend.cs:266-281; CudaBackend.Decoding.cs:43-130; capture mode "relaxed" as
 * CudaDriver.cs:149).
 * ------------------------------------------------------------------------------------------------ */
NS_API int ns_capture_begin(ns_device_t dev);
NS_API int ns_capture_end(ns_device_t dev, ns_graph_t* graph);
NS_API int ns_capture_abort(ns_device_t dev);
NS_API int ns_graph_launch(ns_device_t dev, ns_graph_t graph);
NS_API int ns_graph_destroy(ns_graph_t graph);

/* Events on the device object's stream, for device-side timing (cuEvent* of the driver API). */
NS_API int ns_event_create(ns_device_t dev, uint64_t* event);
NS_API int ns_event_record(ns_device_t dev, uint64_t event);
NS_API int ns_event_elapsed_ms(ns_device_t dev, uint64_t start, uint64_t stop, float* ms);  /* waits for `stop` */
/* Work queued on dev's stream after this call waits for `event`, which may have been recorded on another device object of
 * the same GPU (cuStreamWaitEvent; the reference has one stream per device and no counterpart). */
NS_API int ns_stream_wait_event(ns_device_t dev, uint64_t event);
NS_API int ns_event_destroy(ns_device_t dev, uint64_t event);

/* ------------------------------------------------------------------------------------------------
 * Products on the tensor cores.  These replace the hot uses of Backend.BatchedMatMul
 * (Backends/Backend.cs:121-129 -> CudaBackend.BatchedMatMul, CudaBackend.cs:390-408 -> matmul_f32,
 * PtxKernels.cs:484-627) together with the bias / bias+GELU / residual kernels that follow it
 * (add_rowvec_f32 PtxKernels.cs:225-234, bias_gelu_f32 PtxKernels.Decoding.cs:93-114, add_f32).
 * ------------------------------------------------------------------------------------------------ */

/* Row-wise symmetric int8 quantisation: scale[r] = absmax/127 (1 when the row is zero),
 * q = clamp(rint(x/scale), -127, 127).  x is [rows, cols] of in_dtype (NS_F32 or NS_BF16). */
NS_API int ns_quantize_rows_i8(ns_device_t dev, uint64_t x, int in_dtype, int64_t rows, int cols, uint64_t q, uint64_t scale);

/* int8 x int8 -> int32 product with the dequantising epilogue fused:
 *   y[m,n] = epi( ((float)sum_k aq[m,k]*wq[n,k]) * a_scale[m] * w_scale[n] )   (each step rounded to float)
 * aq [M,K] int8, wq [N,K] int8 (one row per output channel), a_scale [M], w_scale [N], bias [N] or 0,
 * residual [M,N] of residual_dtype or 0, y [M,N] of out_dtype (NS_F32 or NS_BF16).
 * raw_s32: when non-zero, the exact int32 accumulators [M,N] are stored there as well.
 * K must be a multiple of 16. */
NS_API int ns_qmatmul_i8(ns_device_t dev, uint64_t aq, uint64_t a_scale, uint64_t wq, uint64_t w_scale, uint64_t bias,
                         uint64_t residual, int residual_dtype, int M, int N, int K, int epilogue, int out_dtype,
                         uint64_t y, uint64_t raw_s32);

/* The same product for callers that must not cause a device allocation (a host that records its step into a CUDA
 * graph with no warm-up run, or one that budgets device memory itself).  No counterpart in the reference.
 * Partial sums of a K-split product go to a fixed 8 MiB array inside the library instead of the device object's
 * scratch block: a shape that needs more (k_splits * M * N * 4 bytes) is rejected with NS_ERR_MEMORY.  The first
 * call on a device looks up the array's address and must come before any stream capture; all calls share the array,
 * so calls that overlap on the GPU race.  No raw accumulator output. */
NS_API int ns_qmatmul_i8_static(ns_device_t dev, uint64_t aq, uint64_t a_scale, uint64_t wq, uint64_t w_scale, uint64_t bias,
                                uint64_t residual, int residual_dtype, int M, int N, int K, int epilogue, int out_dtype, uint64_t y);

/* BENCH HOOK, not for hosts: the int8 product's main loop alone -- TMA loads and tcgen05 MMAs of the same kernels,
 * accumulators read from tensor memory and discarded, nothing dequantised and nothing written.  Timing it gives the
 * int8 tensor-core rate this library's load / MMA pipeline reaches on a shape, the yardstick the full product
 * (with its epilogue) is compared with.  No counterpart in the reference. */
NS_API int ns_bench_i8_mainloop(ns_device_t dev, uint64_t aq, uint64_t wq, int M, int N, int K);

/* bf16 product with float accumulation: C[b] = A[b] * op(B[b]); A [m,k] bf16; B [k,n] bf16 (transB = 0)
 * or [n,k] (transB = 1); C [m,n] of out_dtype.  Batch stride = one full matrix, as in the reference.
 * bias [n] float or 0 is added per column when epilogue says so.  k and n multiples of 8. */
NS_API int ns_matmul_bf16(ns_device_t dev, uint64_t a, uint64_t b, uint64_t c, int batch, int m, int n, int k,
                          int transB, uint64_t bias, uint64_t residual, int residual_dtype, int epilogue, int out_dtype);

/* ------------------------------------------------------------------------------------------------
 * Row-wise operators of the bf16 / int8 decoder path.
 * ------------------------------------------------------------------------------------------------ */

/* LayerNorm over the last dimension, float statistics, two passes, biased variance
 * (Backend.LayerNormFused, Backends/Backend.cs:227; kernel layernorm_fused_f32,
 * PtxKernels.Decoding.cs:61-90).  x [rows, cols] of in_dtype (NS_F32 / NS_BF16); gamma, beta float.
 * out_dtype NS_F32 / NS_BF16: y = LN(x).  out_dtype NS_I8: LN(x) is rounded to bf16 and quantised per
 * row as ns_quantize_rows_i8 does (q to y, scales to y_scale [rows]) -- the input of the next int8
 * product, without a round trip through memory. */
NS_API int ns_layernorm(ns_device_t dev, uint64_t x, int in_dtype, uint64_t gamma, uint64_t beta, int64_t rows, int cols, float eps,
                        int out_dtype, uint64_t y, uint64_t y_scale);

/* y[b, i, :] = tok_table[ids[b, i], :] + pos_table[pos + i, :]   (Embedding.ForwardCore, Layers/Embedding.cs:38,
 * + PositionalEncoding.ForwardCached, Layers/Attention.cs:268-269: two gather_f32 launches and an add there).
 * ids int32 [batch, steps] on the device; pos_dev: int32 device word holding the position of the first
 * new token (0 = position 0).  Ids are clamped to the table as the reference's GPU gather does. */
NS_API int ns_embed_pos(ns_device_t dev, uint64_t ids, uint64_t tok_table, uint64_t pos_table, int table_dtype, uint64_t pos_dev,
                        int batch, int steps, int dim, int vocab, int max_pos, int out_dtype, uint64_t y);

/* ids[r] = index of the first maximum of x[r, 0..cols)  (Tensor.ArgMax -> argmax_f32, PtxKernels.Advanced.cs:144-152;
 * "first maximum wins", CpuBackend.Advanced.cs:117-138).  x float, rows row_stride elements apart; ids int32. */
NS_API int ns_argmax_i32(ns_device_t dev, uint64_t x, int rows, int cols, int64_t row_stride, uint64_t ids);

/* counter[0] += delta on the device (DecodingContext.EndStep's affine_f32 on Position, Layers/Decoding.cs:121-127). */
NS_API int ns_add_i32(ns_device_t dev, uint64_t counter, int32_t delta);

/* Element-wise float <-> bf16 conversion (round to nearest even). */
NS_API int ns_convert(ns_device_t dev, uint64_t x, int in_dtype, uint64_t y, int out_dtype, int64_t n);

/* Synthetic inputs generated on the device (benchmarks): y[i] = mean + std * N(0,1) from a counter-based
 * hash of (seed, i); NS_I8 output is rint() clamped to [-127, 127].  ids: uniform int32 in [0, bound). */
NS_API int ns_fill_normal(ns_device_t dev, uint64_t y, int dtype, int64_t n, uint32_t seed, float mean, float std);
NS_API int ns_fill_ids(ns_device_t dev, uint64_t y, int64_t n, uint32_t seed, uint32_t bound);

/* ------------------------------------------------------------------------------------------------
 * float32 operator surface: the Backend methods one cached decoder step calls, with the reference's
 * argument lists (Backends/Backend.cs, line of each method in brackets).  Storage handles become
 * device addresses; every count is in floats, as in the reference.
 * ------------------------------------------------------------------------------------------------ */
/* [129] c[b] = op(a[b]) * op(b[b]) + beta * c[b]; each element one fused-multiply-add chain over k. */
NS_API int ns_f32_batched_matmul(ns_device_t dev, uint64_t a, uint64_t b, uint64_t c, int batch, int m, int n, int k,
                                 int transA, int transB, float beta);
/* [224] y[r,:] = softmax(scale * x[r,:] + mask[r % maskRows,:]); mask may be 0. */
NS_API int ns_f32_scale_mask_softmax(ns_device_t dev, uint64_t x, uint64_t mask, uint64_t y, int rows, int cols, int maskRows, float scale);
/* [227] */
NS_API int ns_f32_layernorm_fused(ns_device_t dev, uint64_t x, uint64_t gamma, uint64_t beta, uint64_t y, int rows, int cols, float eps);
/* [230] y[i] = gelu(x[i] + bias[i % cols]) */
NS_API int ns_f32_bias_gelu(ns_device_t dev, uint64_t x, uint64_t bias, uint64_t y, int64_t n, int cols);
/* [107] c[r,j] = a[r,j] + v[j] */
NS_API int ns_f32_add_row_vector(ns_device_t dev, uint64_t a, uint64_t v, uint64_t c, int rows, int cols);
/* [95] Binary(Add): c = a + b */
NS_API int ns_f32_add(ns_device_t dev, uint64_t a, uint64_t b, uint64_t c, int64_t n);
/* [98] y = alpha * x + beta */
NS_API int ns_f32_affine(ns_device_t dev, uint64_t x, uint64_t y, int64_t n, float alpha, float beta);
/* [119] y[i] += scale * s[0] */
NS_API int ns_f32_add_broadcast_scalar(ns_device_t dev, uint64_t s, uint64_t y, int64_t n, float scale);
/* [235] mask[i,j] = j <= position + i ? 0 : -1e9; position is a float in device memory */
NS_API int ns_f32_decoder_mask(ns_device_t dev, uint64_t position, uint64_t mask, int rows, int capacity);
/* [238] cache[h, position + t, :] = source[h, t, :] */
NS_API int ns_f32_key_value_write(ns_device_t dev, uint64_t source, uint64_t cache, uint64_t position, int heads, int steps, int capacity, int dim);
/* [172] y[i,:] = table[indices[i],:]; indices are float-encoded, truncated and clamped (GPU behaviour of the reference) */
NS_API int ns_f32_gather(ns_device_t dev, uint64_t table, uint64_t indices, uint64_t y, int count, int dim, int vocabulary);
/* [140] y[r] = (float) index of the first maximum of row r */
NS_API int ns_f32_argmax(ns_device_t dev, uint64_t x, uint64_t y, int rows, int cols);
/* same, row r starting at x[r * row_stride + row_offset] (the sampler's rowStride/rowOffset convention, Backend.cs:248) */
NS_API int ns_f32_argmax_strided(ns_device_t dev, uint64_t x, uint64_t y, int rows, int cols, int64_t row_stride, int64_t row_offset);
/* [193] y (+)= x permuted; outShape / inStrides have `rank` (<= 6) entries */
NS_API int ns_f32_permute(ns_device_t dev, uint64_t x, uint64_t y, const int* outShape, const int* inStrides, int rank, int accumulate);
/* [199] dst[dstOffset + r*dstStride + c] (+)= src[srcOffset + r*srcStride + c] */
NS_API int ns_f32_copy2d(ns_device_t dev, uint64_t src, int64_t srcOffset, int srcStride, uint64_t dst, int64_t dstOffset, int dstStride,
                         int rows, int cols, int accumulate);
/* [248] SampleRows (kernel sample_rows_f32, Backends/Cuda/PtxKernels.Decoding.cs:170-350; CPU twin
 * Backends/Cpu/CpuBackend.Decoding.cs:114-245).  Row r reads logits[r * rowStride + rowOffset + j], j < vocabulary;
 * writes ids[r] (float-encoded) and 13 statistics at stats[(step[0] * rows + r) * 13]: id, probability, entropy in
 * bits, five (alternative id, probability) pairs (-1, 0 when fewer are kept).  step[0] is a float in device memory,
 * so a recorded graph stays valid.  temperature is floored at 1e-3; topK 0 = all; topP 1 = off; minP 0 = off. */
NS_API int ns_f32_sample_rows(ns_device_t dev, uint64_t logits, uint64_t ids, uint64_t stats, uint64_t step, int rows, int vocabulary,
                              int rowStride, int rowOffset, float temperature, int topK, float topP, float minP, uint32_t seed);
/* [257] PenalizeRows (penalize_rows_f32, PtxKernels.Decoding.cs:352-433): work[r,:] = logits row r, then every distinct
 * token among the last min(length[0], lastN, capacity) entries of history[r,:] (a ring indexed modulo capacity) gets
 * x = x > 0 ? x / repeat : x * repeat; x -= presence + frequency * occurrences. */
NS_API int ns_f32_penalize_rows(ns_device_t dev, uint64_t logits, uint64_t work, uint64_t history, uint64_t length, int rows, int vocabulary,
                                int rowStride, int rowOffset, int capacity, int lastN, float repeat, float presence, float frequency);
/* [261] HistoryPush (history_push_f32, PtxKernels.Decoding.cs:435-447): history[r, length[0] % capacity] = ids[r]. */
NS_API int ns_f32_history_push(ns_device_t dev, uint64_t ids, uint64_t history, uint64_t length, int rows, int capacity);

/* ------------------------------------------------------------------------------------------------
 * Key/value cache and attention.  Replaces KeyValueCache + Tensor.WriteKeyValues (Layers/Decoding.cs:14-35,
 * Tensor.Decoding.cs:62-66 -> kv_write_f32, PtxKernels.Decoding.cs:130-143) and the three-kernel attention of
 * MultiHeadAttention.ForwardCached / ForwardCore (Layers/Attention.cs:46-118: matmul_f32, scale_mask_softmax_f32,
 * matmul_f32 with the score tensor in memory).  Keys, values, queries and outputs are bf16.
 * ------------------------------------------------------------------------------------------------ */

/* Two zero-initialised pools (keys, values) of bf16 [num_pages, heads, page_size, head_dim]; head_dim 32, 64 or 128.
 * A page table (int32 [batch, max_pages], device memory, owned by the caller) maps (sequence, position / page_size)
 * to a page; the identity table gives the reference's contiguous cache. */
NS_API int ns_kv_cache_create(ns_device_t dev, int num_pages, int page_size, int heads, int head_dim, ns_kv_cache_t* cache);
/* The same over pools the caller allocated with ns_alloc (256-byte aligned, num_pages * heads * page_size * head_dim * 2 bytes
 * each) and keeps: the pools of every layer can then live in one allocation that other processes map (ns_ipc_handle). */
NS_API int ns_kv_cache_create_in(ns_device_t dev, int num_pages, int page_size, int heads, int head_dim, uint64_t k_pool, uint64_t v_pool,
                                 ns_kv_cache_t* cache);
NS_API int ns_kv_cache_destroy(ns_kv_cache_t cache);
/* The exchange step between a batch-sharded prompt read and tensor-parallel decoding (several GPUs; no counterpart in the
 * single-device reference, it serves the prompt read of CharGpt.Generate, samples/Shared/Gpt/CharGpt.cs:261-270): `src` holds
 * all heads of this rank's n_seqs sequences (global sequence numbers seq0 ..); for each of them the first pages_used pages of
 * every head are copied into the cache of the rank that owns the head (heads / world consecutive heads per rank):
 * dst_k_pools / dst_v_pools are the `world` ranks' pools as mapped in this process (its own pool at its own rank),
 * dst_table the page table the destination caches share.  `layers` > 1 copies that many layers in the one launch: `src` and
 * the pool addresses are layer 0's, the pools of layer l lie l * src_layer_stride / dst_layer_stride BYTES further on (all
 * layers of a model in one allocation, same geometry and page tables).  Plain 16-byte stores over NVLink; queued on the stream. */
NS_API int ns_kv_scatter_heads(ns_device_t dev, ns_kv_cache_t src, uint64_t src_table, int src_max_pages, int n_seqs, int seq0, int pages_used,
                               const uint64_t* dst_k_pools, const uint64_t* dst_v_pools, int world, int dst_heads, int dst_num_pages,
                               uint64_t dst_table, int dst_max_pages, int layers, uint64_t src_layer_stride, uint64_t dst_layer_stride);
NS_API int ns_kv_cache_pools(ns_kv_cache_t cache, uint64_t* k_pool, uint64_t* v_pool, uint64_t* bytes_each);

/* cache[b, pos + i, h, :] = k/v[(b * steps + i) * src_stride + h * head_dim + :] for i < steps; pos is an int32 in
 * device memory (pos_dev), so a captured graph stays valid at every position (Layers/Decoding.cs:81-82). */
NS_API int ns_kv_append(ns_device_t dev, ns_kv_cache_t cache, uint64_t k, uint64_t v, int64_t src_stride, uint64_t page_table,
                        int max_pages, uint64_t pos_dev, int batch, int steps);

/* o[b, i, h, :] = softmax_j((q[b, i, h, :] . K[b, j, h, :]) * scale) . V[b, j, h, :] over cached positions j <= pos + i.
 * q element (b, i, h, d) at q[(b * steps + i) * q_stride + h * head_dim + d], o likewise with o_stride.
 * Uses the device object's scratch block when the work is split along the cache.  The output bits of a row depend on the row's
 * cached data, max_pages and the page size only, not on batch or steps (a sequence decoded in a batch equals the sequence
 * decoded alone, as DecodingTests.cs:100-142 asks of the reference): the cache is walked in chunks fixed by its capacity and
 * the chunks' partial results are folded in chunk order, by one CTA or by several. */
NS_API int ns_attention_decode(ns_device_t dev, ns_kv_cache_t cache, uint64_t q, int64_t q_stride, uint64_t o, int64_t o_stride,
                               uint64_t page_table, int max_pages, uint64_t pos_dev, int batch, int steps, float scale);

/* ns_attention_decode, and the output rows [batch * steps, heads * head_dim] (o_stride = heads * head_dim) also leave as
 * int8 rows q_out with one float scale per row in q_scale -- ns_quantize_rows_i8 of the bf16 output, bit for bit, done
 * by the last CTA that finishes a row.  This is the input of the attention output projection (Layers/Attention.cs:113-117);
 * it saves the decoding step a launch.  batch * steps <= 4000. */
NS_API int ns_attention_decode_quant(ns_device_t dev, ns_kv_cache_t cache, uint64_t q, int64_t q_stride, uint64_t o, int64_t o_stride,
                                     uint64_t page_table, int max_pages, uint64_t pos_dev, int batch, int steps, float scale, uint64_t q_out,
                                     uint64_t q_scale);

/* Attention over a whole sequence (MultiHeadAttention.ForwardCore, Layers/Attention.cs:46-91) without the
 * [T, T] score tensor: o[b, h, i, :] = softmax_j((q[b,h,i,:] . k[b,h,j,:]) * scale + mask) . v[b,h,j,:], mask = -inf
 * for j > i when causal.  head_dim must be 128.  Element (b, h, s, d) of each tensor sits at
 * base[b * strides[0] + h * strides[1] + s * strides[2] + d] (strides in elements, multiples of 8), so both
 * [batch, heads, seq, 128] buffers and the [batch * seq, 3 * D] output of a fused QKV product can be used in place. */
NS_API int ns_attention_prefill(ns_device_t dev, uint64_t q, uint64_t k, uint64_t v, uint64_t o, int batch, int heads, int seq, int head_dim,
                                const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                                float scale, int causal);

/* ------------------------------------------------------------------------------------------------
 * Linear objects.  Replace Linear's parameters and ForwardCore (Layers/Linear.cs:25-47): the float [K, N]
 * weight of the reference (host memory, as read from its weight file) is transposed to one row per output
 * channel, converted (NS_BF16) or quantised per output channel (NS_I8) and kept on the device; the product and
 * the bias / bias+GELU / bias+residual kernels that follow it in the reference run as one kernel.
 * ------------------------------------------------------------------------------------------------ */

/* w_kn: float [K, N] on the host; bias: float [N] on the host or NULL.
 * split NS_SPLIT_COLUMN: this rank owns N / tp_size outputs.  The columns are taken as col_groups equal blocks and
 * each rank owns the same slice of every block (col_groups = 3 for a fused [Q|K|V] projection, so a rank gets the
 * Q, K and V columns of its own heads; 1 otherwise).  split NS_SPLIT_ROW: this rank owns K / tp_size inputs and its
 * forward yields a partial sum (see ns_bias_residual).  The reference has no counterpart for the split. */
NS_API int ns_linear_create(ns_device_t dev, int K, int N, int mode, const float* w_kn, const float* bias, int split, int col_groups,
                            int tp_rank, int tp_size, ns_linear_t* linear);
NS_API int ns_linear_destroy(ns_linear_t linear);
NS_API int ns_linear_info(ns_linear_t linear, int* k_local, int* n_local, int* mode, uint64_t* w, uint64_t* w_scale, uint64_t* bias);
/* y[M, N_local] = epilogue(x . W^T).  NS_I8 layer: x int8 [M, K_local] with x_scale float [M] (from ns_quantize_rows_i8 or
 * ns_layernorm with NS_I8 output).  NS_BF16 layer: x bf16, x_scale 0.  A row shard (tp_size > 1) takes NS_EPI_NONE only. */
NS_API int ns_linear_forward(ns_device_t dev, ns_linear_t linear, uint64_t x, uint64_t x_scale, int M, int epilogue, uint64_t residual,
                             int residual_dtype, int out_dtype, uint64_t y);
/* Host-to-host forward: y_host[M, N] = epilogue(x_host[M, K] . W^T), float32 in host memory on both sides (pinned memory
 * for full speed).  Replaces the caller's sequence Tensor.From -> Linear.Forward -> Tensor.ToArray (Tensor.cs:87,204;
 * Backend.Upload / Download, Backends/Backend.cs:77-79, CudaBackend.cs:283-301), whose three steps run one after another:
 * here row chunks of `chunk_rows` (0 = about 32 MiB each, shorter at both ends) flow through an upload stream, the
 * device's stream (quantise or convert, product) and a download stream, so both copy directions and the compute overlap,
 * also between back-to-back calls.  x_host is read from the moment of the call; ns_stream_sync (or an event recorded
 * after the call) covers the downloads into y_host.  epilogue: NS_EPI_NONE, NS_EPI_BIAS or NS_EPI_BIAS_GELU.  Not
 * capturable; not for tensor-parallel shards. */
NS_API int ns_linear_forward_host(ns_device_t dev, ns_linear_t linear, const float* x_host, int M, int epilogue, float* y_host, int chunk_rows);

/* ------------------------------------------------------------------------------------------------
 * Fused row kernels of the decoding step.  With the few rows of a step, time goes to the NUMBER of launches; these
 * take over a product's epilogue so that the split-K second kernel and the row operator that follows are one launch.
 * ------------------------------------------------------------------------------------------------ */
/* The int8 product of `linear` WITHOUT its epilogue: exact int32 partial sums [splits, M, N_local] are left in the device
 * object's scratch block (valid until the next call on this device that uses the scratch block: another product with a
 * split K, or decode attention with a split cache); `partial` and `splits` describe them.  M * N_local <= 2^24. */
NS_API int ns_linear_forward_partial(ns_device_t dev, ns_linear_t linear, uint64_t x, int M, uint64_t* partial, int* splits);
/* x_out[m,n] = bf16(((float) sum_s partial[s,m,n] * x_scale[m]) * w_scale[n] + bias[n] + residual[m,n]) (residual bf16, may be
 * 0), then, when gamma != 0: q, q_scale = int8 row quantisation of bf16(LayerNorm(x_out)) -- the input of the next product.
 * Replaces x + Linear(...) followed by LayerNorm (Layers/Attention.cs:201-205; add_rowvec_f32, add_f32,
 * layernorm_fused_f32 PtxKernels.Decoding.cs:61-90) for a row-split or K-split product.  q_scale may be x_scale. */
NS_API int ns_finish_norm_quant(ns_device_t dev, uint64_t partial, int splits, ns_linear_t linear, uint64_t x_scale, uint64_t residual,
                                int64_t rows, uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q, uint64_t q_scale);
/* q, q_scale = int8 row quantisation of bf16(GELU(((float) sum_s partial[s,m,n] * x_scale[m]) * w_scale[n] + bias[n])): the input
 * of FF2 straight from FF1's partial sums.  Replaces Linear + BiasGelu (Layers/Attention.cs:207-209; bias_gelu_f32,
 * PtxKernels.Decoding.cs:93-114) for a K-split product followed by the next product's row quantisation.  N_local a multiple of
 * 256 up to 8192, buffers 16-byte aligned; q_scale may be x_scale. */
NS_API int ns_finish_gelu_quant(ns_device_t dev, uint64_t partial, int splits, ns_linear_t linear, uint64_t x_scale, int64_t rows, uint64_t q,
                                uint64_t q_scale);
/* qkv[m, 0:3d] = bf16(dequantised partial sums + bias) of the fused QKV product, and its K and V thirds appended to the cache
 * at position pos_dev[0] + step (as ns_kv_append).  Replaces the product's epilogue + KeyValueWrite
 * (Layers/Attention.cs:98-118; kv_write_f32 PtxKernels.Decoding.cs:130-143). */
NS_API int ns_finish_kv_append(ns_device_t dev, uint64_t partial, int splits, ns_linear_t linear, uint64_t x_scale, int batch, int steps,
                               uint64_t qkv, ns_kv_cache_t cache, uint64_t page_table, int max_pages, uint64_t pos_dev);

/* One launch per Linear of the decoding step: the int8 product of `linear` (x int8 [rows, K_local], x_scale float [rows]) and, as a
 * second phase of the SAME kernel after a device-wide arrival counter, the row operator that follows it in the decoder
 * block (TransformerEncoderLayer.ForwardCached, Layers/Attention.cs:201-211).  rows <= 256 (the few rows of a decoding
 * step); N_local a multiple of 256 up to 8192 for the two row-wise forms; buffers 16-byte aligned.  Results are
 * bit-identical to the two-launch forms above.  All three use the device object's scratch block and synchronisation words:
 * calls on one device object must not overlap on the GPU.
 *   ns_linear_forward_norm_quant = ns_linear_forward_partial + ns_finish_norm_quant   (attention output projection, FF2)
 *   ns_linear_forward_gelu_quant = product + bias + GELU -> bf16 -> ns_quantize_rows_i8 (FF1; bias_gelu_f32, PtxKernels.Decoding.cs:93-114)
 *   ns_linear_forward_kv_append  = ns_linear_forward_partial + ns_finish_kv_append    (fused QKV projection) */
NS_API int ns_linear_forward_norm_quant(ns_device_t dev, ns_linear_t linear, uint64_t x, uint64_t x_scale, uint64_t residual, int64_t rows,
                                        uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q, uint64_t q_scale);
NS_API int ns_linear_forward_gelu_quant(ns_device_t dev, ns_linear_t linear, uint64_t x, uint64_t x_scale, int64_t rows, uint64_t q, uint64_t q_scale);
NS_API int ns_linear_forward_kv_append(ns_device_t dev, ns_linear_t linear, uint64_t x, uint64_t x_scale, int batch, int steps, uint64_t qkv,
                                       ns_kv_cache_t cache, uint64_t page_table, int max_pages, uint64_t pos_dev);

/* ------------------------------------------------------------------------------------------------
 * Tensor parallelism over NCCL.  No counterpart in the reference (single device; Device.cs:54-64).
 * ------------------------------------------------------------------------------------------------ */
/* y = (partial + bias[col]) + residual: what a row-parallel layer does after its partial sums (float [rows, cols])
 * have been reduced across ranks.  bias and residual may be 0. */
NS_API int ns_bias_residual(ns_device_t dev, uint64_t partial, uint64_t bias, uint64_t residual, int residual_dtype, int64_t rows, int cols,
                            int out_dtype, uint64_t y);
/* Greedy token over a vocabulary split by columns: per row the first maximum of this rank's slice
 * (value, column + col_offset) ... */
NS_API int ns_argmax_partial(ns_device_t dev, uint64_t x, int rows, int cols, int64_t row_stride, int col_offset, uint64_t out_val, uint64_t out_idx);
/* ... and the merge of the gathered [parts, rows] pairs: largest value, ties to the smallest column (first maximum wins). */
NS_API int ns_argmax_merge(ns_device_t dev, uint64_t vals, uint64_t idx, int parts, int rows, uint64_t ids);

/* id128: 128 bytes, made on one rank and given to the others by the host program. */
NS_API int ns_comm_unique_id(void* id128);
NS_API int ns_comm_init_rank(ns_device_t dev, const void* id128, int rank, int size, ns_comm_t* comm);
NS_API int ns_comm_info(ns_comm_t comm, int* rank, int* size, int* nccl_version);
/* In-place sum over ranks / gather of `count` elements per rank, queued on the device's stream (capturable). */
NS_API int ns_allreduce(ns_device_t dev, ns_comm_t comm, uint64_t buf, int64_t count, int dtype);
NS_API int ns_allgather(ns_device_t dev, ns_comm_t comm, uint64_t src, uint64_t dst, int64_t count, int dtype);
NS_API int ns_comm_async_error(ns_comm_t comm, int* nccl_result);
NS_API int ns_comm_abort(ns_comm_t comm);     /* after a peer failed: does not wait for the peers */
NS_API int ns_comm_destroy(ns_comm_t comm);

/* The exchange step of the tensor-parallel decoder over peer memory (one process per GPU, up to 8 ranks of one machine).
 * Every rank creates a group (one device block: flags + two slots of `slot_bytes`), hands its 64-byte handle to the other
 * ranks by the host program's own means, and connects with the `world` handles in rank order.  New: the reference has no
 * multi-GPU code (Tensor.To goes through a host array, Tensor.cs:244-253). */
NS_API int ns_peer_group_create(ns_device_t dev, int rank, int world, uint64_t slot_bytes, ns_peer_group_t* group);
NS_API int ns_peer_group_handle(ns_peer_group_t group, void* handle64);
/* handles: world x 64 bytes in rank order.  Null: the other ranks become stand-ins that never arrive (a test of the bounded
 * wait on one GPU: the next ns_tp_reduce_norm_quant gives up after about a second with status 400 + the missing rank). */
NS_API int ns_peer_group_connect(ns_peer_group_t group, const void* handles);
/* Device address of this rank's slot (0 or 1): the row-parallel product writes its float partial rows [rows, cols] there. */
NS_API int ns_peer_group_slot(ns_peer_group_t group, int slot, uint64_t* ptr);
/* x_out[m,n] = bf16(sum over ranks, in rank order, of their slot's partial[m,n] + bias[n] + residual[m,n]) (bias float, residual
 * bf16, either may be 0), then, when gamma != 0: q, q_scale = int8 row quantisation of bf16(LayerNorm(x_out)).  One kernel in
 * place of all-reduce + add_rowvec_f32 + add_f32 + layernorm_fused_f32 (Layers/Attention.cs:201-205,
 * PtxKernels.Decoding.cs:61-90).  Every rank must call it for the same slot in the same order; a rank that waits for a peer
 * for about a second gives up and reports NS_ERR_KERNEL at the next ns_stream_sync.  rows <= 64 x SM count, cols a multiple
 * of 256 up to 8192. */
NS_API int ns_tp_reduce_norm_quant(ns_device_t dev, ns_peer_group_t group, int slot, uint64_t bias, uint64_t residual, int64_t rows, int cols,
                                   uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q, uint64_t q_scale);
/* The row-parallel product of `linear` (a row shard: x int8 [rows, K_local]) AND the exchange above in one launch: the kernel
 * writes this rank's float partial rows into its slot, all its CTAs arrive on a device-wide counter, one CTA then raises
 * the ranks' flags and the CTAs that own rows wait for every rank's flag and finish as ns_tp_reduce_norm_quant does.  K is
 * not split inside a rank.  rows <= min(256, SM count).  Same call order rule and bounded waits (status 400 + rank for a
 * missing rank, 410 for this rank's own CTAs).  Serves x + Linear(...) -> LayerNorm of Layers/Attention.cs:201-205 on
 * several GPUs; no counterpart in the single-device reference. */
NS_API int ns_linear_forward_tp_norm_quant(ns_device_t dev, ns_linear_t linear, ns_peer_group_t group, int slot, uint64_t x, uint64_t x_scale,
                                           uint64_t residual, int64_t rows, uint64_t x_out, uint64_t gamma, uint64_t beta, float eps, uint64_t q,
                                           uint64_t q_scale);
NS_API int ns_peer_group_destroy(ns_peer_group_t group);

#ifdef __cplusplus
}
#endif
#endif /* NS_B200_H */
