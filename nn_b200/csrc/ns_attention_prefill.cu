// Causal attention forward for a whole sequence (prefill), head_dim 128, bf16 in / bf16 out, on the
// sm_100a tensor cores: S = Q.K^T and O += P.V are tcgen05.mma with accumulators in tensor memory,
// Q/K/V tiles arrive by TMA, the softmax is computed online (running maximum and sum per row) so the
// [T, T] score tensor never exists.
//
// Reference path: MultiHeadAttention.ForwardCore (src/NeuralSharp/Layers/Attention.cs:46-91): three
// narrow+permute copies, matmul_f32 (Q.K^T) into a [N*H, T, T] tensor, scale_mask_softmax_f32 with an
// additive -1e9 mask (one thread per row, PtxKernels.Decoding.cs:24-58), matmul_f32 (P.V), permute back.
// Skipping the key blocks above the diagonal is exact: exp(-1e9 - max) is 0 in float.  The head
// split/merge copies disappear because the tensor maps take the (batch, head, position) strides of
// the caller's buffers.
//
// One persistent CTA per SM draws (batch, head, 128 query rows) tiles from a global counter (tiles of one head adjacent,
// heavy tiles first); tensor memory and barriers are set up once, and the next tile's Q and first K blocks are loaded
// (and its first scores computed) while the current tile's output is merged and stored.  Against one CTA per tile this
// gave 65 -> 56 us at 512 positions and 403 -> 369 us at 2048 (8 x 32 heads); a static round-robin share per CTA lost
// 8 % at 8192 positions to the tail, the counter does not.  320 threads:
//   warp 0      one lane issues TMA loads: Q once, then K_j and V_j (128 keys each) into a 2-stage ring
//   warp 1      one lane issues the MMAs: S_{j+1} = Q.K_{j+1}^T is issued before P_j.V_j, so the tensor
//               cores work on the next scores while the softmax warps handle block j
//   warps 2..9  softmax, in two groups of four warps.  Group g owns the key blocks of parity g with its own score
//               buffer, P buffer, output accumulator O_g and running (maximum, sum): thread r owns query row r
//               (= tensor-memory lane r), reads its 128 scores with tcgen05.ld, masks, updates max/sum, writes P_j as
//               bf16 into shared memory in the 128-byte-swizzled K-major layout the MMA reads, and rescales O_g in
//               tensor memory when the row maximum grew by more than 2^8 (otherwise the old reference maximum is
//               kept, which is exact because the sum and O_g share it).  The groups never wait for each other inside
//               the loop, and the two warps on one scheduler are in different phases of their blocks, so one keeps
//               the exponential unit busy while the other waits on tensor memory or writes P.  After the last block
//               the two partial results of a row are merged (weights exp2(m_g - m) / l), and each group stores 64 of
//               the 128 output dims through shared memory with TMA stores.
// Tensor memory: S_0 at columns [0,128), S_1 at [128,256), O_0 at [256,384), O_1 at [384,512).
// Every mbarrier wait is bounded; a wait that runs out reports a status code and the CTA leaves.
#include <math.h>

#include "ns_common.cuh"

namespace {

constexpr int FA_THREADS = 320;  // producer warp, MMA warp, 8 softmax warps
constexpr int FA_BLOCK = 128;  // query rows per CTA = keys per block = head_dim
constexpr uint32_t FA_TILE_BYTES = 128 * 128 * 2;  // 32 KB: two [128 x 64] halves of 16 KB
constexpr uint32_t FA_HALF_BYTES = 128 * 64 * 2;
constexpr uint32_t FA_SMEM_BYTES = 1024 + 7 * FA_TILE_BYTES + 256;  // Q, 2 x (K, V), 2 x P, barriers

struct FaParams {
    int batch, heads, seq;
    int causal;
    float scale_log2;  // scale * log2(e)
    int* status;
    int* tile_counter; // zeroed before the launch: CTAs draw their tiles from it in order
};

struct FaMaps {
    CUtensorMap q, k, v;  // box [64 dims, 128 rows]
    CUtensorMap o;        // box [64 dims, 32 rows] (one softmax warp's rows)
};

__device__ __forceinline__ float fa_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// bf16(lo) in the low half, bf16(hi) in the high half, both round to nearest even: one instruction
__device__ __forceinline__ uint32_t fa_pack_bf16(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

enum { BAR_Q = 0, BAR_Q_FREE = 1, BAR_K0 = 2, BAR_V0 = 4, BAR_K_EMPTY0 = 6, BAR_V_EMPTY0 = 8, BAR_S_FULL0 = 10, BAR_S_FREE0 = 12, BAR_P_FULL0 = 14,
       BAR_PV_DONE0 = 16, BAR_FIN = 18, BAR_FIN2 = 19, BAR_O_FREE = 20, BAR_TILE0 = 21, BAR_COUNT = 25 };

// Tiles are drawn from a global counter in this order: the tiles of one (batch, head) are adjacent, heavy tiles (late
// query rows see more keys) first -- CTAs that run together then read the same K/V blocks at about the same time and all
// but the first reader hit in L2, and whichever CTA is free takes the next tile, so the CTAs finish together.
struct FaTile {
    int b, h, q0, n_blocks;
};
__device__ __forceinline__ void fa_tile(const FaParams& p, int n_qt, int idx, FaTile& t)
{
    const int qt = n_qt - 1 - idx % n_qt;
    const int bh = idx / n_qt;
    t.b = bh / p.heads;
    t.h = bh % p.heads;
    t.q0 = qt * FA_BLOCK;
    t.n_blocks = p.causal ? qt + 1 : n_qt;
}

__global__ void __launch_bounds__(FA_THREADS, 1) ns_attention_prefill_kernel(const __grid_constant__ FaMaps maps, const FaParams p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag_storage;
    volatile int* abort_flag = &abort_flag_storage;
    const uint32_t smem_base = (ns_smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;
    auto k_smem = [&](int s) { return smem_base + FA_TILE_BYTES * (1 + 2 * s); };
    auto v_smem = [&](int s) { return smem_base + FA_TILE_BYTES * (2 + 2 * s); };
    auto p_smem = [&](int g) { return smem_base + FA_TILE_BYTES * (5 + g); };
    const uint32_t bar_base = smem_base + 7 * FA_TILE_BYTES;
    auto bar = [&](int i) { return bar_base + 8u * i; };
    const uint32_t tmem_slot = bar_base + 8u * BAR_COUNT;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qt = (p.seq + FA_BLOCK - 1) / FA_BLOCK;
    const int total = p.batch * p.heads * n_qt;
    // The producer draws the tile index and hands it to the other roles through a ring of four words, each with its own
    // barrier.  A softmax group with no block in a short tile can lag the producer by more than one tile, which the
    // parity of a single barrier could not tell apart; it cannot lag by four (a tile's first P.V waits until both groups
    // have read out the previous tile's output), so a ring of four is safe.
    const uint32_t tile_ring = bar_base + 8u * BAR_COUNT + 16u;
    auto next_tile = [&](int it, FaTile& t) {
        if (!ns_mbar_wait(bar(BAR_TILE0 + (it & 3)), (it >> 2) & 1, abort_flag, p.status, 300 + 11)) return false;
        int idx;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(idx) : "r"(tile_ring + 4u * (it & 3)) : "memory");
        if (idx < 0) return false;
        fa_tile(p, n_qt, idx, t);
        return true;
    };

    if (threadIdx.x == 0) {
        abort_flag_storage = 0;
        ns_mbar_init(bar(BAR_Q), 1);
        ns_mbar_init(bar(BAR_Q_FREE), 1);
        for (int s = 0; s < 2; s++) {
            ns_mbar_init(bar(BAR_K0 + s), 1);
            ns_mbar_init(bar(BAR_V0 + s), 1);
            ns_mbar_init(bar(BAR_K_EMPTY0 + s), 1);
            ns_mbar_init(bar(BAR_V_EMPTY0 + s), 1);
            ns_mbar_init(bar(BAR_S_FULL0 + s), 1);
            ns_mbar_init(bar(BAR_S_FREE0 + s), 128);
            ns_mbar_init(bar(BAR_P_FULL0 + s), 128);
            ns_mbar_init(bar(BAR_PV_DONE0 + s), 1);
        }
        ns_mbar_init(bar(BAR_FIN), 256);
        ns_mbar_init(bar(BAR_FIN2), 256);
        ns_mbar_init(bar(BAR_O_FREE), 256);
        for (int i = 0; i < 4; i++) ns_mbar_init(bar(BAR_TILE0 + i), 1);
        ns_fence_barrier_init();
        ns_fence_proxy_async();
        ns_prefetch_tensormap(&maps.q);
        ns_prefetch_tensormap(&maps.k);
        ns_prefetch_tensormap(&maps.v);
        ns_prefetch_tensormap(&maps.o);
    }
    if (warp == 1) {
        ns_tmem_alloc(tmem_slot, 512);
        ns_tmem_relinquish();
    }
    ns_tc_fence_before();
    __syncthreads();
    ns_tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
    const int code = 300;

    // Every role walks the same tile sequence.  Key blocks are numbered through ALL tiles of the CTA (gj): block gj uses K/V
    // slot gj & 1, score buffer / softmax group gj & 1, and its barriers are in phase (gj >> 1) & 1, so nothing restarts
    // at a tile boundary: the next tile's Q and first K blocks are loaded, and its first scores computed, while the softmax
    // warps finish and store the current tile.
    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            auto load_k = [&](const FaTile& t, int j, int gj) {
                const int s = gj & 1;
                if (gj >= 2 && !ns_mbar_wait(bar(BAR_K_EMPTY0 + s), ((gj >> 1) - 1) & 1, abort_flag, p.status, code + 1)) return false;
                ns_mbar_expect_tx(bar(BAR_K0 + s), FA_TILE_BYTES);
                ns_tma_load_4d(k_smem(s), &maps.k, bar(BAR_K0 + s), 0, j * FA_BLOCK, t.h, t.b);
                ns_tma_load_4d(k_smem(s) + FA_HALF_BYTES, &maps.k, bar(BAR_K0 + s), 64, j * FA_BLOCK, t.h, t.b);
                return true;
            };
            auto load_v = [&](const FaTile& t, int j, int gj) {
                const int s = gj & 1;
                if (gj >= 2 && !ns_mbar_wait(bar(BAR_V_EMPTY0 + s), ((gj >> 1) - 1) & 1, abort_flag, p.status, code + 1)) return false;
                ns_mbar_expect_tx(bar(BAR_V0 + s), FA_TILE_BYTES);
                ns_tma_load_4d(v_smem(s), &maps.v, bar(BAR_V0 + s), 0, j * FA_BLOCK, t.h, t.b);
                ns_tma_load_4d(v_smem(s) + FA_HALF_BYTES, &maps.v, bar(BAR_V0 + s), 64, j * FA_BLOCK, t.h, t.b);
                return true;
            };
            bool ok = true;
            int gj0 = 0;
            FaTile t;
            for (int it = 0; ok; it++) {
                // Q is free once every Q.K^T of the previous tile has completed
                if (it > 0) ok = ns_mbar_wait(bar(BAR_Q_FREE), (it - 1) & 1, abort_flag, p.status, code + 1);
                if (!ok) break;
                const int idx = atomicAdd(p.tile_counter, 1);
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile_ring + 4u * (it & 3)), "r"(idx < total ? idx : -1) : "memory");
                ns_mbar_arrive(bar(BAR_TILE0 + (it & 3)));
                if (idx >= total) break;
                fa_tile(p, n_qt, idx, t);
                ns_mbar_expect_tx(bar(BAR_Q), FA_TILE_BYTES);
                ns_tma_load_4d(q_smem, &maps.q, bar(BAR_Q), 0, t.q0, t.h, t.b);
                ns_tma_load_4d(q_smem + FA_HALF_BYTES, &maps.q, bar(BAR_Q), 64, t.q0, t.h, t.b);
                // K_j is wanted early (scores are computed two blocks ahead of the softmax), V_j late: K slots are freed by the
                // Q.K^T that read them, V slots by the P.V, and V trails K by one block
                for (int j = 0; j <= t.n_blocks && ok; j++) {
                    if (j < t.n_blocks) ok = load_k(t, j, gj0 + j);
                    if (ok && j >= 1) ok = load_v(t, j - 1, gj0 + j - 1);
                }
                gj0 += t.n_blocks;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = ns_idesc(1, 1, 0, 0, 128, 128);
            constexpr uint32_t idesc_pv = ns_idesc(1, 1, 0, 1, 128, 128);
            const uint64_t desc_k = ns_desc_base(16, 1024);
            const uint64_t desc_v = ns_desc_base(FA_HALF_BYTES, 1024);  // MN-major: 64-dim halves 16 KB apart, 8 key rows 1 KB apart
            auto issue_qk = [&](int gj, bool last_of_tile) {
                const int s = gj & 1;
                const uint32_t d_tmem = tmem_base + s * 128;
                const uint32_t kb = k_smem(s);
#pragma unroll
                for (int kk = 0; kk < 8; kk++) {
                    const uint32_t off = (kk >> 2) * FA_HALF_BYTES + (kk & 3) * 32;
                    ns_mma_f16(d_tmem, ns_desc_at(desc_k, q_smem + off), ns_desc_at(desc_k, kb + off), idesc_qk, kk > 0 ? 1u : 0u);
                }
                ns_tc_commit(bar(BAR_K_EMPTY0 + s));
                ns_tc_commit(bar(BAR_S_FULL0 + s));
                if (last_of_tile) ns_tc_commit(bar(BAR_Q_FREE));
            };
            auto issue_pv = [&](int gj, bool first_of_group_in_tile) {
                const int g = gj & 1;
                const uint32_t o_tmem = tmem_base + 256 + g * 128;
                const uint32_t vb = v_smem(g);
                const uint32_t pb = p_smem(g);
#pragma unroll
                for (int kk = 0; kk < 8; kk++) {
                    const uint64_t a_desc = ns_desc_at(desc_k, pb + (kk >> 2) * FA_HALF_BYTES + (kk & 3) * 32);
                    const uint64_t b_desc = ns_desc_at(desc_v, vb + kk * (16 * 128));
                    ns_mma_f16(o_tmem, a_desc, b_desc, idesc_pv, (!first_of_group_in_tile || kk > 0) ? 1u : 0u);
                }
                ns_tc_commit(bar(BAR_V_EMPTY0 + g));
                ns_tc_commit(bar(BAR_PV_DONE0 + g));
            };
            bool ok = true;
            int gj0 = 0;
            FaTile t;
            for (int it = 0; ok && next_tile(it, t); it++) {
                ok = ns_mbar_wait(bar(BAR_Q), it & 1, abort_flag, p.status, code + 2);
                // Whatever is ready is issued: S_j = Q.K_j^T as soon as K_j has landed and the owning group has read its previous
                // scores out of the buffer, O_g += P_j.V_j as soon as P_j is written (and, for the first P.V of a tile, once the
                // previous tile's output has been read out of the accumulators).
                int qk = 0, pv = 0;
                bool o_free = it == 0;
                long long t_idle = 0;
                uint32_t spins = 0;
                while (ok && pv < t.n_blocks) {
                    bool progressed = false;
                    const int gq = gj0 + qk;
                    if (qk < t.n_blocks && ns_mbar_try_wait(bar(BAR_K0 + (gq & 1)), (gq >> 1) & 1) &&
                        (gq < 2 || ns_mbar_try_wait(bar(BAR_S_FREE0 + (gq & 1)), ((gq >> 1) - 1) & 1))) {
                        ns_tc_fence_after();
                        issue_qk(gq, qk == t.n_blocks - 1);
                        qk++;
                        progressed = true;
                    }
                    const int gp = gj0 + pv;
                    if (pv < qk && ns_mbar_try_wait(bar(BAR_P_FULL0 + (gp & 1)), (gp >> 1) & 1) &&
                        ns_mbar_try_wait(bar(BAR_V0 + (gp & 1)), (gp >> 1) & 1)) {
                        if (!o_free) o_free = ns_mbar_try_wait(bar(BAR_O_FREE), (it - 1) & 1);
                        if (o_free) {
                            ns_tc_fence_after();
                            issue_pv(gp, pv < 2);
                            pv++;
                            progressed = true;
                        }
                    }
                    if (progressed) {
                        spins = 0;
                    } else if ((++spins & 0x3F) == 0) {
                        if (spins == 0x40) t_idle = clock64();
                        if (*abort_flag != 0) ok = false;
                        else if (clock64() - t_idle > NS_WAIT_LIMIT_CYCLES) {
                            *reinterpret_cast<volatile int*>(p.status) = code + 5;
                            *abort_flag = 1;
                            __threadfence_block();
                            ok = false;
                        }
                    }
                }
                gj0 += t.n_blocks;
            }
        }
    } else {
        // ------------------------------------------------------------ softmax / correction / output
        // Two groups of four warps.  Group g owns the key blocks with gj & 1 == g: its own score buffer S_g, its own P_g in
        // shared memory, its own output accumulator O_g and its own running maximum and sum, so the two groups never
        // wait for each other inside a tile and the two warps that share a scheduler are in different phases of their
        // blocks (one waits on tensor memory or writes P while the other keeps the exponential unit busy).  The two
        // partial results of a row are merged once per tile, after its last block.
        const int quad = warp & 3;
        const int g = (warp - 2) >> 2;
        const int r = quad * 32 + lane;          // row inside the tile = tensor-memory lane
        const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
        const uint32_t s_addr = lane_addr + g * 128;
        const uint32_t o_addr = lane_addr + 256 + g * 128;
        const uint32_t pb = p_smem(g);
        const uint32_t xch_mine = pb + r * 8, xch_other = p_smem(g ^ 1) + r * 8;
        bool ok = true;
        int gj0 = 0;
        int kg = 0;                               // blocks this group has handled so far, over all tiles
        FaTile t;
        for (int it = 0; ok && next_tile(it, t); it++) {
            const int qi = t.q0 + r;             // absolute query position
            float m_ref = -INFINITY;             // reference maximum of this group's blocks of the tile (raw score units)
            float l_run = 0.0f;                  // sum of this group's exponentials relative to m_ref
            int n_mine = 0;
            for (int j = (g - gj0) & 1; j < t.n_blocks && ok; j += 2, n_mine++, kg++) {
                ok = ns_mbar_wait(bar(BAR_S_FULL0 + g), kg & 1, abort_flag, p.status, code + 7);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ns_tc_fence_after();
                uint32_t sb[128];
                {
                    uint32_t t0[32], t1[32], t2[32], t3[32];
                    ns_tmem_ld32(s_addr, t0);
                    ns_tmem_ld32(s_addr + 32, t1);
                    ns_tmem_ld32(s_addr + 64, t2);
                    ns_tmem_ld32(s_addr + 96, t3);
                    ns_tc_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; c++) { sb[c] = t0[c]; sb[32 + c] = t1[c]; sb[64 + c] = t2[c]; sb[96 + c] = t3[c]; }
                }
                ns_tc_fence_before();
                ns_mbar_arrive(bar(BAR_S_FREE0 + g));
                // mask: keys after the query (causal) or past the end of the sequence
                const int kv0 = j * FA_BLOCK;
                const bool need_mask = (p.causal && kv0 + 127 > t.q0) || kv0 + 128 > p.seq;
                float mx;
                if (need_mask) {
                    mx = -INFINITY;
#pragma unroll
                    for (int c = 0; c < 128; c++) {
                        const int kj = kv0 + c;
                        const bool dead = (p.causal && kj > qi) || kj >= p.seq;
                        if (dead) sb[c] = 0xFF800000u;  // -inf
                        mx = fmaxf(mx, __uint_as_float(sb[c]));
                    }
                } else {
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int c = 0; c < 128; c += 4) {
                        m4[0] = fmaxf(m4[0], __uint_as_float(sb[c])); m4[1] = fmaxf(m4[1], __uint_as_float(sb[c + 1]));
                        m4[2] = fmaxf(m4[2], __uint_as_float(sb[c + 2])); m4[3] = fmaxf(m4[3], __uint_as_float(sb[c + 3]));
                    }
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                }
                // reference maximum: raised only when the row maximum outgrew it by more than 8 / scale_log2
                float alpha = 1.0f;
                bool rescale = false;
                if (mx != -INFINITY && (m_ref == -INFINITY || (mx - m_ref) * p.scale_log2 > 8.0f)) {
                    alpha = m_ref == -INFINITY ? 0.0f : fa_exp2((m_ref - mx) * p.scale_log2);
                    rescale = m_ref != -INFINITY;
                    m_ref = mx;
                }
                const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
                const float neg_m = -m_use * p.scale_log2;
                float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                uint32_t pk[64];
#pragma unroll
                for (int c = 0; c < 128; c += 4) {
                    // one MUFU each (results below 2^-126 flush to zero, which is what P wants) and one conversion per pair
                    const float p0 = fa_exp2(fmaf(__uint_as_float(sb[c]), p.scale_log2, neg_m));
                    const float p1 = fa_exp2(fmaf(__uint_as_float(sb[c + 1]), p.scale_log2, neg_m));
                    const float p2 = fa_exp2(fmaf(__uint_as_float(sb[c + 2]), p.scale_log2, neg_m));
                    const float p3 = fa_exp2(fmaf(__uint_as_float(sb[c + 3]), p.scale_log2, neg_m));
                    s4[0] += p0; s4[1] += p1; s4[2] += p2; s4[3] += p3;
                    pk[c >> 1] = fa_pack_bf16(p0, p1);
                    pk[(c >> 1) + 1] = fa_pack_bf16(p2, p3);
                }
                l_run = l_run * alpha + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
                // P_g (and, within a tile, O_g) belong to this group's previous P.V until it has completed
                if (kg > 0) {
                    ok = ns_mbar_wait(bar(BAR_PV_DONE0 + g), (kg - 1) & 1, abort_flag, p.status, code + 8);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    ns_tc_fence_after();
                    if (n_mine > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
                        for (int c = 0; c < 4; c++) {
                            uint32_t ob[32];
                            ns_tmem_ld32(o_addr + c * 32, ob);
                            ns_tc_wait_ld();
#pragma unroll
                            for (int q = 0; q < 32; q++) ob[q] = __float_as_uint(__uint_as_float(ob[q]) * alpha);
                            ns_tmem_st32(o_addr + c * 32, ob);
                        }
                        ns_tc_wait_st();
                    }
                }
                // P_j -> shared memory, K-major halves of 64 keys, 16-byte piece q of row r at q ^ (r & 7)
#pragma unroll
                for (int hf = 0; hf < 2; hf++)
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const uint32_t addr = pb + hf * FA_HALF_BYTES + r * 128 + ((q ^ (r & 7)) * 16);
                        ns_st_shared_v4(addr, pk[hf * 32 + 4 * q], pk[hf * 32 + 4 * q + 1], pk[hf * 32 + 4 * q + 2], pk[hf * 32 + 4 * q + 3]);
                    }
                ns_fence_proxy_async();
                ns_tc_fence_before();
                ns_mbar_arrive(bar(BAR_P_FULL0 + g));
            }
            // this group's last P.V so far (of this tile, or of an earlier one if it had no block here): its P buffer is free
            if (ok && kg > 0) {
                ok = ns_mbar_wait(bar(BAR_PV_DONE0 + g), (kg - 1) & 1, abort_flag, p.status, code + 9);
                ok = __all_sync(0xffffffffu, ok);
            }
            // merge the two groups: (m, l) of each row go through the first kilobyte of the group's own P buffer
            if (ok) {
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xch_mine), "f"(m_ref), "f"(l_run) : "memory");
                ns_tc_fence_before();
                ns_mbar_arrive(bar(BAR_FIN));
                ok = ns_mbar_wait(bar(BAR_FIN), it & 1, abort_flag, p.status, code + 10);
                ok = __all_sync(0xffffffffu, ok);
            }
            float m_o = -INFINITY, l_o = 0.0f;
            if (ok) {
                ns_tc_fence_after();
                asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(m_o), "=f"(l_o) : "r"(xch_other) : "memory");
                // both groups have read before either writes its P buffer again (the next tile's first P, or the staging below)
                ns_mbar_arrive(bar(BAR_FIN2));
                ok = ns_mbar_wait(bar(BAR_FIN2), it & 1, abort_flag, p.status, code + 10);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                const float m_all = fmaxf(m_ref, m_o);
                const float a_mine = m_ref == -INFINITY ? 0.0f : fa_exp2((m_ref - m_all) * p.scale_log2);
                const float a_other = m_o == -INFINITY ? 0.0f : fa_exp2((m_o - m_all) * p.scale_log2);
                // Which group got the tile's even-numbered key blocks depends on how many blocks this CTA has walked before
                // (tiles are drawn from a counter at run time).  The result must not: the two partial results are combined
                // in the order (even blocks, odd blocks) of the TILE, whichever group holds which, with every rounding spelt out.
                const bool mine_even = ((g - gj0) & 1) == 0;
                const float l_even = mine_even ? l_run : l_o, a_even = mine_even ? a_mine : a_other;
                const float l_odd = mine_even ? l_o : l_run, a_odd = mine_even ? a_other : a_mine;
                const float l_tot = __fadd_rn(__fmul_rn(l_even, a_even), __fmul_rn(l_odd, a_odd));
                const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
                const float w_even = __fmul_rn(a_even, inv), w_odd = __fmul_rn(a_odd, inv);
                const uint32_t o_mine = lane_addr + 256 + g * 128, o_other = lane_addr + 256 + (g ^ 1) * 128;
                // group g finishes output dims [64 g, 64 g + 64): (O_mine w_mine + O_other w_other) -> bf16 -> the upper half of
                // its P buffer -> one TMA store per warp.  An accumulator that was not written in this tile (a group without
                // blocks) holds another tile's values: its weight is zero and it is not read.
                const uint32_t stage = pb + FA_HALF_BYTES;
                const bool have_mine = n_mine > 0;
                const bool have_other = t.n_blocks >= 2 || !have_mine;   // uniform over the CTA: the other group had a block
#pragma unroll 1
                for (int c = 0; c < 2; c++) {
                    uint32_t oa[32], ob[32];
#pragma unroll
                    for (int q = 0; q < 32; q++) { oa[q] = 0u; ob[q] = 0u; }
                    if (have_mine) ns_tmem_ld32(o_mine + g * 64 + c * 32, oa);
                    if (have_other) ns_tmem_ld32(o_other + g * 64 + c * 32, ob);
                    ns_tc_wait_ld();
                    uint32_t w[16];
#pragma unroll
                    for (int q = 0; q < 16; q++) {
                        // a written accumulator row is finite (a row without live keys in a group's blocks is a sum of zeros)
                        const float e0 = __uint_as_float(mine_even ? oa[2 * q] : ob[2 * q]), d0 = __uint_as_float(mine_even ? ob[2 * q] : oa[2 * q]);
                        const float e1 = __uint_as_float(mine_even ? oa[2 * q + 1] : ob[2 * q + 1]), d1 = __uint_as_float(mine_even ? ob[2 * q + 1] : oa[2 * q + 1]);
                        const float x0 = fmaf(d0, w_odd, __fmul_rn(e0, w_even));
                        const float x1 = fmaf(d1, w_odd, __fmul_rn(e1, w_even));
                        w[q] = fa_pack_bf16(x0, x1);
                    }
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int piece = c * 4 + q;  // 16-byte piece inside the 128-byte row
                        const uint32_t addr = stage + r * 128 + ((piece ^ (r & 7)) * 16);
                        ns_st_shared_v4(addr, w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    }
                }
                // the accumulators may be overwritten by the next tile's first P.V
                ns_tc_fence_before();
                ns_mbar_arrive(bar(BAR_O_FREE));
                ns_fence_proxy_async();
                __syncwarp();
                if (lane == 0 && t.q0 + quad * 32 < p.seq) {
                    ns_tma_store_4d(&maps.o, stage + quad * 32 * 128, g * 64, t.q0 + quad * 32, t.h, t.b);
                    ns_bulk_commit();
                    ns_bulk_wait_read<0>();
                }
                __syncwarp();
            }
            gj0 += t.n_blocks;
        }
    }

    // ---------------------------------------------------------------- teardown
    ns_tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0 && threadIdx.x == 0) {
        long long t0 = clock64();
        while (clock64() - t0 < 400000) { }
    }
    __syncthreads();
    if (warp == 1) {
        ns_tc_fence_after();
        ns_tmem_dealloc(tmem_base, 512);
    }
}

int make_map(CUtensorMap* m, uint64_t base, int batch, int heads, int seq, int64_t sb, int64_t sh, int64_t ss, uint32_t box_rows)
{
    uint64_t dims[4] = {128, (uint64_t)seq, (uint64_t)heads, (uint64_t)batch};
    uint64_t strides[3] = {(uint64_t)ss * 2, (uint64_t)sh * 2, (uint64_t)sb * 2};
    uint32_t box[4] = {64, box_rows, 1, 1};
    return ns_make_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, reinterpret_cast<const void*>(base), dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

extern "C" int ns_attention_prefill(ns_device_t h, uint64_t q, uint64_t k, uint64_t v, uint64_t o, int batch, int heads, int seq, int head_dim,
                                    const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                                    float scale, int causal)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(q && k && v && o && q_strides && k_strides && v_strides && o_strides, NS_ERR_ARGUMENT, "ns_attention_prefill: null argument");
    NS_REQUIRE(head_dim == 128, NS_ERR_ARGUMENT, "ns_attention_prefill: head_dim must be 128 (got %d)", head_dim);
    NS_REQUIRE(batch > 0 && heads > 0 && seq > 0, NS_ERR_ARGUMENT, "ns_attention_prefill: bad shape");
    const int n_qt = (seq + FA_BLOCK - 1) / FA_BLOCK;
    NS_REQUIRE((int64_t)batch * heads * n_qt < (1LL << 31), NS_ERR_ARGUMENT, "ns_attention_prefill: too many tiles");
    FaMaps maps;
    rc = make_map(&maps.q, q, batch, heads, seq, q_strides[0], q_strides[1], q_strides[2], 128);
    if (rc == NS_OK) rc = make_map(&maps.k, k, batch, heads, seq, k_strides[0], k_strides[1], k_strides[2], 128);
    if (rc == NS_OK) rc = make_map(&maps.v, v, batch, heads, seq, v_strides[0], v_strides[1], v_strides[2], 128);
    if (rc == NS_OK) rc = make_map(&maps.o, o, batch, heads, seq, o_strides[0], o_strides[1], o_strides[2], 32);
    if (rc != NS_OK) return rc;
    // the tile counter: one word at the start of the device object's scratch block, zeroed in stream order
    void* counter = nullptr;
    rc = ns_scratch_reserve(d, 256, &counter);
    if (rc != NS_OK) return rc;
    NS_CUDA(cudaMemsetAsync(counter, 0, sizeof(int), d->stream));
    FaParams p;
    p.tile_counter = reinterpret_cast<int*>(counter);
    p.batch = batch; p.heads = heads; p.seq = seq; p.causal = causal ? 1 : 0;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = d->status_dev;
    static bool configured[64] = {false};
    if (!configured[d->ordinal]) {
        NS_CUDA(cudaFuncSetAttribute(ns_attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_SMEM_BYTES));
        configured[d->ordinal] = true;
    }
    // persistent: one CTA per SM walks its share of the (batch, head, query tile) list
    const int total = batch * heads * n_qt;
    ns_attention_prefill_kernel<<<total < d->sm_count ? total : d->sm_count, FA_THREADS, FA_SMEM_BYTES, d->stream>>>(maps, p);
    NS_CUDA(cudaGetLastError());
    return NS_OK;
}
