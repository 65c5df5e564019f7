// Causal grouped-query attention of many query tokens over the paged cache on the
// fifth-generation tensor cores (prefill, head_dim 64 or 128, pages of 64 keys).
//
// A block takes 128 consecutive query tokens of one sequence and one query head and walks
// over the keys in tiles of 128 (two cache pages).  Inside a block
//   warp 0      one lane loads Q once and then K and V tiles by TMA into two stages of shared
//               memory (128-byte swizzle; a page of one kv head is a [64, 128] box);
//   warp 1      one lane issues tcgen05.mma: S = Q K^T into tensor memory, and, once the
//               softmax warps have turned S into probabilities P in tensor memory,
//               O += P V into a second accumulator (V is the MN-major operand: its rows are
//               keys).  S of the next tile is issued as soon as S of this one has been read,
//               so the tensor cores work on it while the softmax of this tile runs;
//   warps 2..9  two threads per query row (64 keys each): read the row of S from tensor
//               memory, mask it, keep the running maximum and sum in 32-bit, write
//               bfloat16 probabilities into tensor memory, where the second product reads them.  The
//               reference maximum of a row is only moved (and O rescaled in tensor memory)
//               when the true maximum has grown by more than 2^8 since; the result is the
//               same, as O and the sum always share one reference.  The probabilities are
//               2^(s * scale - m) by one multiply-add and the special-function unit, rounded
//               to bfloat16 by integer arithmetic (conversion instructions share the
//               special-function pipe), and are made before the wait for the last product with
//               V, so only their stores lie behind it.
// Measured on B200: with this a tile of 128 keys takes about 3300 cycles, of which the products are
// 1050; removing the exponentials, the maxima or the stores of P from the loop changes nothing, and
// the keys and values streamed from L2 (64 KB a tile, every block its own) come to 5.6 TB/s over all
// SMs: the kernel is bound by that stream, not by the softmax.  Two query tiles per block that share
// each tile of keys would halve it.
// A row at position p sees keys max(0, p - window + 1) .. p of its own sequence.  Whole pages
// are loaded, so rows of a page beyond a sequence's length are multiplied by probability zero:
// the cache must hold finite values everywhere (it is zero-filled when it is made).
// Every wait on a barrier is bounded (status word, as in gemm_tc).
//
// Reference counterpart: att_fused_f16 (internal/device/kernels.metal:657-813) called once per
// row (internal/device/metal.go:1403-1424).
#include "tcgen05.cuh"
#include <math_constants.h>

using namespace tc;

namespace {

constexpr int BM = 128;                 // query rows per block
constexpr int BN = 128;                 // keys per tile
constexpr int PAGE = 64;
constexpr int PANEL = 128 * 128;        // bytes of a [128 rows, 64 elements] panel
constexpr int PARTS = 2;                // softmax threads per query row: each has 128 / PARTS of a tile's keys and HD / PARTS output columns
constexpr int N_SOFTMAX = PARTS * BM;   // softmax threads
constexpr int N_THREADS = 64 + N_SOFTMAX;   // TMA warp, MMA warp, 4 softmax warps per part
constexpr float RESCALE_STEP = 8.0f;    // log2 units the maximum may run ahead of the reference

// HD: the head dimension, 64 or 128: one or two panels of 64 elements.
template <int HD>
struct Smem {
    alignas(1024) uint8_t q[HD / 64][PANEL];          // [d half][128 rows x 128 B]
    alignas(1024) uint8_t k[2][HD / 64][PANEL];       // [stage][d half][128 keys x 128 B]
    alignas(1024) uint8_t v[2][HD / 64][PANEL];       // [stage][d half][128 keys x 128 B]
    alignas(8) uint64_t q_full;
    uint64_t k_full[2], v_full[2], kv_empty[2];
    uint64_t s_full, s_empty, p_full, pv_done;
    uint32_t tmem_base;
    float row_max[2][PARTS][BM];                // [tile parity][part][row]: the parts' maxima of a row
    float row_sum[PARTS][BM];                   // [part][row]: the parts' sums at the end
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// x rounded to bfloat16 precision (nearest; the low 16 bits of the result are zero), x finite and at most 2^100 in
// size: Veltkamp's splitting with 2^16 + 1, three operations of the multiply-add pipe.  The conversion
// instructions share a pipe with the exponentials, and rounding by integer arithmetic took four operations of the
// integer pipe, which with the maxima and the packing made that pipe the busiest of the kernel (60 % against 41 %
// for the exponentials' and 40 % for the tensor cores').
__device__ __forceinline__ float bf16_round(float x) {
    const float p = __fmul_rn(x, 65537.0f);
    return __fadd_rn(__fsub_rn(x, p), p);
}
// 2^x by the special-function unit (relative error about 2^-22; -inf gives 0).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

#define LQ_WAIT(bar, parity, code) \
    if (!mbar_wait(smem_u32(&(bar)), (parity))) { give_up(code); ok = false; }

template <int HD>
__global__ void __launch_bounds__(N_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int* __restrict__ page_table, int pt_stride,
                       const int* __restrict__ slots, const int* __restrict__ kv_len, const int* __restrict__ qb_seq,
                       const int* __restrict__ qb_row, const int* __restrict__ qb_rows, const int* __restrict__ qb_pos,
                       __nv_bfloat16* __restrict__ out, int H, int Hkv, int oob_row, float scale_log2, int window) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int DH = HD / 64;                  // panels of 64 elements along the head dimension
    Smem<HD>& sm = *reinterpret_cast<Smem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 512;          // S in columns 0..127, O in 128..255, P (bfloat16 pairs) in 256..319

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sm.q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&sm.k_full[s]), 1);
            mbar_init(smem_u32(&sm.v_full[s]), 1);
            mbar_init(smem_u32(&sm.kv_empty[s]), 1);
        }
        mbar_init(smem_u32(&sm.s_full), 1);
        mbar_init(smem_u32(&sm.s_empty), N_SOFTMAX);
        mbar_init(smem_u32(&sm.p_full), N_SOFTMAX);
        mbar_init(smem_u32(&sm.pv_done), 1);
        mbar_fence_init();
        prefetch_map(&map_q);
        prefetch_map(&map_k);
        prefetch_map(&map_v);
    }
    if (warp == 1) tmem_alloc(smem_u32(&sm.tmem_base), TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_s = sm.tmem_base, tmem_o = sm.tmem_base + BN, tmem_p = sm.tmem_base + 2 * BN;
    pdl_wait();

    // Heads vary fastest: the work list has the blocks with the most keys first, so the launch order is
    // longest-first over all heads and the short blocks fill the tail.
    const int blk = blockIdx.x / H, h = blockIdx.x % H;
    const int seq = qb_seq[blk], row0 = qb_row[blk], n_rows = qb_rows[blk], pos0 = qb_pos[blk];
    const int kvh = h / (H / Hkv);
    const int len = kv_len[seq];
    const int* pt = page_table + (size_t)slots[seq] * pt_stride;
    const int pos_last = pos0 + n_rows - 1;
    const int key_first = (window > 0 && pos0 >= window) ? pos0 - window + 1 : 0;
    const int tile_lo = key_first / BN, n_tiles = pos_last / BN - tile_lo + 1;
    const int last_page = (len - 1) / PAGE;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            bool ok = true;
            mbar_expect_tx(smem_u32(&sm.q_full), DH * PANEL);
            for (int half = 0; half < DH; ++half)
                tma_load_2d(smem_u32(sm.q[half]), &map_q, h * HD + half * 64, row0, smem_u32(&sm.q_full));
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                LQ_WAIT(sm.kv_empty[s], ((j >> 1) & 1) ^ 1, 1);
                if (!ok) break;
                int rows[2];
                for (int i = 0; i < 2; ++i) {
                    const int pg = (tile_lo + j) * 2 + i;
                    const int page = pg <= last_page ? pt[pg] : -1;
                    rows[i] = page >= 0 ? (page * Hkv + kvh) * PAGE : oob_row;   // out of range: TMA fills zeros
                }
                mbar_expect_tx(smem_u32(&sm.k_full[s]), DH * PANEL);
                for (int half = 0; half < DH; ++half)
                    for (int i = 0; i < 2; ++i)
                        tma_load_2d(smem_u32(sm.k[s][half]) + i * (PANEL / 2), &map_k, half * 64, rows[i], smem_u32(&sm.k_full[s]));
                mbar_expect_tx(smem_u32(&sm.v_full[s]), DH * PANEL);
                for (int half = 0; half < DH; ++half)
                    for (int i = 0; i < 2; ++i)
                        tma_load_2d(smem_u32(sm.v[s][half]) + i * (PANEL / 2), &map_v, half * 64, rows[i], smem_u32(&sm.v_full[s]));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(BM, BN, false);
            constexpr uint32_t idesc_pv = idesc_bf16(BM, HD, true);
            bool ok = true;
            auto issue_s = [&](int s) {
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t a = desc_k_major(smem_u32(sm.q[kk >> 2]) + (kk & 3) * 32);
                    const uint64_t b = desc_k_major(smem_u32(sm.k[s][kk >> 2]) + (kk & 3) * 32);
                    mma_f16(tmem_s, a, b, idesc_s, kk > 0 ? 1u : 0u);
                }
                commit(smem_u32(&sm.s_full));
            };
            LQ_WAIT(sm.q_full, 0, 2);
            if (ok) LQ_WAIT(sm.k_full[0], 0, 3);
            if (ok) { fence_after(); issue_s(0); }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                if (j + 1 < n_tiles) {
                    LQ_WAIT(sm.k_full[s ^ 1], ((j + 1) >> 1) & 1, 3);
                    if (ok) LQ_WAIT(sm.s_empty, j & 1, 4);
                    if (!ok) break;
                    fence_after();
                    issue_s(s ^ 1);
                }
                LQ_WAIT(sm.p_full, j & 1, 5);
                if (ok) LQ_WAIT(sm.v_full[s], (j >> 1) & 1, 6);
                if (!ok) break;
                fence_after();
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t b = desc_mn_major(smem_u32(sm.v[s][0]) + kk * 2048, PANEL);
                    mma_f16_ts(tmem_o, tmem_p + kk * 8, b, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                commit(smem_u32(&sm.kv_empty[s]));
                commit(smem_u32(&sm.pv_done));
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- softmax: PARTS threads per query row,
        // each with 128 / PARTS of the tile's 128 keys (and HD / PARTS of the output columns).
        // A warp reads the 32 lanes of tensor memory that its number modulo 4 names.
        const int quarter = warp & 3, part = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pos_r = pos0 + r;
        const bool row_ok = r < n_rows;
        constexpr int NC = BN / PARTS;                    // keys of a tile of this thread
        constexpr int OC = HD / PARTS;                    // output columns of this thread
        static_assert(NC % 32 == 0 && OC % 32 == 0, "a thread reads whole chunks of 32 columns");
        float m_ref = -CUDART_INF_F, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            LQ_WAIT(sm.s_full, j & 1, 7);
            if (!ok) break;
            fence_after();
            float t[NC];
#pragma unroll
            for (int c = 0; c < NC / 32; ++c)
                ld32(tmem_s + lane_base + part * NC + c * 32, reinterpret_cast<uint32_t*>(t) + c * 32);
            wait_ld();
            fence_before();
            mbar_arrive(smem_u32(&sm.s_empty));          // S may be overwritten by the next tile's product
            const int kb = (tile_lo + j) * BN + part * NC;
            // Tiles that lie wholly inside every row's range (most of them) need no mask.
            const bool whole = n_rows == BM && (tile_lo + j) * BN + BN - 1 <= pos0 && (tile_lo + j) * BN + BN <= len &&
                               (window <= 0 || (tile_lo + j) * BN > pos_last - window);
            // Maxima of the raw scores (the scale is positive: it is applied to the maximum, and to the scores
            // inside the exponent's multiply-add).
            float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            if (whole) {
#pragma unroll
                for (int c = 0; c < NC; ++c) mx[c & 3] = fmaxf(mx[c & 3], t[c]);
            } else {
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int key = kb + c;
                    const bool vis = row_ok && key <= pos_r && key < len && (window <= 0 || key > pos_r - window);
                    t[c] = vis ? t[c] : -CUDART_INF_F;
                    mx[c & 3] = fmaxf(mx[c & 3], t[c]);
                }
            }
            // The row's maximum over all parts.
            const float m_mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
            sm.row_max[j & 1][part][r] = m_mine;
            asm volatile("bar.sync 1, %0;" ::"n"(N_SOFTMAX) : "memory");
            float m_tile = m_mine;
#pragma unroll
            for (int q = 1; q < PARTS; ++q) m_tile = fmaxf(m_tile, sm.row_max[j & 1][(part + q) % PARTS][r]);
            // Move the reference only when the maximum has run ahead of it by more than the step.
            const bool need = m_tile > m_ref + RESCALE_STEP;      // also true for the first visible key (m_ref = -inf)
            const float corr = need ? ex2(m_ref - m_tile) : 1.0f;     // m_ref = -inf gives 0
            if (need) { m_ref = m_tile; l *= corr; }
            if (j > 0 && __any_sync(0xffffffffu, need)) {
                LQ_WAIT(sm.pv_done, (j - 1) & 1, 8);              // O holds everything up to the last tile
                if (!ok) break;
                fence_after();
#pragma unroll 1
                for (int c = 0; c < OC / 32; ++c) {               // this thread's part of the row of O
                    uint32_t o[32];
                    ld32(tmem_o + lane_base + part * OC + c * 32, o);
                    wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    st32(tmem_o + lane_base + part * OC + c * 32, o);
                }
                wait_st();
            }
            const float base = m_ref == -CUDART_INF_F ? 0.f : m_ref;
            // The probabilities, rounded to bfloat16 and packed in pairs, while the last tile's product with V
            // still runs.  The sum runs over them as the product will see them.
            // Rounded on the multiply-add pipe (bf16_round): conversion instructions would share a pipe with the exponentials.
            float sums[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[NC / 2];
#pragma unroll
            for (int c = 0; c < NC / 2; ++c) {
                const float b0 = bf16_round(ex2(fmaf(t[2 * c], scale_log2, -base)));
                const float b1 = bf16_round(ex2(fmaf(t[2 * c + 1], scale_log2, -base)));
                sums[c & 3] += b0 + b1;
                pk[c] = __byte_perm(__float_as_uint(b0), __float_as_uint(b1), 0x7632);      // low half: b0's upper 16 bits, high half: b1's
            }
            if (j > 0) {
                LQ_WAIT(sm.pv_done, (j - 1) & 1, 8);              // the last product has read P
                if (!ok) break;
            }
            // Row r of P goes to lane r of tensor memory, two probabilities per column: keys 2c and 2c + 1 of this
            // thread's part in column part * NC / 2 + c.
#pragma unroll
            for (int c = 0; c < NC / 64; ++c) st32(tmem_p + lane_base + part * (NC / 2) + c * 32, pk + c * 32);
            wait_st();
            l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
            fence_before();
            mbar_arrive(smem_u32(&sm.p_full));
        }
        if (ok) {
            LQ_WAIT(sm.pv_done, (n_tiles - 1) & 1, 9);
        }
        if (ok) {
            fence_after();
            sm.row_sum[part][r] = l;
            asm volatile("bar.sync 1, %0;" ::"n"(N_SOFTMAX) : "memory");
            float total = 0.f;
#pragma unroll
            for (int q = 0; q < PARTS; ++q) total += sm.row_sum[q][r];
            const float inv = 1.0f / total;
            __nv_bfloat16* orow = out + ((size_t)(row0 + r) * H + h) * HD + part * OC;
#pragma unroll 1
            for (int c = 0; c < OC / 32; ++c) {
                uint32_t o[32];
                ld32(tmem_o + lane_base + part * OC + c * 32, o);
                wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        reinterpret_cast<uint4*>(orow + c * 32)[i] =
                            make_uint4(pack2(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv),
                                       pack2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv),
                                       pack2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv),
                                       pack2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv));
                }
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_dealloc(sm.tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ two heads of a group per block
// The same attention with two chains of work per block: the 128 query rows of two heads that share a kv head
// (so each tile of keys and values is loaded once for both), each chain with an S and an O of its own in
// tensor memory and four softmax warps (one thread per row: no exchange of maxima).  While the softmax of
// one chain runs, the tensor cores make the other chain's products, so the chain of hand-overs of a tile
// (scores ready, read, maxima, exponentials, probabilities stored, product issued) of one head hides behind
// the other's.  P takes the place of S in tensor memory (the next S of a chain is issued after its P V, and
// products run in the order of issue).  Twelve warps: 0 loads, 1 issues products, 2 and 3 idle, 4..7 and
// 8..11 the two chains' softmax; the first four give registers up (setmaxnreg) so that a softmax thread can
// hold its row's 128 scores.
constexpr int N_THREADS2 = 384;

template <int HD>
struct Smem2 {
    alignas(1024) uint8_t q[2][HD / 64][PANEL];       // [chain][d half][128 rows x 128 B]
    alignas(1024) uint8_t k[2][HD / 64][PANEL];       // [stage][d half][128 keys x 128 B]
    alignas(1024) uint8_t v[2][HD / 64][PANEL];
    alignas(8) uint64_t q_full;
    uint64_t k_full[2], v_full[2], kv_empty[2];
    uint64_t s_full[2], p_full[2], pv_done[2];        // per chain
    uint32_t tmem_base;
};

template <int HD>
__global__ void __launch_bounds__(N_THREADS2, 1)
attn_prefill_two_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const int* __restrict__ page_table, int pt_stride,
                        const int* __restrict__ slots, const int* __restrict__ kv_len, const int* __restrict__ qb_seq,
                        const int* __restrict__ qb_row, const int* __restrict__ qb_rows, const int* __restrict__ qb_pos,
                        __nv_bfloat16* __restrict__ out, int H, int Hkv, int oob_row, float scale_log2, int window) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int DH = HD / 64;
    Smem2<HD>& sm = *reinterpret_cast<Smem2<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 512;          // S (then P) of the chains in columns 0..127 and 128..255, O from 256 on

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sm.q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&sm.k_full[s]), 1);
            mbar_init(smem_u32(&sm.v_full[s]), 1);
            mbar_init(smem_u32(&sm.kv_empty[s]), 1);
            mbar_init(smem_u32(&sm.s_full[s]), 1);
            mbar_init(smem_u32(&sm.p_full[s]), BM);
            mbar_init(smem_u32(&sm.pv_done[s]), 1);
        }
        mbar_fence_init();
        prefetch_map(&map_q);
        prefetch_map(&map_k);
        prefetch_map(&map_v);
    }
    if (warp == 1) tmem_alloc(smem_u32(&sm.tmem_base), TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = sm.tmem_base;
    pdl_wait();

    // Pairs of heads vary fastest: the blocks with the most keys come first over all heads.
    const int pairs = H >> 1;
    const int blk = blockIdx.x / pairs, h0 = (blockIdx.x % pairs) * 2;
    const int seq = qb_seq[blk], row0 = qb_row[blk], n_rows = qb_rows[blk], pos0 = qb_pos[blk];
    const int kvh = h0 / (H / Hkv);
    const int len = kv_len[seq];
    const int* pt = page_table + (size_t)slots[seq] * pt_stride;
    const int pos_last = pos0 + n_rows - 1;
    const int key_first = (window > 0 && pos0 >= window) ? pos0 - window + 1 : 0;
    const int tile_lo = key_first / BN, n_tiles = pos_last / BN - tile_lo + 1;
    const int last_page = (len - 1) / PAGE;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ TMA producer
            bool ok = true;
            mbar_expect_tx(smem_u32(&sm.q_full), 2 * DH * PANEL);
            for (int c = 0; c < 2; ++c)
                for (int half = 0; half < DH; ++half)
                    tma_load_2d(smem_u32(sm.q[c][half]), &map_q, (h0 + c) * HD + half * 64, row0, smem_u32(&sm.q_full));
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                LQ_WAIT(sm.kv_empty[s], ((j >> 1) & 1) ^ 1, 1);
                if (!ok) break;
                int rows[2];
                for (int i = 0; i < 2; ++i) {
                    const int pg = (tile_lo + j) * 2 + i;
                    const int page = pg <= last_page ? pt[pg] : -1;
                    rows[i] = page >= 0 ? (page * Hkv + kvh) * PAGE : oob_row;   // out of range: TMA fills zeros
                }
                mbar_expect_tx(smem_u32(&sm.k_full[s]), DH * PANEL);
                for (int half = 0; half < DH; ++half)
                    for (int i = 0; i < 2; ++i)
                        tma_load_2d(smem_u32(sm.k[s][half]) + i * (PANEL / 2), &map_k, half * 64, rows[i], smem_u32(&sm.k_full[s]));
                mbar_expect_tx(smem_u32(&sm.v_full[s]), DH * PANEL);
                for (int half = 0; half < DH; ++half)
                    for (int i = 0; i < 2; ++i)
                        tma_load_2d(smem_u32(sm.v[s][half]) + i * (PANEL / 2), &map_v, half * 64, rows[i], smem_u32(&sm.v_full[s]));
            }
        } else if (warp == 1 && lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            constexpr uint32_t idesc_s = idesc_bf16(BM, BN, false);
            constexpr uint32_t idesc_pv = idesc_bf16(BM, HD, true);
            bool ok = true;
            auto issue_s = [&](int c, int s) {          // S of chain c from the keys in stage s
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t a = desc_k_major(smem_u32(sm.q[c][kk >> 2]) + (kk & 3) * 32);
                    const uint64_t b = desc_k_major(smem_u32(sm.k[s][kk >> 2]) + (kk & 3) * 32);
                    mma_f16(tmem_base + c * BN, a, b, idesc_s, kk > 0 ? 1u : 0u);
                }
                commit(smem_u32(&sm.s_full[c]));
            };
            LQ_WAIT(sm.q_full, 0, 2);
            if (ok) LQ_WAIT(sm.k_full[0], 0, 3);
            if (ok) { fence_after(); issue_s(0, 0); issue_s(1, 0); }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                for (int c = 0; c < 2 && ok; ++c) {
                    LQ_WAIT(sm.p_full[c], j & 1, 5);
                    if (ok && c == 0) LQ_WAIT(sm.v_full[s], (j >> 1) & 1, 6);
                    if (!ok) break;
                    fence_after();
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk) {
                        const uint64_t b = desc_mn_major(smem_u32(sm.v[s][0]) + kk * 2048, PANEL);
                        mma_f16_ts(tmem_base + 2 * BN + c * HD, tmem_base + c * BN + kk * 8, b, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    if (c == 1) commit(smem_u32(&sm.kv_empty[s]));      // every product that reads this stage has been issued
                    commit(smem_u32(&sm.pv_done[c]));
                    if (j + 1 < n_tiles) {
                        // The chain's next S takes the place of its P: issued after P V, it runs after it.
                        if (c == 0) LQ_WAIT(sm.k_full[s ^ 1], ((j + 1) >> 1) & 1, 3);
                        if (!ok) break;
                        fence_after();
                        issue_s(c, s ^ 1);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- softmax: one thread per query row and chain
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int chain = (warp - 4) >> 2, quarter = warp & 3;
        const int h = h0 + chain;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t tmem_s = tmem_base + chain * BN + lane_base;              // S, then P in its first 64 columns
        const uint32_t tmem_o = tmem_base + 2 * BN + chain * HD + lane_base;
        const int pos_r = pos0 + r;
        const bool row_ok = r < n_rows;
        float m_ref = -CUDART_INF_F, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            LQ_WAIT(sm.s_full[chain], j & 1, 7);         // S of this tile is there, and so is the last tile's P V (issued before it)
            if (!ok) break;
            fence_after();
            float t[BN];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) ld32(tmem_s + c * 32, reinterpret_cast<uint32_t*>(t) + c * 32);
            wait_ld();
            const int kb = (tile_lo + j) * BN;
            const bool whole = n_rows == BM && kb + BN - 1 <= pos0 && kb + BN <= len && (window <= 0 || kb > pos_last - window);
            float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            if (whole) {
#pragma unroll
                for (int c = 0; c < BN; ++c) mx[c & 3] = fmaxf(mx[c & 3], t[c]);
            } else {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int key = kb + c;
                    const bool vis = row_ok && key <= pos_r && key < len && (window <= 0 || key > pos_r - window);
                    t[c] = vis ? t[c] : -CUDART_INF_F;
                    mx[c & 3] = fmaxf(mx[c & 3], t[c]);
                }
            }
            const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
            // Move the reference only when the maximum has run ahead of it by more than the step.
            const bool need = m_tile > m_ref + RESCALE_STEP;
            const float corr = need ? ex2(m_ref - m_tile) : 1.0f;
            if (need) { m_ref = m_tile; l *= corr; }
            if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t o[32];
                    ld32(tmem_o + c * 32, o);
                    wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    st32(tmem_o + c * 32, o);
                }
            }
            const float base = m_ref == -CUDART_INF_F ? 0.f : m_ref;
            float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t pk[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float b0 = bf16_round(ex2(fmaf(t[half * 64 + 2 * c], scale_log2, -base)));
                    const float b1 = bf16_round(ex2(fmaf(t[half * 64 + 2 * c + 1], scale_log2, -base)));
                    sums[c & 3] += b0 + b1;
                    pk[c] = __byte_perm(__float_as_uint(b0), __float_as_uint(b1), 0x7632);
                }
                st32(tmem_s + half * 32, pk);           // keys 64 half + 2c, + 1 in column 32 half + c
            }
            wait_st();
            l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
            fence_before();
            mbar_arrive(smem_u32(&sm.p_full[chain]));
        }
        if (ok) {
            LQ_WAIT(sm.pv_done[chain], (n_tiles - 1) & 1, 9);
        }
        if (ok) {
            fence_after();
            const float inv = 1.0f / l;
            __nv_bfloat16* orow = out + ((size_t)(row0 + r) * H + h) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                ld32(tmem_o + c * 32, o);
                wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        reinterpret_cast<uint4*>(orow + c * 32)[i] =
                            make_uint4(pack2(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv),
                                       pack2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv),
                                       pack2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv),
                                       pack2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv));
                }
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace

namespace {
template <int HD>
int launch_hd(const void* q, int q_stride, int T, const void* k_pages, const void* v_pages, int n_pages,
              const int* page_table, int pt_stride, const int* slots, const int* kv_len, const int* qb_seq,
              const int* qb_row, const int* qb_rows, const int* qb_pos, void* out, int n_blocks, int H, int Hkv,
              float scale, int window, cudaStream_t stream) {
    CUtensorMap mq, mk, mv;
    const long kv_rows = (long)n_pages * Hkv * PAGE;
    int rc = make_map_bf16(&mq, q, T, q_stride, q_stride, BM);
    if (rc == LQ_OK) rc = make_map_bf16(&mk, k_pages, kv_rows, HD, HD, PAGE);
    if (rc == LQ_OK) rc = make_map_bf16(&mv, v_pages, kv_rows, HD, HD, PAGE);
    if (rc != LQ_OK) return rc;
    constexpr size_t smem = sizeof(Smem<HD>) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        configured = true;
    }
    static const bool one_chain = [] { const char* v = getenv("LQ_ATTN_ONE_CHAIN"); return v && v[0] == '1'; }();
    if ((H / Hkv) % 2 == 0 && !one_chain) {
        // Two heads of a group per block: they share the block's tiles of keys and values.
        constexpr size_t smem2 = sizeof(Smem2<HD>) + 1024;
        static_assert(smem2 <= 232448, "more shared memory than a block may have");
        static bool configured2 = false;
        if (!configured2) {
            if (cudaFuncSetAttribute(attn_prefill_two_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2) != cudaSuccess)
                return lq_launch_status();
            configured2 = true;
        }
        return launch_pdl(attn_prefill_two_kernel<HD>, dim3(n_blocks * (H / 2)), dim3(N_THREADS2), smem2, stream, mq, mk, mv,
                          page_table, pt_stride, slots, kv_len, qb_seq, qb_row, qb_rows, qb_pos, (__nv_bfloat16*)out, H, Hkv,
                          (int)kv_rows, scale * 1.4426950408889634f, window);
    }
    return launch_pdl(attn_prefill_tc_kernel<HD>, dim3(n_blocks * H), dim3(N_THREADS), smem, stream, mq, mk, mv, page_table,
                      pt_stride, slots, kv_len, qb_seq, qb_row, qb_rows, qb_pos, (__nv_bfloat16*)out, H, Hkv,
                      (int)kv_rows, scale * 1.4426950408889634f, window);
}
}  // namespace

// q: [T, q_stride] bfloat16 rows whose first H*hd elements hold the query heads; out [T, H*hd].  hd is 64 or 128.
// k_pages, v_pages: [n_pages, Hkv, 64, hd] bfloat16 of one cache entry, finite everywhere.
// qb_*: the work list, n_blocks entries: sequence, first packed row, rows (<= 128), position of the first row.
LQ_EXPORT int lq_attn_prefill_tc(const void* q, int q_stride, int T, const void* k_pages, const void* v_pages,
                                 int n_pages, const int* page_table, int pt_stride, const int* slots, const int* kv_len,
                                 const int* qb_seq, const int* qb_row, const int* qb_rows, const int* qb_pos, void* out,
                                 int n_blocks, int H, int Hkv, int hd, int page_size, float scale, int window,
                                 cudaStream_t stream) {
    if (n_blocks <= 0) return LQ_OK;
    if ((hd != 64 && hd != 128) || page_size != PAGE || H % Hkv || q_stride % 8 || ((uintptr_t)q & 15)) return LQ_BAD_SIZE;
    if (hd == 64)
        return launch_hd<64>(q, q_stride, T, k_pages, v_pages, n_pages, page_table, pt_stride, slots, kv_len, qb_seq, qb_row,
                             qb_rows, qb_pos, out, n_blocks, H, Hkv, scale, window, stream);
    return launch_hd<128>(q, q_stride, T, k_pages, v_pages, n_pages, page_table, pt_stride, slots, kv_len, qb_seq, qb_row,
                          qb_rows, qb_pos, out, n_blocks, H, Hkv, scale, window, stream);
}

LQ_EXPORT int lq_attn_prefill_tc_status() { return tc::status_read(); }

// The same word in host memory that the device writes through (readable without a CUDA call); null when
// it could not be set up.
LQ_EXPORT int* lq_attn_prefill_tc_status_word() { return tc::status_word(); }
