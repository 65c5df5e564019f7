// Attention of single query tokens over the paged cache, split along the keys
// (decoding: one new token for each sequence of the batch).
//
// The step is bound by reading K and V once from HBM.  A block serves one token, one
// kv head and one slice of that sequence's keys; the query heads that share the kv
// head are the rows of the m16n8k16 tile (grouped-query attention reads each key once
// for the whole group).  The 8 warps take 16-key tiles in turn; each warp keeps a ring of
// three tiles in shared memory, filled by cp.async two tiles ahead of the one it works on,
// so that a block has about 128 KB of keys and values on their way at any time (with the
// loads held in registers instead, one tile ahead was all that fitted, and the stream
// stalled on memory latency at 3.7 TB/s).  Fragments come from the ring by ldmatrix.
// Softmax runs online in 32-bit; the warps of a block and then the slices of a
// sequence are merged by their running maximum and sum, in a fixed order.
//
// Slices write unnormalised partial outputs [token, head, slice, head_dim] with
// (max, sum) to scratch memory; the block that parks its slice last for a (token, kv head)
// merges them (a counter per pair; without counters a second kernel merges).
//
// With a work list (lq_attn_decode_work) the blocks form teams of one block per (kv head, row tile);
// a team walks a list of segments (token, range of key tiles) that the host has cut so that every
// team reads the same number of tiles, however unequal the sequences are: a long sequence is
// shared by several teams, short ones share a team, and all blocks run as one wave.
//
// Reference counterpart: att_fused_f16 (internal/device/kernels.metal:657-813), one
// threadgroup per query head, scores in threadgroup memory.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int DW = 8;            // warps per block
constexpr int TILE = 16;         // keys per warp tile
constexpr int RING = 3;          // tiles of a warp in shared memory: one in use, two on their way
constexpr int PAD = 8;           // elements of padding per shared-memory row (ldmatrix without bank conflicts)
constexpr int MAX_SPLITS = 32;   // most slices a sequence's keys are cut into

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    int bytes = valid ? 16 : 0;     // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// HD: head_dim rounded up to 32, 64 or 128; the real head_dim hd is a multiple of 8.
// Two blocks share an SM where their rings allow it (head_dim up to 64), so the registers are held to half the file.
template <int HD>
__global__ void __launch_bounds__(DW * 32, HD <= 64 ? 2 : 1)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_pages,
                   const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ page_table, int pt_stride,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                   __nv_bfloat16* __restrict__ out, int H, int Hkv, int hd, int page_size, float scale, int window,
                   int n_splits, int part_stride, const int* __restrict__ work, const char* next_w, unsigned next_piece,
                   int early_loads) {
    constexpr int LD = HD + PAD;                   // shared-memory row length in elements
    constexpr int KD = HD / 16;                    // k16 steps over the head dimension
    constexpr int STAGE = 2 * TILE * LD;           // elements of one tile: K rows, then V rows
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [DW][RING][STAGE]
    // After the loop the same memory holds each warp's state for the merge.
    float (*sm_o)[16][HD + 1] = reinterpret_cast<float (*)[16][HD + 1]>(smem_raw);
    float (*sm_m)[16] = reinterpret_cast<float (*)[16]>(smem_raw + sizeof(float) * DW * 16 * (HD + 1));
    float (*sm_l)[16] = sm_m + DW;
    __shared__ float sm_w[16][MAX_SPLITS];       // weights of the slices when this block merges them
    __shared__ float sm_inv[16];
    __shared__ int sm_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = H / Hkv, gtiles = (G + 15) / 16;
    // Without a work list: grid (slices, kv heads x row tiles, tokens), one segment per block.
    // With one: grid (kv heads x row tiles, teams); the list starts with teams + 1 offsets into its
    // segments, five integers each: token, first and last + 1 key tile (counted from the first
    // tile the token sees), which part of the token this is, and how many parts the token has.
    const int head_tile = work ? blockIdx.x : blockIdx.y;
    const int kvh = head_tile / gtiles, gt = head_tile % gtiles;
    int seg = 0, seg_end = 1;
    const int* segments = nullptr;
    if (work) {
        seg = work[blockIdx.y];
        seg_end = work[blockIdx.y + 1];
        segments = work + gridDim.y + 1;
    }
    const size_t head_off = (size_t)kvh * page_size * hd;
    __nv_bfloat16* my_ring = ring + (size_t)warp * RING * STAGE;
    // No pdl_launch_dependents() here: released early, the blocks of the product that follows moved
    // onto the SMs this kernel leaves free and fetched weights against it (measured: the step ran
    // 50 % slower).  Released late instead (once a block's keys and values have all arrived) it still lost 40 %:
    // the product after this one releases its own successor at its start, and that one (the gate and up
    // product, six waves of blocks) then takes the places that the product before it still needs.
    // The kernel after this one starts when this one ends.
    bool waited = false;
    for (; seg < seg_end; ++seg) {
    if (waited) __syncthreads();        // the merge of the segment before has read the shared memory that the ring refills
    int tok, split, parts, seg_lo, seg_hi;
    if (work) {
        const int* s = segments + 5 * seg;
        tok = s[0]; seg_lo = s[1]; seg_hi = s[2]; split = s[3]; parts = s[4];
    } else {
        tok = blockIdx.z; split = blockIdx.x; parts = n_splits; seg_lo = seg_hi = 0;
    }
    // Positions, slots and page table are written before the step starts, never by a kernel of the
    // step, so they may be read before the kernel ahead is known to have finished.
    const int pos = tok_pos[tok], len = pos + 1;
    const int start = (window > 0 && pos >= window) ? pos - window + 1 : 0;
    const int* pt = page_table + (size_t)slots[tok_seq[tok]] * pt_stride;

    const int first_tile = start / TILE;
    const int n_tiles = (len + TILE - 1) / TILE - first_tile;
    int tile_lo, tile_hi;
    if (work) {
        tile_lo = first_tile + seg_lo;
        tile_hi = min(first_tile + n_tiles, first_tile + seg_hi);
    } else {
        const int per_split = (n_tiles + parts - 1) / parts;
        tile_lo = first_tile + split * per_split;
        tile_hi = min(first_tile + n_tiles, tile_lo + per_split);
    }

    // This warp's tiles are tile_lo + warp, + DW, ...; `n` counts them.
    auto issue = [&](int n) {
        const int tile = tile_lo + warp + n * DW;
        if (tile < tile_hi) {
            const int kb = tile * TILE;
            const int page = pt[kb / page_size];
            const size_t off = (size_t)page * Hkv * page_size * hd + head_off + (size_t)(kb % page_size) * hd;
            __nv_bfloat16* ks = my_ring + (size_t)(n % RING) * STAGE;
            __nv_bfloat16* vs = ks + TILE * LD;
            for (int i = lane; i < TILE * (HD / 8); i += 32) {
                const int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
                const bool ok = kb + r < len && c < hd;
                const size_t src = off + (size_t)(ok ? r : 0) * hd + (ok ? c : 0);
                cp_async16((uint32_t)__cvta_generic_to_shared(ks + r * LD + c), k_pages + src, ok);
                cp_async16((uint32_t)__cvta_generic_to_shared(vs + r * LD + c), v_pages + src, ok);
            }
        }
        cp_async_commit();          // an empty group when there is no tile: the count of groups stays in step
    };
    // The keys and values of earlier positions were stored by earlier steps: a warp whose first tiles
    // do not hold the token's own position (which the kernel ahead is writing) asks for them at once.
    const int own_tile = pos / TILE;
    bool early = waited || early_loads != 0;       // after the wait nothing of the step is still being written
    if (!waited) {
#pragma unroll
        for (int n = 0; n < RING - 1; ++n) early = early && (tile_lo + warp + n * DW != own_tile);
    }
    if (early) {
#pragma unroll
        for (int n = 0; n < RING - 1; ++n) issue(n);
    }
    if (!waited) pdl_wait();
    waited = true;
    if (!early) {
#pragma unroll
        for (int n = 0; n < RING - 1; ++n) issue(n);
    }
    // Query heads of the group as the rows of the mma tile (rows g and g + 8 of this thread).
    const int r0 = gt * 16 + g, r1 = r0 + 8;
    const bool r0ok = r0 < G, r1ok = r1 < G;
    const __nv_bfloat16* q0p = q + (size_t)tok * q_stride + (size_t)(kvh * G + (r0ok ? r0 : 0)) * hd;
    const __nv_bfloat16* q1p = q + (size_t)tok * q_stride + (size_t)(kvh * G + (r1ok ? r1 : 0)) * hd;
    uint32_t qf[KD][4];
#pragma unroll
    for (int kk = 0; kk < KD; ++kk) {
        const int d0 = kk * 16 + 2 * t, d1 = d0 + 8;
        qf[kk][0] = (r0ok && d0 < hd) ? *reinterpret_cast<const uint32_t*>(q0p + d0) : 0u;
        qf[kk][1] = (r1ok && d0 < hd) ? *reinterpret_cast<const uint32_t*>(q1p + d0) : 0u;
        qf[kk][2] = (r0ok && d1 < hd) ? *reinterpret_cast<const uint32_t*>(q0p + d1) : 0u;
        qf[kk][3] = (r1ok && d1 < hd) ? *reinterpret_cast<const uint32_t*>(q1p + d1) : 0u;
    }

    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;


    const int my_tiles = tile_lo + warp < tile_hi ? (tile_hi - tile_lo - warp + DW - 1) / DW : 0;
    for (int n = 0; n < my_tiles; ++n) {
        issue(n + RING - 1);
        cp_async_wait<RING - 1>();
        __syncwarp();
        const int kb = (tile_lo + warp + n * DW) * TILE;
        const __nv_bfloat16* ks = my_ring + (size_t)(n % RING) * STAGE;
        const __nv_bfloat16* vs = ks + TILE * LD;
        // S = Q K^T for the tile's two groups of 8 keys.
        float s[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KD; ++kk) {
            // matrices (keys 0-7, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 0-7), (keys 8-15, d 8-15)
            const int r = (lane & 7) + (lane >> 4) * 8, c = kk * 16 + ((lane >> 3) & 1) * 8;
            uint32_t b0, b1, b2, b3;
            ldsm_x4((uint32_t)__cvta_generic_to_shared(ks + r * LD + c), b0, b1, b2, b3);
            mma_bf16(s[0], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
            mma_bf16(s[1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
        }
        float tm0 = -CUDART_INF_F, tm1 = -CUDART_INF_F;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                int key = kb + nt * 8 + 2 * t + i;
                bool ok = key >= start && key < len;
                s[nt][i] = ok ? s[nt][i] * scale : -CUDART_INF_F;
                s[nt][2 + i] = ok ? s[nt][2 + i] * scale : -CUDART_INF_F;
                tm0 = fmaxf(tm0, s[nt][i]);
                tm1 = fmaxf(tm1, s[nt][2 + i]);
            }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        const float nm0 = fmaxf(m0, tm0), nm1 = fmaxf(m1, tm1);
        // A tile of this warp always holds at least one visible key (kb <= pos, kb + 15 >= start),
        // so nm0 and nm1 are finite.
        const float c0 = expf(m0 - nm0), c1 = expf(m1 - nm1);
        m0 = nm0;
        m1 = nm1;
        uint32_t pa[4];
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            // The sum runs over the probabilities as the product will see them (rounded to
            // bfloat16), so that the weights of a row add up to one exactly.
            float p00 = round_bf16(expf(s[nt][0] - nm0)), p01 = round_bf16(expf(s[nt][1] - nm0));
            float p10 = round_bf16(expf(s[nt][2] - nm1)), p11 = round_bf16(expf(s[nt][3] - nm1));
            ps0 += p00 + p01;
            ps1 += p10 + p11;
            pa[nt * 2 + 0] = pack_bf16(p00, p01);
            pa[nt * 2 + 1] = pack_bf16(p10, p11);
        }
        l0 = l0 * c0 + ps0;
        l1 = l1 * c1 + ps1;
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            // V transposed on load: matrices (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
            const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 16 + (lane >> 4) * 8;
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t((uint32_t)__cvta_generic_to_shared(vs + r * LD + c), b0, b1, b2, b3);
            float (&oa)[4] = o[2 * dp];
            float (&ob)[4] = o[2 * dp + 1];
            oa[0] *= c0; oa[1] *= c0; oa[2] *= c1; oa[3] *= c1;
            ob[0] *= c0; ob[1] *= c0; ob[2] *= c1; ob[3] *= c1;
            mma_bf16(oa, pa[0], pa[1], pa[2], pa[3], b0, b1);
            mma_bf16(ob, pa[0], pa[1], pa[2], pa[3], b2, b3);
        }
        __syncwarp();       // every lane is done with the slot before a later copy refills it
    }
    cp_async_wait<0>();
    if (next_w && threadIdx.x == 0 && seg == seg_end - 1) {
        // The weights that the stream reads after this kernel: each block asks for one piece of their
        // first bytes to be brought into L2 now that its own keys and values have arrived.
        const size_t b = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(next_w + b * next_piece), "r"(next_piece) : "memory");
    }
    // Row sums: add the four threads of a row.
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();        // all rings are idle: their memory now holds the warps' states
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
        const int d = j * 8 + 2 * t;
        sm_o[warp][g][d] = o[j][0];
        sm_o[warp][g][d + 1] = o[j][1];
        sm_o[warp][g + 8][d] = o[j][2];
        sm_o[warp][g + 8][d + 1] = o[j][3];
    }
    if (t == 0) {
        sm_m[warp][g] = m0; sm_m[warp][g + 8] = m1;
        sm_l[warp][g] = l0; sm_l[warp][g + 8] = l1;
    }
    __syncthreads();
    const int rows = min(16, G - gt * 16);
    for (int i = threadIdx.x; i < rows * hd; i += DW * 32) {
        int r = i / hd, d = i % hd;
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < DW; ++w) mx = fmaxf(mx, sm_m[w][r]);
        float acc = 0.f, l = 0.f;
        if (mx > -CUDART_INF_F) {
#pragma unroll
            for (int w = 0; w < DW; ++w) {
                float f = expf(sm_m[w][r] - mx);   // a warp without tiles has m = -inf: f = 0
                acc += sm_o[w][r][d] * f;
                l += sm_l[w][r] * f;
            }
        }
        int h = kvh * G + gt * 16 + r;
        if (parts == 1) {
            out[((size_t)tok * H + h) * hd + d] = __float2bfloat16_rn(acc / l);
        } else {
            size_t base = ((size_t)tok * H + h) * part_stride + split;
            part_o[base * hd + d] = acc;
            if (d == 0) { part_ml[base * 2] = mx; part_ml[base * 2 + 1] = l; }
        }
    }
    if (parts == 1 || counters == nullptr) continue;
    // The block that parks its slice last merges all slices of its (token, kv head, row tile):
    // out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M), slices in their order.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = counters + (size_t)tok * Hkv * gtiles + head_tile;
        int old = atomicAdd(counter, 1);
        sm_last = (old == parts - 1);
        if (sm_last) *counter = 0;                  // ready for the next call
    }
    __syncthreads();
    if (!sm_last) continue;
    __threadfence();
    // Weights of the slices, one warp per row and one lane per slice (at most 32 slices).
    for (int r = warp; r < rows; r += DW) {
        const float* ml = part_ml + ((size_t)tok * H + kvh * G + gt * 16 + r) * part_stride * 2;
        const float m = lane < parts ? __ldcg(ml + 2 * lane) : -CUDART_INF_F;
        const float ls = lane < parts ? __ldcg(ml + 2 * lane + 1) : 0.f;
        const float mx = warp_max(m);
        const float w = m > -CUDART_INF_F ? expf(m - mx) : 0.f;
        const float l = warp_sum(ls * w);        // the same order of additions whichever block merges
        if (lane < parts) sm_w[r][lane] = w;
        if (lane == 0) sm_inv[r] = 1.0f / l;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows * hd; i += DW * 32) {
        const int r = i / hd, d = i % hd;
        const int h = kvh * G + gt * 16 + r;
        const float* po = part_o + ((size_t)tok * H + h) * part_stride * hd + d;
        float acc = 0.f;
#pragma unroll 8
        for (int s2 = 0; s2 < parts; ++s2) acc += __ldcg(po + (size_t)s2 * hd) * sm_w[r][s2];
        out[((size_t)tok * H + h) * hd + d] = __float2bfloat16_rn(acc * sm_inv[r]);
    }
    }   // segments
}

// Merge the slices of one (token, head): out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M).
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  __nv_bfloat16* __restrict__ out, int hd, int n_splits) {
    __shared__ float w[MAX_SPLITS];
    __shared__ float inv;
    const size_t th = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const float* ml = part_ml + th * n_splits * 2;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float m = lane < n_splits ? ml[2 * lane] : -CUDART_INF_F;
        const float ls = lane < n_splits ? ml[2 * lane + 1] : 0.f;
        const float mx = warp_max(m);
        const float f = m > -CUDART_INF_F ? expf(m - mx) : 0.f;
        const float l = warp_sum(ls * f);
        if (lane < n_splits) w[lane] = f;
        if (lane == 0) inv = 1.0f / l;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < n_splits; ++s) acc += part_o[(th * n_splits + s) * hd + d] * w[s];
        out[th * hd + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int HD>
int launch(const void* q, int q_stride, const void* k_pages, const void* v_pages, const int* page_table, int pt_stride,
           const int* tok_pos, const int* tok_seq, const int* slots, float* part_o, float* part_ml, int* counters,
           void* out, int T, int H, int Hkv, int hd, int page_size, float scale, int window, int n_splits,
           const int* work, int teams, const void* next_w, long next_bytes, int early_loads, cudaStream_t stream) {
    int G = H / Hkv, gtiles = (G + 15) / 16;
    dim3 grid(n_splits, Hkv * gtiles, T);
    if (work) grid = dim3(Hkv * gtiles, teams, 1);      // n_splits is then the room for parts per token in the scratch
    const long n_blocks = (long)grid.x * grid.y * grid.z;
    long piece = (next_w && !((uintptr_t)next_w & 15)) ? next_bytes / n_blocks / 16 * 16 : 0;
    if (piece > (1 << 20)) piece = 1 << 20;
    if (piece <= 0) next_w = nullptr;
    constexpr size_t ring = (size_t)DW * RING * 2 * TILE * (HD + PAD) * 2;
    constexpr size_t merge = sizeof(float) * DW * 16 * (HD + 1) + sizeof(float) * 2 * DW * 16;
    constexpr size_t smem = ring > merge ? ring : merge;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        configured = true;
    }
    int rc = launch_pdl(attn_decode_kernel<HD>, grid, dim3(DW * 32), smem, stream, (const __nv_bfloat16*)q, q_stride,
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table, pt_stride, tok_pos, tok_seq, slots,
        part_o, part_ml, counters, (__nv_bfloat16*)out, H, Hkv, hd, page_size, scale, window, n_splits, n_splits, work,
        (const char*)next_w, (unsigned)piece, early_loads);
    if (rc != LQ_OK || n_splits == 1 || counters != nullptr) return rc;
    return launch_pdl(attn_merge_kernel, dim3(T * H), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml,
                      (__nv_bfloat16*)out, hd, n_splits);
}

}  // namespace

// q: rows of q_stride elements whose first H*hd hold the query heads; out [T, H*hd].
// part_o needs T*H*n_splits*hd floats and part_ml T*H*n_splits*2 floats when n_splits > 1.
// counters (optional): T * Hkv * ceil(H/Hkv/16) ints that are zero between calls; with them the
// block that finishes a (token, kv head) last merges the slices itself, without them a second
// kernel does.  head_dim must be a multiple of 8 and at most 128; page_size a multiple of 16;
// at most 32 slices.
namespace {
// The sizes that the kernel takes (every entry point refuses the others before it touches anything).
bool sizes_ok(int H, int Hkv, int hd, int page_size, int q_stride, int n_splits) {
    return H > 0 && Hkv > 0 && hd > 0 && hd % 8 == 0 && hd <= 128 && H % Hkv == 0 && page_size > 0 &&
           page_size % TILE == 0 && q_stride % 8 == 0 && n_splits >= 1 && n_splits <= MAX_SPLITS;
}
}  // namespace

// next_w, next_bytes (or null): weights that are read next on this stream; their first next_bytes
// are asked into L2 as the blocks finish.
// early_loads: non-zero when, of all keys and values that a token reads, only those at its own
// position can have been written by the kernel ahead on the stream (one new token per sequence):
// the others are then requested before that kernel is known to have finished.
//
// work, teams (or null, 0): the list of segments described in the kernel, teams + 1 offsets and then
// five integers a segment; the grid is then one block per (kv head, row tile, team), n_splits is the
// room for one token's parts in the scratch (part_o: T*H*n_splits*hd floats), no token may have more
// parts than that, and the counters are required when any token has more than one part.
LQ_EXPORT int lq_attn_decode_work(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                  const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                                  const int* slots, float* part_o, float* part_ml, int* counters, void* out, int T,
                                  int H, int Hkv, int hd, int page_size, float scale, int window, int n_splits,
                                  const int* work, int teams, const void* next_w, long next_bytes, int early_loads,
                                  cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (!sizes_ok(H, Hkv, hd, page_size, q_stride, n_splits)) return LQ_BAD_SIZE;
    if (n_splits > 1 && (!part_o || !part_ml)) return LQ_BAD_SIZE;
    if (work && (teams < 1 || teams > 65535 || (n_splits > 1 && !counters))) return LQ_BAD_SIZE;
#define LQ_GO(HD) return launch<HD>(q, q_stride, k_pages, v_pages, page_table, pt_stride, tok_pos, tok_seq, slots, \
                                    part_o, part_ml, counters, out, T, H, Hkv, hd, page_size, scale, window, n_splits, \
                                    work, teams, next_w, next_bytes, early_loads, stream)
    if (hd <= 32) LQ_GO(32);
    if (hd <= 64) LQ_GO(64);
    LQ_GO(128);
#undef LQ_GO
}

LQ_EXPORT int lq_attn_decode_next(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                  const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                                  const int* slots, float* part_o, float* part_ml, int* counters, void* out, int T,
                                  int H, int Hkv, int hd, int page_size, float scale, int window, int n_splits,
                                  const void* next_w, long next_bytes, int early_loads, cudaStream_t stream) {
    return lq_attn_decode_work(q, q_stride, k_pages, v_pages, page_table, pt_stride, tok_pos, tok_seq, slots, part_o,
                               part_ml, counters, out, T, H, Hkv, hd, page_size, scale, window, n_splits, nullptr, 0,
                               next_w, next_bytes, early_loads, stream);
}

LQ_EXPORT int lq_attn_decode_merged(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                    const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                                    const int* slots, float* part_o, float* part_ml, int* counters, void* out, int T,
                                    int H, int Hkv, int hd, int page_size, float scale, int window, int n_splits,
                                    cudaStream_t stream) {
    return lq_attn_decode_next(q, q_stride, k_pages, v_pages, page_table, pt_stride, tok_pos, tok_seq, slots, part_o,
                               part_ml, counters, out, T, H, Hkv, hd, page_size, scale, window, n_splits, nullptr, 0, 0, stream);
}

// The same without counters: the slices are merged by a second kernel.
LQ_EXPORT int lq_attn_decode(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                             const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                             const int* slots, float* part_o, float* part_ml, void* out, int T, int H, int Hkv,
                             int hd, int page_size, float scale, int window, int n_splits, cudaStream_t stream) {
    return lq_attn_decode_merged(q, q_stride, k_pages, v_pages, page_table, pt_stride, tok_pos, tok_seq, slots, part_o,
                                 part_ml, nullptr, out, T, H, Hkv, hd, page_size, scale, window, n_splits, stream);
}

// ------------------------------------------------------------------ the entry point that allocates nothing
// Declared and described in attn_decode_static.h.  No counterpart in the reference.
#include "attn_decode_static.h"

namespace {

constexpr int STATIC_MAX_DEVICES = 64;

// The scratch of lq_attn_decode_static.  In host code this name is a handle for the runtime,
// not a device address: the address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float lq_attn_static_scratch[LQ_ATTN_STATIC_FLOATS];

float* static_scratch_of_current_device(int* error) {
    static float* address[STATIC_MAX_DEVICES] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *error = (int)e; return nullptr; }
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) { *error = LQ_BAD_SIZE; return nullptr; }
    if (!address[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, lq_attn_static_scratch);   // the current device's copy of the array
        if (e != cudaSuccess) { *error = (int)e; return nullptr; }
        address[dev] = p;
    }
    *error = LQ_OK;
    return address[dev];
}

}  // namespace

LQ_EXPORT long lq_attn_decode_static_floats(void) { return LQ_ATTN_STATIC_FLOATS; }

LQ_EXPORT int lq_attn_decode_static(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                    const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                                    const int* slots, void* out, int T, int H, int Hkv, int head_dim, int page_size,
                                    float scale, int window, int n_splits, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    // Everything is checked before anything is queued: a refused call leaves the shared array alone.
    if (!sizes_ok(H, Hkv, head_dim, page_size, q_stride, n_splits)) return LQ_BAD_SIZE;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    int* counters = nullptr;
    if (n_splits > 1) {
        const long long rows = (long long)T * H * n_splits;
        const long long n_counters = (long long)T * Hkv * ((H / Hkv + 15) / 16);
        if (rows * (head_dim + 2) + n_counters > (long long)LQ_ATTN_STATIC_FLOATS) return LQ_STATIC_TOO_SMALL;
        int error = LQ_OK;
        float* base = static_scratch_of_current_device(&error);
        if (!base) return error;
        part_o = base;                                        // [T, H, n_splits, head_dim]
        part_ml = base + rows * head_dim;                     // [T, H, n_splits, 2]
        counters = (int*)(base + rows * (head_dim + 2));      // one per (token, kv head, row tile)
        // The counters must start at zero; whatever an earlier call left there is cleared (no allocation).
        cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)n_counters * sizeof(int), stream);
        if (e != cudaSuccess) return (int)e;
    }
    return lq_attn_decode_merged(q, q_stride, k_pages, v_pages, page_table, pt_stride, tok_pos, tok_seq, slots, part_o,
                                 part_ml, counters, out, T, H, Hkv, head_dim, page_size, scale, window, n_splits, stream);
}
