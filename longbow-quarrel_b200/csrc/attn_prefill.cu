// Causal grouped-query attention of many query tokens over the paged cache (prefill).
//
// A block takes 64 consecutive query tokens of one sequence and one query head; its four
// warps own 16 rows each.  Keys and values are read page by page (a page is a 64-key
// tile of one kv head) with cp.async into padded shared memory, two tiles in flight.
// Scores and the weighted sum run on the tensor cores (mma.sync m16n8k16, bfloat16 in,
// float32 out); the softmax is computed online in 32-bit: running maximum and sum per row,
// the output rescaled when the maximum grows.  A row at position p sees keys
// max(0, p - window + 1) .. p of its own sequence, whatever else the batch holds.
//
// The work list (which block serves which rows) is made on the host: sequence, first
// packed row, number of rows, position of the first row.
//
// Reference counterpart: att_fused_f16 (internal/device/kernels.metal:657-813) called once
// per row (internal/device/metal.go:1403-1424).
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int BLOCK_M = 64;
constexpr int BLOCK_N = 64;
constexpr int PAD = 8;          // elements of padding per shared-memory row: ldmatrix without bank conflicts
constexpr int NT = 128;

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
template <int HD>
__global__ void __launch_bounds__(NT)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_pages,
                    const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ page_table, int pt_stride,
                    const int* __restrict__ slots, const int* __restrict__ kv_len, const int* __restrict__ qb_seq,
                    const int* __restrict__ qb_row, const int* __restrict__ qb_rows, const int* __restrict__ qb_pos,
                    __nv_bfloat16* __restrict__ out, int H, int Hkv, int hd, float scale_log2, int window) {
    constexpr int LD = HD + PAD;                       // shared-memory row length in elements
    constexpr int KD = HD / 16;                        // k16 steps over the head dimension
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);              // [64][LD]
    __nv_bfloat16* sk = sq + BLOCK_M * LD;                                        // [2][64][LD]
    __nv_bfloat16* sv = sk + 2 * BLOCK_N * LD;                                    // [2][64][LD]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    // Heads vary fastest: the work list has the blocks with the most keys first, so the launch order is
    // longest-first over all heads and the short blocks fill the tail.
    const int blk = blockIdx.x / H, h = blockIdx.x % H;
    pdl_launch_dependents();
    pdl_wait();
    const int seq = qb_seq[blk], row0 = qb_row[blk], n_rows = qb_rows[blk], pos0 = qb_pos[blk];
    const int kvh = h / (H / Hkv);
    const int len = kv_len[seq];
    const int* pt = page_table + (size_t)slots[seq] * pt_stride;
    const int pos_last = pos0 + n_rows - 1;
    const int key_first = (window > 0 && pos0 >= window) ? pos0 - window + 1 : 0;
    const int tile_lo = key_first / BLOCK_N, tile_hi = pos_last / BLOCK_N;       // inclusive

    // ---- loads
    auto load_q = [&]() {
        for (int i = tid; i < BLOCK_M * (HD / 8); i += NT) {
            int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
            bool ok = r < n_rows && c < hd;
            const __nv_bfloat16* src = q + (size_t)(row0 + (ok ? r : 0)) * q_stride + (size_t)h * hd + (ok ? c : 0);
            cp_async16((uint32_t)__cvta_generic_to_shared(sq + r * LD + c), src, ok);
        }
    };
    auto load_kv = [&](int tile, int stage) {
        const int page = pt[tile];
        const size_t base = ((size_t)page * Hkv + kvh) * BLOCK_N * hd;
        const int kb = tile * BLOCK_N;
        for (int i = tid; i < BLOCK_N * (HD / 8); i += NT) {
            int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
            bool ok = kb + r < len && c < hd;
            size_t off = base + (size_t)(ok ? r : 0) * hd + (ok ? c : 0);
            cp_async16((uint32_t)__cvta_generic_to_shared(sk + (stage * BLOCK_N + r) * LD + c), k_pages + off, ok);
            cp_async16((uint32_t)__cvta_generic_to_shared(sv + (stage * BLOCK_N + r) * LD + c), v_pages + off, ok);
        }
    };
    load_q();
    load_kv(tile_lo, 0);
    cp_async_commit();

    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    uint32_t qf[KD][4];

    const int prow0 = pos0 + warp * 16 + g, prow1 = prow0 + 8;          // positions of this thread's two rows
    const bool row0ok = warp * 16 + g < n_rows, row1ok = warp * 16 + g + 8 < n_rows;
    const int warp_pos_hi = min(pos_last, pos0 + warp * 16 + 15);        // last position any row of the warp has
    const int warp_key_lo = (window > 0) ? max(0, pos0 + warp * 16 - window + 1) : 0;

    for (int tile = tile_lo; tile <= tile_hi; ++tile) {
        const int stage = (tile - tile_lo) & 1;
        if (tile + 1 <= tile_hi) load_kv(tile + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (tile == tile_lo) {
#pragma unroll
            for (int kk = 0; kk < KD; ++kk) {
                // A fragment of Q: matrices (rows 0-7, d 0-7), (rows 8-15, d 0-7), (rows 0-7, d 8-15), (rows 8-15, d 8-15)
                int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = kk * 16 + (lane >> 4) * 8;
                ldsm_x4((uint32_t)__cvta_generic_to_shared(sq + r * LD + c), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            }
        }
        const int kb = tile * BLOCK_N;
        if (kb <= warp_pos_hi && kb + BLOCK_N > warp_key_lo) {
            const __nv_bfloat16* ks = sk + stage * BLOCK_N * LD;
            const __nv_bfloat16* vs = sv + stage * BLOCK_N * LD;
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KD; ++kk) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {
                    // B fragments of K for key tiles 2jp and 2jp+1: matrices (keys 0-7, d 0-7), (keys 0-7, d 8-15),
                    // (keys 8-15, d 0-7), (keys 8-15, d 8-15)
                    int r = jp * 16 + (lane & 7) + (lane >> 4) * 8, c = kk * 16 + ((lane >> 3) & 1) * 8;
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4((uint32_t)__cvta_generic_to_shared(ks + r * LD + c), b0, b1, b2, b3);
                    mma_bf16(s[2 * jp], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
                    mma_bf16(s[2 * jp + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
                }
            }
            // mask and running maximum
            float tm0 = -CUDART_INF_F, tm1 = -CUDART_INF_F;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    int key = kb + j * 8 + 2 * t + i;
                    bool ok0 = row0ok && key <= prow0 && (window <= 0 || key > prow0 - window);
                    bool ok1 = row1ok && key <= prow1 && (window <= 0 || key > prow1 - window);
                    s[j][i] = ok0 ? s[j][i] * scale_log2 : -CUDART_INF_F;
                    s[j][2 + i] = ok1 ? s[j][2 + i] * scale_log2 : -CUDART_INF_F;
                    tm0 = fmaxf(tm0, s[j][i]);
                    tm1 = fmaxf(tm1, s[j][2 + i]);
                }
            tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
            tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
            tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
            tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
            const float nm0 = fmaxf(m0, tm0), nm1 = fmaxf(m1, tm1);
            const float u0 = nm0 == -CUDART_INF_F ? 0.f : nm0, u1 = nm1 == -CUDART_INF_F ? 0.f : nm1;
            const float c0 = exp2f(m0 - u0), c1 = exp2f(m1 - u1);     // m = -inf gives 0
            m0 = nm0;
            m1 = nm1;
            float ps0 = 0.f, ps1 = 0.f;
            uint32_t pa[4][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // The sum runs over the probabilities as the product will see them (rounded to
                // bfloat16), so that the weights of a row add up to one exactly.
                float p00 = round_bf16(exp2f(s[j][0] - u0)), p01 = round_bf16(exp2f(s[j][1] - u0));
                float p10 = round_bf16(exp2f(s[j][2] - u1)), p11 = round_bf16(exp2f(s[j][3] - u1));
                ps0 += p00 + p01;
                ps1 += p10 + p11;
                pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p00, p01);
                pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p10, p11);
            }
            l0 = l0 * c0 + ps0;
            l1 = l1 * c1 + ps1;
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {          // 16 keys per step
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    // B fragments of V, transposed on load: matrices (keys 0-7, d 0-7), (keys 8-15, d 0-7),
                    // (keys 0-7, d 8-15), (keys 8-15, d 8-15)
                    int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 16 + (lane >> 4) * 8;
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t((uint32_t)__cvta_generic_to_shared(vs + r * LD + c), b0, b1, b2, b3);
                    mma_bf16(o[2 * dp], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    mma_bf16(o[2 * dp + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        }
        __syncthreads();      // everyone is done with this stage before the next load overwrites it
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
        int d = j * 8 + 2 * t;
        if (d >= hd) continue;
        if (row0ok) {
            size_t off = ((size_t)(row0 + warp * 16 + g) * H + h) * hd + d;
            *reinterpret_cast<uint32_t*>(out + off) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
        }
        if (row1ok) {
            size_t off = ((size_t)(row0 + warp * 16 + g + 8) * H + h) * hd + d;
            *reinterpret_cast<uint32_t*>(out + off) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
        }
    }
}

template <int HD>
int launch(const void* q, int q_stride, const void* k_pages, const void* v_pages, const int* page_table, int pt_stride,
           const int* slots, const int* kv_len, const int* qb_seq, const int* qb_row, const int* qb_rows,
           const int* qb_pos, void* out, int n_blocks, int H, int Hkv, int hd, float scale, int window,
           cudaStream_t stream) {
    constexpr size_t smem = (size_t)(BLOCK_M + 4 * BLOCK_N) * (HD + PAD) * 2;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        configured = true;
    }
    dim3 grid(n_blocks * H);
    return launch_pdl(attn_prefill_kernel<HD>, grid, dim3(NT), smem, stream, (const __nv_bfloat16*)q, q_stride,
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table, pt_stride, slots, kv_len, qb_seq, qb_row,
        qb_rows, qb_pos, (__nv_bfloat16*)out, H, Hkv, hd, scale * 1.4426950408889634f, window);
}

}  // namespace

// q: rows of q_stride elements whose first H*hd hold the query heads; out [T, H*hd].
// qb_*: the work list, n_blocks entries: sequence, first packed row, rows (<= 64), position of the first row.
// head_dim a multiple of 8 and at most 128; the cache's page size must be 64.
LQ_EXPORT int lq_attn_prefill(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                              const int* page_table, int pt_stride, const int* slots, const int* kv_len,
                              const int* qb_seq, const int* qb_row, const int* qb_rows, const int* qb_pos, void* out,
                              int n_blocks, int H, int Hkv, int hd, int page_size, float scale, int window,
                              cudaStream_t stream) {
    if (n_blocks <= 0) return LQ_OK;
    if (hd % 8 || hd > 128 || hd <= 0 || H % Hkv || page_size != BLOCK_N || q_stride % 8) return LQ_BAD_SIZE;
#define LQ_GO(HD) return launch<HD>(q, q_stride, k_pages, v_pages, page_table, pt_stride, slots, kv_len, qb_seq, qb_row, \
                                    qb_rows, qb_pos, out, n_blocks, H, Hkv, hd, scale, window, stream)
    if (hd <= 32) LQ_GO(32);
    if (hd <= 64) LQ_GO(64);
    LQ_GO(128);
#undef LQ_GO
}
