// The work of one block on 16 rows of W for few rows of x: the body of gemm_skinny.cu's kernel, kept apart
// from the launch so that another kernel can run the same units (a kernel that ran a layer's three products
// after the attention in one launch, its blocks meeting at barriers, did so; measured on B200 it was 9 to 14 us
// a layer slower than three launches, balanced grid or not, and was taken out).
//
// Eight warps take the 32-wide k chunks in turn, stream their part of W straight from global memory
// into mma fragments (16-byte loads, no shared-memory staging: nothing is reused), multiply on the
// tensor cores with the tokens as the n side of m16n8k16, and sum their partial results in a fixed
// order through shared memory.  A unit keeps all of K, so an output depends only on its own row of x
// and W, not on how many other rows the batch has or on which block the unit ran.
//
// The k index inside a chunk is permuted the same way for W and x (a thread's eight consecutive
// elements feed two mma k-slot groups), which a dot product allows and which makes every global
// load a 16-byte one.
#pragma once
#include "common.cuh"

#define EPI_BF16 0
#define EPI_F32 1
#define EPI_RESID 2
#define EPI_SWIGLU 3
#define EPI_QKV 4       // q, k, v rows: rotate q and k, store k and v into the cache pages

namespace skinny {

constexpr int WARPS = 8;
constexpr int ROWS = 16;     // rows of W per unit
constexpr int KC = 32;       // k per chunk
// Chunks per warp and round.  With one group of 8 tokens a thread holds four chunks of W and of x; with two groups
// it holds two chunks of W and of both groups' x (the same registers): x read inside the products instead, from
// L1, made two groups 1.4 times slower than one.  More groups read x inside the products.
template <int MT> struct Round { static constexpr int UNROLL = MT == 2 ? 2 : 4; static constexpr int XG = MT <= 2 ? MT : 0; };

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// Activations.  FRESH: they may have been written by another block of the same launch, so the load
// must not be served from this SM's L1 or read-only cache (ld.global.cg: from L2); no kernel sets it now.
template <bool FRESH> __device__ __forceinline__ uint4 ld_act16(const void* p) {
    return FRESH ? __ldcg(reinterpret_cast<const uint4*>(p)) : __ldg(reinterpret_cast<const uint4*>(p));
}
template <bool FRESH> __device__ __forceinline__ float ld_actf(const float* p) { return FRESH ? __ldcg(p) : *p; }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// What the q/k/v epilogue needs beside the product: where each token stands and where its cache
// page is.  W holds H query heads, then Hkv key heads, then Hkv value heads, hd rows each.
struct QkvArgs {
    const float* cos_t;       // [positions, hd / 2] or null (no rotation)
    const float* sin_t;
    const int* tok_pos;
    const int* tok_seq;
    const int* slots;
    const int* page_table;
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    int pt_stride, H, Hkv, hd, page_size;
};

// RMS norm folded into the products on either side of it (null pointers: not used).
struct NormArgs {
    const float* in_sums;     // [rows of x, in_blocks]: sums of squares of the rows that x was made from
    int in_blocks;
    float in_inv_width, in_eps;
    const float* out_gain;    // [N] gain of the norm that reads the residual next (EPI_RESID only)
    __nv_bfloat16* out_x;     // [M, N] residual * gain
    float* out_sums;          // [M, units of this product]
};

// Work of one warp on `UNROLL` chunks: the W rows of the unit as mma A fragments, and (for
// few tokens) the tokens' x as B fragments, all loaded before any of it is used.
template <int MT>
struct Frags {
    static constexpr int UNROLL = Round<MT>::UNROLL;
    uint4 a0[UNROLL], a1[UNROLL];
    uint4 b[Round<MT>::XG > 0 ? Round<MT>::XG : 1][UNROLL];      // x of the tokens, kept for at most two groups of 8
};

template <int MT> struct Scratch {
    float red[WARPS][ROWS][MT * 8 + 1];
    float row_scale[MT * 8];
};

// One unit: 16 rows of W times all rows of x.  `begin` works out where the rows lie; `first_w` requests the
// first round of W (weights are written by no kernel, so this may run before the producer of x is known to
// have finished); `run` does the rest and needs x.
template <int MT, int EPI, bool FRESH>
struct Unit {
    static constexpr int UNROLL = Round<MT>::UNROLL;
    static constexpr int XG = Round<MT>::XG;
    static constexpr int STEP = WARPS * UNROLL;
    const __nv_bfloat16 *X, *w0, *w1;
    int M, N, K, n0, n1, c_hi, warp, lane, g, t;
    bool r0ok, r1ok;

    __device__ __forceinline__ void begin(const __nv_bfloat16* X_, const __nv_bfloat16* W, int M_, int N_, int K_,
                                          const QkvArgs& qkv, int unit) {
        X = X_; M = M_; N = N_; K = K_;
        warp = threadIdx.x >> 5; lane = threadIdx.x & 31;
        g = lane >> 2; t = lane & 3;
        // The unit's 16 rows of W.  Normally consecutive; for q/k/v the first 8 are elements
        // j0..j0+7 of a head and the last 8 their rotation partners j0 + hd/2 .. (same head).
        n0 = unit * ROWS; n1 = n0 + 8;
        if (EPI == EPI_QKV) {
            const int per_head = qkv.hd / 16;             // units per head
            const int head = unit / per_head, j0 = (unit % per_head) * 8;
            n0 = head * qkv.hd + j0;
            n1 = n0 + qkv.hd / 2;
        }
        const int r0 = n0 + g, r1 = n1 + g;
        r0ok = r0 < N; r1ok = r1 < N;
        w0 = W + (size_t)(r0ok ? r0 : 0) * K;
        w1 = W + (size_t)(r1ok ? r1 : 0) * K;
        c_hi = (K + KC - 1) / KC;                         // the unit's chunks of K: all of them
    }
    __device__ __forceinline__ void load_w(int c0, Frags<MT>& f) const {
        const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int c = c0 + u * WARPS;
            int k = c * KC + t * 8;
            bool ok = c < c_hi && k < K;       // K is a multiple of 8, so a started 16-byte piece is whole
            f.a0[u] = (ok && r0ok) ? ldg_stream(w0 + k) : zero;
            f.a1[u] = (ok && r1ok) ? ldg_stream(w1 + k) : zero;
        }
    }
    __device__ __forceinline__ void load_x(int c0, Frags<MT>& f) const {
        if (XG > 0) {
            const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                int c = c0 + u * WARPS;
                int k = c * KC + t * 8;
                bool ok = c < c_hi && k < K;
#pragma unroll
                for (int j = 0; j < XG; ++j)
                    f.b[j][u] = (ok && j * 8 + g < M) ? ld_act16<FRESH>(X + (size_t)(j * 8 + g) * K + k) : zero;
            }
        }
    }
    __device__ __forceinline__ void compute(int c0, const Frags<MT>& f, float (&acc)[MT][4]) const {
        const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int c = c0 + u * WARPS;
            int k = c * KC + t * 8;
            bool ok = c < c_hi && k < K;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                uint4 b;
                if (XG > 0) {
                    b = f.b[j][u];
                } else {
                    int m = j * 8 + g;
                    b = (ok && m < M) ? ld_act16<FRESH>(X + (size_t)m * K + k) : zero;
                }
                mma_bf16(acc[j], f.a0[u].x, f.a1[u].x, f.a0[u].y, f.a1[u].y, b.x, b.y);
                mma_bf16(acc[j], f.a0[u].z, f.a1[u].z, f.a0[u].w, f.a1[u].w, b.z, b.w);
            }
        }
    }
    // The first round of W, requested before x is known to be there.
    __device__ __forceinline__ void first_w(Frags<MT>& fa) const {
        if (warp < c_hi) load_w(warp, fa);
    }
    // Everything after first_w: x must be readable now.  `unit` and `n_units` place the unit's sums of
    // squares in norm.out_sums [M, n_units].
    __device__ __forceinline__ void run(Frags<MT>& fa, Scratch<MT>& sm, void* Cout, const float* residual,
                                        const QkvArgs& qkv, const NormArgs& norm, int unit, int n_units) const {
        // What the epilogue of this thread's first output needs from memory is requested now, so that it travels
        // while the weights stream: the residual and the next norm's gain, or the token's position, angles and
        // cache page (each a chain of dependent loads otherwise paid after the last product).
        constexpr int OUT_ROWS = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? ROWS / 2 : ROWS;
        const int m_first = threadIdx.x / OUT_ROWS, r_first = threadIdx.x % OUT_ROWS;
        const bool has_first = threadIdx.x < MT * 8 * OUT_ROWS && m_first < M;
        float pre_res = 0.f, pre_gain = 0.f, pre_cos = 1.f, pre_sin = 0.f;
        __nv_bfloat16* pre_dst = nullptr;
        if (EPI == EPI_RESID && has_first && n0 + r_first < N) {
            pre_res = ld_actf<FRESH>(residual + (size_t)m_first * N + n0 + r_first);
            if (norm.out_x) pre_gain = norm.out_gain[n0 + r_first];
        }
        if (EPI == EPI_QKV && has_first) {
            const int hd = qkv.hd, half = hd >> 1;
            const int head = n0 / hd, j = n0 % hd + r_first;
            const int pos = qkv.tok_pos[m_first];
            if (head < qkv.H + qkv.Hkv && qkv.cos_t) {
                pre_cos = qkv.cos_t[(size_t)pos * half + j];
                pre_sin = qkv.sin_t[(size_t)pos * half + j];
            }
            if (head < qkv.H) {
                pre_dst = (__nv_bfloat16*)Cout + (size_t)m_first * qkv.H * hd + (size_t)head * hd + j;
            } else {
                const int kvh = (head - qkv.H) % qkv.Hkv;
                __nv_bfloat16* pages = head < qkv.H + qkv.Hkv ? qkv.k_pages : qkv.v_pages;
                const int page = qkv.page_table[(size_t)qkv.slots[qkv.tok_seq[m_first]] * qkv.pt_stride + pos / qkv.page_size];
                pre_dst = pages + (((size_t)page * qkv.Hkv + kvh) * qkv.page_size + pos % qkv.page_size) * hd + j;
            }
        }
        if (norm.in_sums) {
            // 1 / rms of every row of x, from the sums its producer left: lanes stride over the blocks,
            // then a butterfly -- the same order whatever the batch.
            for (int m = warp; m < M; m += WARPS) {
                float ss = 0.f;
                for (int b = lane; b < norm.in_blocks; b += 32) ss += ld_actf<FRESH>(norm.in_sums + (size_t)m * norm.in_blocks + b);
                ss = warp_sum(ss);
                if (lane == 0) sm.row_scale[m] = rsqrtf(ss * norm.in_inv_width + norm.in_eps);
            }
        }
        float acc[MT][4];
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
        if (MT == 2) {
            // Two groups of tokens: a round is two chunks, so two rounds are kept in flight beyond the one that is
            // being multiplied (as many bytes of W on their way as with one group and rounds of four chunks).
            Frags<MT> fb, fc;
            int c0 = warp;
            if (c0 < c_hi) load_x(c0, fa);
            if (c0 + STEP < c_hi) { load_w(c0 + STEP, fb); load_x(c0 + STEP, fb); }
            while (c0 < c_hi) {
                if (c0 + 2 * STEP < c_hi) { load_w(c0 + 2 * STEP, fc); load_x(c0 + 2 * STEP, fc); }
                compute(c0, fa, acc);
                c0 += STEP;
                if (c0 >= c_hi) break;
                if (c0 + 2 * STEP < c_hi) { load_w(c0 + 2 * STEP, fa); load_x(c0 + 2 * STEP, fa); }
                compute(c0, fb, acc);
                c0 += STEP;
                if (c0 >= c_hi) break;
                if (c0 + 2 * STEP < c_hi) { load_w(c0 + 2 * STEP, fb); load_x(c0 + 2 * STEP, fb); }
                compute(c0, fc, acc);
                c0 += STEP;
            }
        } else if (MT <= 2) {
            // Few tokens: the loads of the next round are in flight while the current one is multiplied.
            Frags<MT> fb;
            int c0 = warp;
            if (c0 < c_hi) load_x(c0, fa);
            while (c0 < c_hi) {
                if (c0 + STEP < c_hi) { load_w(c0 + STEP, fb); load_x(c0 + STEP, fb); }
                compute(c0, fa, acc);
                c0 += STEP;
                if (c0 >= c_hi) break;
                if (c0 + STEP < c_hi) { load_w(c0 + STEP, fa); load_x(c0 + STEP, fa); }
                compute(c0, fb, acc);
                c0 += STEP;
            }
        } else {
            // More tokens need the registers for their sums: one round at a time.
            for (int c0 = warp; c0 < c_hi; c0 += STEP) {
                if (c0 != warp) load_w(c0, fa);
                compute(c0, fa, acc);
            }
        }
#pragma unroll
        for (int j = 0; j < MT; ++j) {
            sm.red[warp][g][j * 8 + 2 * t] = acc[j][0];
            sm.red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
            sm.red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
            sm.red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
        }
        __syncthreads();
        // One thread per (token, row): consecutive threads write consecutive outputs of a token.
        auto total = [&](int r, int m) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += sm.red[w][r][m];
            return v;
        };
        for (int i = threadIdx.x; i < MT * 8 * OUT_ROWS; i += WARPS * 32) {
            int m = i / OUT_ROWS, r = i % OUT_ROWS;
            if (EPI == EPI_RESID && norm.out_x) {
                // New residual, what the next norm makes of it, and the row's sum of squares over the
                // unit's columns: 16 consecutive lanes hold one row.
                const int n = n0 + r;
                const bool ok = m < M && n < N;
                const size_t o = (size_t)m * N + n;
                float v = 0.f;
                if (ok) {
                    const bool first = i == (int)threadIdx.x;
                    v = (first ? pre_res : ld_actf<FRESH>(residual + o)) + total(r, m) * (norm.in_sums ? sm.row_scale[m] : 1.f);
                    ((float*)Cout)[o] = v;
                    norm.out_x[o] = __float2bfloat16_rn(v * (first ? pre_gain : norm.out_gain[n]));
                }
                float ss = v * v;
#pragma unroll
                for (int d = 8; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
                if (r == 0 && m < M) norm.out_sums[(size_t)m * n_units + unit] = ss;
                continue;
            }
            if (m >= M) continue;
            const float sc = norm.in_sums ? sm.row_scale[m] : 1.f;
            float s = total(r, m) * sc;
            if (EPI == EPI_QKV) {
                // s and u are elements j and j + hd/2 of one head of token m.  (A thread has one output: 8 rows of
                // at most 16 tokens; where it stands and where it goes was looked up before the products.)
                float u = total(r + 8, m) * sc;
                const float y0 = s * pre_cos - u * pre_sin, y1 = s * pre_sin + u * pre_cos;
                pre_dst[0] = __float2bfloat16_rn(y0);
                pre_dst[qkv.hd >> 1] = __float2bfloat16_rn(y1);
            } else if (EPI == EPI_SWIGLU) {
                float u = total(r + 8, m) * sc;
                int f = (n0 >> 1) + r;
                if (f < (N >> 1))
                    ((__nv_bfloat16*)Cout)[(size_t)m * (N >> 1) + f] = __float2bfloat16_rn(u * (s / (1.0f + expf(-s))));
            } else {
                int n = n0 + r;
                if (n >= N) continue;
                size_t o = (size_t)m * N + n;
                if (EPI == EPI_BF16) ((__nv_bfloat16*)Cout)[o] = __float2bfloat16_rn(s);
                else if (EPI == EPI_F32) ((float*)Cout)[o] = s;
                else ((float*)Cout)[o] = (i == (int)threadIdx.x ? pre_res : ld_actf<FRESH>(residual + o)) + s;
            }
        }
    }
};

static inline int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

}  // namespace skinny
