// y = x . W^T for few rows of x (decoding: one token for each sequence of the batch).
//
// With at most 64 rows every weight is used once, so the product is bound by
// reading W from HBM.  Each block owns 16 rows of W and all of K; its 8 warps take
// the 32-wide k chunks in turn, stream their part of W straight from global memory
// into mma fragments (16-byte loads, no shared-memory staging: nothing is reused),
// multiply on the tensor cores with the tokens as the n side of m16n8k16, and sum
// their partial results in a fixed order through shared memory.  A block keeps all of
// K: measured on B200, cutting K between blocks made every shape slower.  An output therefore
// depends only on its own row of x and W, not on how many other rows the batch has.
//
// The k index inside a chunk is permuted the same way for W and x (a thread's eight
// consecutive elements feed two mma k-slots groups), which a dot product allows and
// which makes every global load a 16-byte one.
//
// Epilogues: bfloat16 store; float32 store; float32 residual add in place;
// SwiGLU over weight rows interleaved in blocks of 8 (8 gate rows, then their 8 up
// rows), writing up * silu(gate).
//
// RMS norm around the product, without a kernel of its own: the residual epilogue can also
// write what the next norm makes of the new residual r, split in two -- r * gain rounded to
// bfloat16, and for every row the sum of r^2 over the block's 16 columns.  A product that reads
// such rows multiplies its result by 1 / sqrt(sum / width + eps), summed over the blocks in a
// fixed order: (x * gain * s) . w = s * ((x * gain) . w).
//
// Reference counterpart: the mat-vec kernels linear_f16 / linear_f16_f32
// (internal/device/kernels.metal:105-132,1084-1106), one output row per SIMD group.
#include "common.cuh"

#define EPI_BF16 0
#define EPI_F32 1
#define EPI_RESID 2
#define EPI_SWIGLU 3
#define EPI_QKV 4       // q, k, v rows: rotate q and k, store k and v into the cache pages

namespace {

constexpr int WARPS = 8;
constexpr int ROWS = 16;     // rows of W per block
constexpr int KC = 32;       // k per chunk
constexpr int UNROLL = 4;    // chunks per warp and round

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
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
    float* out_sums;          // [M, blocks of this launch]
};

// The weights that the stream reads next (of the product that follows this one): the last blocks of
// this launch ask for their first bytes to be brought into L2, so that HBM stays busy while this
// launch runs out and the next one starts from L2.  ptr null: nothing is asked for.
struct NextWeights {
    const char* ptr;
    unsigned bytes_per_block;   // a multiple of 16
    int first_block;            // blocks from this one on ask for one piece each
};

// Work of one warp on `UNROLL` chunks: the W rows of the block as mma A fragments, and (for
// few tokens) the tokens' x as B fragments, all loaded before any of it is used.
template <int MT>
struct Frags {
    uint4 a0[UNROLL], a1[UNROLL];
    uint4 b[UNROLL];                    // x of the tokens, kept only when there is one group of 8 tokens
};

template <int MT, int EPI>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, void* Cout,
                   const float* residual, int M, int N, int K, const QkvArgs qkv, const NormArgs norm,
                   const NextWeights next) {
    __shared__ float red[WARPS][ROWS][MT * 8 + 1];
    __shared__ float row_scale[MT * 8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // The block's 16 rows of W.  Normally consecutive; for q/k/v the first 8 are elements
    // j0..j0+7 of a head and the last 8 their rotation partners j0 + hd/2 .. (same head).
    int n0 = blockIdx.x * ROWS, n1 = n0 + 8;
    if (EPI == EPI_QKV) {
        const int per_head = qkv.hd / 16;             // blocks per head
        const int head = blockIdx.x / per_head, j0 = (blockIdx.x % per_head) * 8;
        n0 = head * qkv.hd + j0;
        n1 = n0 + qkv.hd / 2;
    }
    const int r0 = n0 + g, r1 = n1 + g;
    const bool r0ok = r0 < N, r1ok = r1 < N;
    const __nv_bfloat16* w0 = W + (size_t)(r0ok ? r0 : 0) * K;
    const __nv_bfloat16* w1 = W + (size_t)(r1ok ? r1 : 0) * K;
    const int c_lo = 0, c_hi = (K + KC - 1) / KC;      // the block's chunks of K: all of them
    constexpr int STEP = WARPS * UNROLL;

    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    const uint4 zero = make_uint4(0, 0, 0, 0);
    auto load_w = [&](int c0, Frags<MT>& f) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int c = c0 + u * WARPS;
            int k = c * KC + t * 8;
            bool ok = c < c_hi && k < K;       // K is a multiple of 8, so a started 16-byte piece is whole
            f.a0[u] = (ok && r0ok) ? ldg_stream(w0 + k) : zero;
            f.a1[u] = (ok && r1ok) ? ldg_stream(w1 + k) : zero;
        }
    };
    auto load_x = [&](int c0, Frags<MT>& f) {
        if (MT == 1) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                int c = c0 + u * WARPS;
                int k = c * KC + t * 8;
                bool ok = c < c_hi && k < K;
                f.b[u] = (ok && g < M) ? ldg_cached(X + (size_t)g * K + k) : zero;
            }
        }
    };
    auto load = [&](int c0, Frags<MT>& f) { load_w(c0, f); load_x(c0, f); };
    // Weights are written by no kernel, so the first round of them is loaded before the kernel
    // ahead of this one is known to have finished; x and the output wait for pdl_wait().
    pdl_launch_dependents();
    if (next.ptr && (int)blockIdx.x >= next.first_block && threadIdx.x == 0) {
        const char* piece = next.ptr + (size_t)((int)blockIdx.x - next.first_block) * next.bytes_per_block;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(piece), "r"(next.bytes_per_block) : "memory");
    }
    auto compute = [&](int c0, const Frags<MT>& f) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int c = c0 + u * WARPS;
            int k = c * KC + t * 8;
            bool ok = c < c_hi && k < K;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                uint4 b;
                if (MT == 1) {
                    b = f.b[u];
                } else {
                    int m = j * 8 + g;
                    b = (ok && m < M) ? ldg_cached(X + (size_t)m * K + k) : zero;
                }
                mma_bf16(acc[j], f.a0[u].x, f.a1[u].x, f.a0[u].y, f.a1[u].y, b.x, b.y);
                mma_bf16(acc[j], f.a0[u].z, f.a1[u].z, f.a0[u].w, f.a1[u].w, b.z, b.w);
            }
        }
    };
    if (MT <= 2) {
        // Few tokens: the loads of the next round are in flight while the current one is multiplied.
        Frags<MT> fa, fb;
        int c0 = c_lo + warp;
        if (c0 < c_hi) load_w(c0, fa);
        pdl_wait();
        if (c0 < c_hi) load_x(c0, fa);
        while (c0 < c_hi) {
            if (c0 + STEP < c_hi) load(c0 + STEP, fb);
            compute(c0, fa);
            c0 += STEP;
            if (c0 >= c_hi) break;
            if (c0 + STEP < c_hi) load(c0 + STEP, fa);
            compute(c0, fb);
            c0 += STEP;
        }
    } else {
        // More tokens need the registers for their sums: one round at a time.
        Frags<MT> fa;
        int c0 = c_lo + warp;
        if (c0 < c_hi) load_w(c0, fa);
        pdl_wait();
        for (; c0 < c_hi; c0 += STEP) {
            if (c0 != c_lo + warp) load_w(c0, fa);
            compute(c0, fa);
        }
    }
    if (norm.in_sums) {
        // 1 / rms of every row of x, from the sums its producer left: lanes stride over the blocks,
        // then a butterfly -- the same order whatever the batch.
        for (int m = warp; m < M; m += WARPS) {
            float ss = 0.f;
            for (int b = lane; b < norm.in_blocks; b += 32) ss += norm.in_sums[(size_t)m * norm.in_blocks + b];
            ss = warp_sum(ss);
            if (lane == 0) row_scale[m] = rsqrtf(ss * norm.in_inv_width + norm.in_eps);
        }
    }
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        red[warp][g][j * 8 + 2 * t] = acc[j][0];
        red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
        red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
        red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    // One thread per (token, row): consecutive threads write consecutive outputs of a token.
    constexpr int OUT_ROWS = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? ROWS / 2 : ROWS;
    auto total = [&](int r, int m) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[w][r][m];
        return v;
    };
    for (int i = threadIdx.x; i < MT * 8 * OUT_ROWS; i += WARPS * 32) {
        int m = i / OUT_ROWS, r = i % OUT_ROWS;
        if (EPI == EPI_RESID && norm.out_x) {
            // New residual, what the next norm makes of it, and the row's sum of squares over the
            // block's columns: 16 consecutive lanes hold one row.
            const int n = n0 + r;
            const bool ok = m < M && n < N;
            const size_t o = (size_t)m * N + n;
            float v = 0.f;
            if (ok) {
                v = residual[o] + total(r, m) * (norm.in_sums ? row_scale[m] : 1.f);
                ((float*)Cout)[o] = v;
                norm.out_x[o] = __float2bfloat16_rn(v * norm.out_gain[n]);
            }
            float ss = v * v;
#pragma unroll
            for (int d = 8; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
            if (r == 0 && m < M) norm.out_sums[(size_t)m * gridDim.x + blockIdx.x] = ss;
            continue;
        }
        if (m >= M) continue;
        const float sc = norm.in_sums ? row_scale[m] : 1.f;
        float s = total(r, m) * sc;
        if (EPI == EPI_QKV) {
            // s and u are elements j and j + hd/2 of one head of token m.
            float u = total(r + 8, m) * sc;
            const int hd = qkv.hd, half = hd >> 1;
            const int head = n0 / hd, j = n0 % hd + r;
            const int pos = qkv.tok_pos[m];
            if (head < qkv.H + qkv.Hkv && qkv.cos_t) {
                float c = qkv.cos_t[(size_t)pos * half + j], sn = qkv.sin_t[(size_t)pos * half + j];
                float y0 = s * c - u * sn, y1 = s * sn + u * c;
                s = y0;
                u = y1;
            }
            if (head < qkv.H) {
                __nv_bfloat16* o = (__nv_bfloat16*)Cout + (size_t)m * qkv.H * hd + (size_t)head * hd + j;
                o[0] = __float2bfloat16_rn(s);
                o[half] = __float2bfloat16_rn(u);
            } else {
                const int kvh = (head - qkv.H) % qkv.Hkv;
                __nv_bfloat16* pages = head < qkv.H + qkv.Hkv ? qkv.k_pages : qkv.v_pages;
                const int page = qkv.page_table[(size_t)qkv.slots[qkv.tok_seq[m]] * qkv.pt_stride + pos / qkv.page_size];
                __nv_bfloat16* o = pages + (((size_t)page * qkv.Hkv + kvh) * qkv.page_size + pos % qkv.page_size) * hd + j;
                o[0] = __float2bfloat16_rn(s);
                o[half] = __float2bfloat16_rn(u);
            }
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
            else ((float*)Cout)[o] = residual[o] + s;
        }
    }
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

template <int MT>
int launch_mt(const void* X, const void* W, void* C, const float* residual, int M, int N, int K, int epi,
              cudaStream_t stream, const NormArgs norm, const void* next_w, long next_bytes,
              const QkvArgs qkv = QkvArgs{}) {
    dim3 grid((N + ROWS - 1) / ROWS), block(WARPS * 32);
    // The blocks of the last wave (two a SM) share the bytes asked for.
    NextWeights next{nullptr, 0u, 0};
    if (next_w && next_bytes >= 16 && !((uintptr_t)next_w & 15)) {
        const int askers = (int)grid.x < 2 * sm_count() ? (int)grid.x : 2 * sm_count();
        const long piece = next_bytes / askers / 16 * 16;
        if (piece > 0) next = NextWeights{(const char*)next_w, (unsigned)piece, (int)grid.x - askers};
    }
    const __nv_bfloat16* x = (const __nv_bfloat16*)X;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    switch (epi) {
        case EPI_BF16: return launch_pdl(gemm_skinny_kernel<MT, EPI_BF16>, grid, block, 0, stream, x, w, C, residual, M, N, K, qkv, norm, next);
        case EPI_F32: return launch_pdl(gemm_skinny_kernel<MT, EPI_F32>, grid, block, 0, stream, x, w, C, residual, M, N, K, qkv, norm, next);
        case EPI_RESID: return launch_pdl(gemm_skinny_kernel<MT, EPI_RESID>, grid, block, 0, stream, x, w, C, residual, M, N, K, qkv, norm, next);
        case EPI_SWIGLU: return launch_pdl(gemm_skinny_kernel<MT, EPI_SWIGLU>, grid, block, 0, stream, x, w, C, residual, M, N, K, qkv, norm, next);
        case EPI_QKV: return launch_pdl(gemm_skinny_kernel<MT, EPI_QKV>, grid, block, 0, stream, x, w, C, residual, M, N, K, qkv, norm, next);
        default: return LQ_BAD_DTYPE;
    }
    return lq_launch_status();
}

}  // namespace

// X [M, K] bf16, W [N, K] bf16; M <= 64, K % 8 == 0.  For EPI_SWIGLU, N counts the
// interleaved gate and up rows (N % 16 == 0) and C is [M, N / 2].
// in_sums (or null): x is (rows * gain) of an RMS norm whose 1 / rms is still to be applied;
// in_sums [M, in_blocks] holds the rows' sums of squares, in_inv_width = 1 / width, in_eps the norm's eps.
// next_w, next_bytes (or null): weights that are read next on this stream; their first next_bytes
// are asked into L2 while this product runs out.
// out_gain, out_x, out_sums (EPI_RESID only, or null): also write (new residual * out_gain) as
// bfloat16 [M, N] and the sums of squares [M, lq_gemm_skinny_blocks(N)] for the product that follows.
LQ_EXPORT int lq_gemm_skinny(const void* X, const void* W, void* C, const float* residual, int M, int N, int K,
                             int epi, const float* in_sums, int in_blocks, float in_inv_width, float in_eps,
                             const float* out_gain, void* out_x, float* out_sums, const void* next_w, long next_bytes,
                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LQ_OK;
    if (M > 64 || K % 8 != 0 || K <= 0) return LQ_BAD_SIZE;
    if (epi == EPI_SWIGLU && N % 16 != 0) return LQ_BAD_SIZE;
    if (epi == EPI_RESID && residual == nullptr) return LQ_BAD_SIZE;
    if (in_sums && in_blocks <= 0) return LQ_BAD_SIZE;
    if (out_x && (epi != EPI_RESID || !out_gain || !out_sums)) return LQ_BAD_SIZE;
    const NormArgs norm{in_sums, in_blocks, in_inv_width, in_eps, out_x ? out_gain : nullptr,
                        (__nv_bfloat16*)out_x, out_x ? out_sums : nullptr};
    int mt = (M + 7) / 8;
    switch (mt) {
        case 1: return launch_mt<1>(X, W, C, residual, M, N, K, epi, stream, norm, next_w, next_bytes);
        case 2: return launch_mt<2>(X, W, C, residual, M, N, K, epi, stream, norm, next_w, next_bytes);
        case 3: case 4: return launch_mt<4>(X, W, C, residual, M, N, K, epi, stream, norm, next_w, next_bytes);
        default: return launch_mt<8>(X, W, C, residual, M, N, K, epi, stream, norm, next_w, next_bytes);
    }
}

// Blocks of a product with N output columns: the second size of out_sums.
LQ_EXPORT int lq_gemm_skinny_blocks(int N) { return (N + ROWS - 1) / ROWS; }

// The q/k/v projection of decoding with its epilogue fused: X [M <= 16, K] . W^T for
// W [(H + 2 Hkv) hd, K]; q and k are rotated by the cos/sin tables at each token's position
// (tables null: no rotation); q goes to q_out [M, H hd], k and v go into the token's cache page.
// hd % 16 == 0.  Replaces the product, the rotation kernel and the cache write of a decode step.
// in_sums ...: as for lq_gemm_skinny.
LQ_EXPORT int lq_gemm_skinny_qkv(const void* X, const void* W, void* q_out, int M, int K, const float* cos_t,
                                 const float* sin_t, const int* tok_pos, const int* tok_seq, const int* slots,
                                 const int* page_table, int pt_stride, void* k_pages, void* v_pages, int H, int Hkv,
                                 int hd, int page_size, const float* in_sums, int in_blocks, float in_inv_width,
                                 float in_eps, const void* next_w, long next_bytes, cudaStream_t stream) {
    if (M <= 0) return LQ_OK;
    if (M > 16 || K % 8 != 0 || K <= 0 || hd % 16 != 0 || H <= 0 || Hkv <= 0) return LQ_BAD_SIZE;
    if (in_sums && in_blocks <= 0) return LQ_BAD_SIZE;
    QkvArgs a{cos_t, sin_t, tok_pos, tok_seq, slots, page_table, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
              pt_stride, H, Hkv, hd, page_size};
    const NormArgs norm{in_sums, in_blocks, in_inv_width, in_eps, nullptr, nullptr, nullptr};
    const int N = (H + 2 * Hkv) * hd;
    if (M <= 8) return launch_mt<1>(X, W, q_out, nullptr, M, N, K, EPI_QKV, stream, norm, next_w, next_bytes, a);
    return launch_mt<2>(X, W, q_out, nullptr, M, N, K, EPI_QKV, stream, norm, next_w, next_bytes, a);
}
