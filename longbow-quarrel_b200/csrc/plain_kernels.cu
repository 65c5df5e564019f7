// Plain kernels for every operation of the decoder, in 32-bit and in bfloat16 storage.
//
// These are the kernels of the true 32-bit path (every product and sum in IEEE
// float, FFMA on the CUDA cores, no tensor-core mode of reduced precision), and the
// twins beside which each tuned bfloat16 kernel is checked.  Every reduction runs in
// an order that depends only on the row's own sizes, never on what else is in the
// batch, so a position's result does not change with the way the work is cut.
//
// Counterparts in the reference (23skdu/longbow-quarrel), by formula:
//   embedding     internal/device/kernels.metal:465   embedding_f16
//   rmsnorm       internal/device/kernels.metal:905   rmsnorm_f32_to_f16_v4
//   linear        internal/device/kernels.metal:105   linear_f16 (y = x W^T, F32 accumulate)
//   rope          internal/device/kernels.metal:430   rope_f16 (half-split pairs)
//   store K/V     internal/device/kernels.metal:1221  store_kv_f16
//   attention     internal/device/kernels.metal:657   att_fused_f16
//   swiglu        internal/device/cpu_ref.go:133      CPUSwiGLU (no clamp)
#include "common.cuh"
#include <math_constants.h>

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                 float* __restrict__ out, int D, int V) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= V) tok = 0;  // range is checked on the host before launch
    const TW* row = table + (size_t)tok * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[(size_t)t * D + i] = to_f32(row[i]);
}

LQ_EXPORT int lq_embedding(const void* table, int table_dtype, const int* tokens, float* out,
                           int T, int D, int V, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (table_dtype == LQ_F32)
        return launch_pdl(embedding_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)table, tokens, out, D, V);
    else if (table_dtype == LQ_BF16)
        return launch_pdl(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)table, tokens, out, D, V);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

// ------------------------------------------------------------------ rmsnorm
// x is the 32-bit residual stream.  rows (optional) picks the rows to normalise.
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                               const int* __restrict__ rows, TO* __restrict__ out, int D, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float partial[32];
    __shared__ float scale_s;
    int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = xr[i];
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    float scale = scale_s;
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        out[(size_t)r * D + i] = from_f32<TO>(xr[i] * scale * gain[i]);
}

// Rows whose length is a multiple of 4 and at most 256 * 4 * RMS_VEC: each thread keeps its
// part of the row in registers (one read of x), float4 loads, packed stores.  The sum of squares
// runs in an order fixed by the row length alone.
constexpr int RMS_VEC = 8;   // float4 pieces per thread

template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ gain, const int* __restrict__ rows,
                   TO* __restrict__ out, int D, float eps) {
    __shared__ float partial[8];
    __shared__ float scale_s;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, n4 = D >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * D);
    float4 v[RMS_VEC];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        int c = threadIdx.x + i * 256;
        v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        s = fmaf(v[i].x, v[i].x, s); s = fmaf(v[i].y, v[i].y, s);
        s = fmaf(v[i].z, v[i].z, s); s = fmaf(v[i].w, v[i].w, s);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        int c = threadIdx.x + i * 256;
        if (c >= n4) break;
        float4 g = g4[c];
        float o0 = v[i].x * scale * g.x, o1 = v[i].y * scale * g.y, o2 = v[i].z * scale * g.z, o3 = v[i].w * scale * g.w;
        if (sizeof(TO) == 4) {
            reinterpret_cast<float4*>(out + (size_t)r * D)[c] = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
            uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            reinterpret_cast<uint2*>(out + (size_t)r * D)[c] = packed;
        }
    }
}

LQ_EXPORT int lq_rmsnorm(const float* x, const float* gain, const int* rows, void* out, int out_dtype,
                         int n_rows, int D, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return LQ_OK;
    if (out_dtype != LQ_F32 && out_dtype != LQ_BF16) return LQ_BAD_DTYPE;
    const bool vec = D % 4 == 0 && D <= 256 * 4 * RMS_VEC && (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)out) & 15) == 0;
    if (out_dtype == LQ_F32)
        return vec ? launch_pdl(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (float*)out, D, eps)
                   : launch_pdl(rmsnorm_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (float*)out, D, eps);
    return vec ? launch_pdl(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (__nv_bfloat16*)out, D, eps)
               : launch_pdl(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (__nv_bfloat16*)out, D, eps);
}

// ------------------------------------------------------------------ linear (FFMA)
// C[M,N] = A[M,K] . W[N,K]^T (+ residual[M,N]).  Each output is one chain of fused
// multiply-adds over k = 0..K-1 in rising order, whatever M is.
constexpr int GT = 64;   // tile of C
constexpr int GK = 16;   // k step

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C,
                  const float* __restrict__ residual, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[GK][GT + 1];
    __shared__ float Ws[GK][GT + 1];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int i = threadIdx.x; i < GT * GK; i += 256) {
            int r = i / GK, c = i % GK;
            int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * K + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (residual) v += residual[(size_t)gm * N + gn];
            C[(size_t)gm * N + gn] = from_f32<TC>(v);
        }
    }
}

template <typename TA, typename TW>
static int gemm_plain_c(const void* A, const void* W, void* C, int c_dtype, const float* residual,
                        int M, int N, int K, cudaStream_t stream) {
    dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
    if (c_dtype == LQ_F32)
        return launch_pdl(gemm_plain_kernel<TA, TW, float>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, (float*)C, residual, M, N, K);
    else if (c_dtype == LQ_BF16)
        return launch_pdl(gemm_plain_kernel<TA, TW, __nv_bfloat16>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, (__nv_bfloat16*)C, residual, M, N, K);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

LQ_EXPORT int lq_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                            const float* residual, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LQ_OK;
    if (a_dtype == LQ_F32 && w_dtype == LQ_F32) return gemm_plain_c<float, float>(A, W, C, c_dtype, residual, M, N, K, stream);
    if (a_dtype == LQ_F32 && w_dtype == LQ_BF16) return gemm_plain_c<float, __nv_bfloat16>(A, W, C, c_dtype, residual, M, N, K, stream);
    if (a_dtype == LQ_BF16 && w_dtype == LQ_F32) return gemm_plain_c<__nv_bfloat16, float>(A, W, C, c_dtype, residual, M, N, K, stream);
    if (a_dtype == LQ_BF16 && w_dtype == LQ_BF16) return gemm_plain_c<__nv_bfloat16, __nv_bfloat16>(A, W, C, c_dtype, residual, M, N, K, stream);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ rope + cache write
// qkv [T, (H + 2 Hkv) hd] holds q, k, v of each token side by side.  q and k are
// rotated in place (pairs i, i + hd/2; angle = position * f_i from the cos/sin
// tables, which may be null for no rotation); k and v are then stored into the
// token's cache page.  A page holds [Hkv][page_size][hd] of one layer.
// With has_kv == 0 the rows hold q only (a layer that reads another layer's cache).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ slots,
                                     const int* __restrict__ page_table, int pt_stride,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     int H, int Hkv, int hd, int page_size, int has_kv) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x;
    int pos = tok_pos[t];
    int half = hd >> 1;
    int row_w = (H + (has_kv ? 2 * Hkv : 0)) * hd;
    T* row = qkv + (size_t)t * row_w;
    const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (has_kv) {
        int slot = slots[tok_seq[t]];
        int page = page_table[(size_t)slot * pt_stride + pos / page_size];
        size_t base = ((size_t)page * Hkv * page_size + (pos % page_size)) * hd;
        kdst = k_pages + base;
        vdst = v_pages + base;
    }
    int n_rot = (H + (has_kv ? Hkv : 0)) * half;
    for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
        int head = i / half, j = i % half;
        T* p = row + (size_t)head * hd;
        float x0 = to_f32(p[j]), x1 = to_f32(p[j + half]);
        float y0 = x0, y1 = x1;
        if (cs) {
            float c = cs[j], s = sn[j];
            y0 = x0 * c - x1 * s;
            y1 = x0 * s + x1 * c;
        }
        T o0 = from_f32<T>(y0), o1 = from_f32<T>(y1);
        p[j] = o0;
        p[j + half] = o1;
        if (head >= H) {
            T* d = kdst + (size_t)(head - H) * page_size * hd;
            d[j] = o0;
            d[j + half] = o1;
        }
    }
    if (has_kv) {
        const T* vsrc = row + (size_t)(H + Hkv) * hd;
        for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) {
            int head = i / hd, j = i % hd;
            vdst[(size_t)head * page_size * hd + j] = vsrc[i];
        }
    }
}

// The same work with 16-byte accesses, for half head sizes that are a multiple of the vector
// length (8 bfloat16 or 4 float32): a thread rotates VEC pairs of one head at a time.
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
                         const int* __restrict__ page_table, int pt_stride, T* __restrict__ k_pages,
                         T* __restrict__ v_pages, int H, int Hkv, int hd, int page_size, int has_kv) {
    constexpr int VEC = Vec16<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = hd >> 1, pieces = half / VEC;
    const int row_w = (H + (has_kv ? 2 * Hkv : 0)) * hd;
    T* row = qkv + (size_t)t * row_w;
    const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (has_kv) {
        int slot = slots[tok_seq[t]];
        int page = page_table[(size_t)slot * pt_stride + pos / page_size];
        size_t base = ((size_t)page * Hkv * page_size + (pos % page_size)) * hd;
        kdst = k_pages + base;
        vdst = v_pages + base;
    }
    const int n_rot = (H + (has_kv ? Hkv : 0)) * pieces;
    for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
        const int head = i / pieces, j = (i % pieces) * VEC;
        T* p = row + (size_t)head * hd;
        uint4 a = *reinterpret_cast<const uint4*>(p + j), b = *reinterpret_cast<const uint4*>(p + j + half);
        const T* x0 = reinterpret_cast<const T*>(&a);
        const T* x1 = reinterpret_cast<const T*>(&b);
        uint4 oa, ob;
        T* y0 = reinterpret_cast<T*>(&oa);
        T* y1 = reinterpret_cast<T*>(&ob);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float u = to_f32(x0[e]), w = to_f32(x1[e]);
            float c = cs ? cs[j + e] : 1.f, s = sn ? sn[j + e] : 0.f;
            y0[e] = from_f32<T>(u * c - w * s);
            y1[e] = from_f32<T>(u * s + w * c);
        }
        *reinterpret_cast<uint4*>(p + j) = oa;
        *reinterpret_cast<uint4*>(p + j + half) = ob;
        if (head >= H) {
            T* d = kdst + (size_t)(head - H) * page_size * hd;
            *reinterpret_cast<uint4*>(d + j) = oa;
            *reinterpret_cast<uint4*>(d + j + half) = ob;
        }
    }
    if (has_kv) {
        const T* vsrc = row + (size_t)(H + Hkv) * hd;
        const int per_head = hd / VEC;
        for (int i = threadIdx.x; i < Hkv * per_head; i += blockDim.x) {
            int head = i / per_head, j = (i % per_head) * VEC;
            *reinterpret_cast<uint4*>(vdst + (size_t)head * page_size * hd + j) =
                *reinterpret_cast<const uint4*>(vsrc + (size_t)head * hd + j);
        }
    }
}

template <typename T>
static int rope_launch(void* qkv, const float* cos_t, const float* sin_t, const int* tok_pos, const int* tok_seq,
                       const int* slots, const int* page_table, int pt_stride, void* k_pages, void* v_pages, int Tn,
                       int H, int Hkv, int hd, int page_size, int has_kv, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    const bool vec = (hd / 2) % VEC == 0 && (((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
    auto kernel = vec ? rope_kv_write_vec_kernel<T> : rope_kv_write_kernel<T>;
    return launch_pdl(kernel, dim3(Tn), dim3(256), 0, stream, (T*)qkv, cos_t, sin_t, tok_pos, tok_seq, slots, page_table,
                      pt_stride, (T*)k_pages, (T*)v_pages, H, Hkv, hd, page_size, has_kv);
}

LQ_EXPORT int lq_rope_kv_write(void* qkv, int dtype, const float* cos_t, const float* sin_t,
                               const int* tok_pos, const int* tok_seq, const int* slots,
                               const int* page_table, int pt_stride, void* k_pages, void* v_pages,
                               int T, int H, int Hkv, int hd, int page_size, int has_kv,
                               cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (hd % 2) return LQ_BAD_SIZE;
    if (dtype == LQ_F32)
        return rope_launch<float>(qkv, cos_t, sin_t, tok_pos, tok_seq, slots, page_table, pt_stride, k_pages, v_pages,
                                  T, H, Hkv, hd, page_size, has_kv, stream);
    if (dtype == LQ_BF16)
        return rope_launch<__nv_bfloat16>(qkv, cos_t, sin_t, tok_pos, tok_seq, slots, page_table, pt_stride, k_pages,
                                          v_pages, T, H, Hkv, hd, page_size, has_kv, stream);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ attention over the cache
// One block per (token, query head).  Keys start..pos of the token's own sequence are
// read from its pages in chunks of ATT_CHUNK; the running maximum, sum and output
// are carried from chunk to chunk, and inside a chunk every sum runs in key order.
// The same kernel serves a prompt's tokens and a decoded token, so both reduce in the
// same order.
constexpr int ATT_CHUNK = 128;

template <typename T>
__global__ void __launch_bounds__(ATT_CHUNK)
attention_plain_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages,
                       const T* __restrict__ v_pages, const int* __restrict__ page_table, int pt_stride,
                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ slots, T* __restrict__ out, int H, int Hkv, int hd,
                       int page_size, float scale, int window) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    float* qs = sm;              // [hd]
    float* sc = sm + hd;         // [ATT_CHUNK]
    int* pg = (int*)(sc + ATT_CHUNK);  // [ATT_CHUNK] page of each key of the chunk
    int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    int pos = tok_pos[t];
    int slot = slots[tok_seq[t]];
    int kvh = h / (H / Hkv);
    int start = (window > 0 && pos >= window) ? pos - window + 1 : 0;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int i = tid; i < hd; i += ATT_CHUNK) qs[i] = to_f32(qrow[i]);
    __syncthreads();
    float m = -CUDART_INF_F, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;  // output dims tid and tid + ATT_CHUNK (hd <= 256)
    const int* pt = page_table + (size_t)slot * pt_stride;
    for (int base = start; base <= pos; base += ATT_CHUNK) {
        int n = min(ATT_CHUNK, pos - base + 1);
        float s = -CUDART_INF_F;
        if (tid < n) {
            int key = base + tid;
            int page = pt[key / page_size];
            pg[tid] = page;
            const T* kr = k_pages + (((size_t)page * Hkv + kvh) * page_size + key % page_size) * hd;
            float d = 0.f;
            for (int i = 0; i < hd; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
            s = d * scale;
        }
        sc[tid] = s;
        __syncthreads();
        float cm = m;
        for (int j = 0; j < n; ++j) cm = fmaxf(cm, sc[j]);
        float corr = expf(m - cm);  // m = -inf at the first chunk gives 0
        __syncthreads();
        if (tid < n) sc[tid] = expf(sc[tid] - cm);
        __syncthreads();
        float ls = 0.f;
        for (int j = 0; j < n; ++j) ls += sc[j];
        l = l * corr + ls;
        for (int rep = 0; rep < 2; ++rep) {
            int d = tid + rep * ATT_CHUNK;
            if (d >= hd) break;
            float a = 0.f;
            for (int j = 0; j < n; ++j) {
                int key = base + j;
                const T* vr = v_pages + (((size_t)pg[j] * Hkv + kvh) * page_size + key % page_size) * hd;
                a = fmaf(sc[j], to_f32(vr[d]), a);
            }
            if (rep == 0) acc0 = acc0 * corr + a; else acc1 = acc1 * corr + a;
        }
        m = cm;
        __syncthreads();
    }
    T* orow = out + ((size_t)t * H + h) * hd;
    if (tid < hd) orow[tid] = from_f32<T>(acc0 / l);
    if (tid + ATT_CHUNK < hd) orow[tid + ATT_CHUNK] = from_f32<T>(acc1 / l);
}

LQ_EXPORT int lq_attention_plain(const void* q, int q_stride, int dtype, const void* k_pages, const void* v_pages,
                                 const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                                 const int* slots, void* out, int T, int H, int Hkv, int hd, int page_size,
                                 float scale, int window, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (hd > 2 * ATT_CHUNK || H % Hkv) return LQ_BAD_SIZE;
    dim3 grid(T, H);
    size_t smem = (hd + 2 * ATT_CHUNK) * sizeof(float);
    if (dtype == LQ_F32)
        return launch_pdl(attention_plain_kernel<float>, grid, dim3(ATT_CHUNK), smem, stream, (const float*)q, q_stride, (const float*)k_pages,
            (const float*)v_pages, page_table, pt_stride, tok_pos, tok_seq, slots, (float*)out, H, Hkv, hd, page_size, scale, window);
    else if (dtype == LQ_BF16)
        return launch_pdl(attention_plain_kernel<__nv_bfloat16>, grid, dim3(ATT_CHUNK), smem, stream, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table, pt_stride, tok_pos, tok_seq, slots,
            (__nv_bfloat16*)out, H, Hkv, hd, page_size, scale, window);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

// ------------------------------------------------------------------ swiglu
// out = up * gate / (1 + e^-gate) from gu [T, 2F].  block == 0: gate in columns
// [0, F), up in [F, 2F).  block == b > 0: columns alternate b gate, b up, b gate, ...
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total, int block) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t t = i / F;
    int f = (int)(i % F);
    int gi = block ? (f / block) * 2 * block + f % block : f;
    int ui = block ? gi + block : F + f;
    float g = to_f32(gu[t * 2 * F + gi]);
    float u = to_f32(gu[t * 2 * F + ui]);
    out[i] = from_f32<T>(u * (g / (1.0f + expf(-g))));
}

LQ_EXPORT int lq_swiglu(const void* gu, void* out, int dtype, int T, int F, int block, cudaStream_t stream) {
    size_t total = (size_t)T * F;
    if (total == 0) return LQ_OK;
    if (block < 0 || (block && F % block)) return LQ_BAD_SIZE;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == LQ_F32)
        return launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, F, total, block);
    else if (dtype == LQ_BF16)
        return launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, F, total, block);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

// ------------------------------------------------------------------ clearing the unwritten end of a page
// A page that a sequence is given may hold what another sequence left there.  Kernels that load whole
// pages multiply the rows beyond the sequence's length by probability zero, which gives zero only for
// finite values; so the rows of a new page that the step will not write are cleared before the step.
// pages [entry][page][kv head][token][head_dim]; work item = (page, first row to clear).
#define LQ_CLEAR_MAX 120
struct ClearList { int page[LQ_CLEAR_MAX]; int first_row[LQ_CLEAR_MAX]; };

__global__ void clear_page_tails_kernel(uint32_t* __restrict__ k_pages, uint32_t* __restrict__ v_pages, ClearList list,
                                        size_t entry_words, size_t page_words, int Hkv, int page_size, int row_words) {
    const int item = blockIdx.x, entry = blockIdx.y, head = blockIdx.z;
    const int first = list.first_row[item];
    const size_t base = (size_t)entry * entry_words + (size_t)list.page[item] * page_words
                      + ((size_t)head * page_size + first) * row_words;
    const int n = (page_size - first) * row_words;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        k_pages[base + i] = 0u;
        v_pages[base + i] = 0u;
    }
}

LQ_EXPORT int lq_clear_page_tails(void* k_pages, void* v_pages, int dtype, const int* pages, const int* first_rows,
                                  int n_items, int n_entries, int n_pages, int Hkv, int page_size, int hd,
                                  cudaStream_t stream) {
    if (n_items <= 0 || n_entries <= 0) return LQ_OK;
    if (dtype != LQ_F32 && dtype != LQ_BF16) return LQ_BAD_DTYPE;
    const int elt = dtype == LQ_F32 ? 4 : 2;
    if ((hd * elt) % 4) return LQ_BAD_SIZE;
    const int row_words = hd * elt / 4;
    const size_t page_words = (size_t)Hkv * page_size * row_words;
    for (int at = 0; at < n_items; at += LQ_CLEAR_MAX) {
        ClearList list;
        const int n = n_items - at < LQ_CLEAR_MAX ? n_items - at : LQ_CLEAR_MAX;
        for (int i = 0; i < n; ++i) {
            if (pages[at + i] < 0 || pages[at + i] >= n_pages || first_rows[at + i] < 0 || first_rows[at + i] > page_size)
                return LQ_BAD_SIZE;
            list.page[i] = pages[at + i];
            list.first_row[i] = first_rows[at + i];
        }
        int rc = launch_after(clear_page_tails_kernel, dim3(n, n_entries, Hkv), dim3(256), 0, stream, (uint32_t*)k_pages,
                              (uint32_t*)v_pages, list, page_words * (size_t)n_pages, page_words, Hkv, page_size, row_words);
        if (rc != LQ_OK) return rc;
    }
    return LQ_OK;
}
