// Choosing the next token from a row of logits, one block per row, on the device.
//
// The decisions are those of the reference's sampler (internal/engine/sampler.go:72-105):
//   1. any NaN or Inf among the logits -> the first finite index (:73-75,116-123);
//   2. repetition penalty > 1: each distinct id among the last tokens of the history has
//      its logit divided by the penalty if positive, multiplied if negative (:249-275);
//   3. temperature 0 -> the first maximum (:282-307);
//   4. p = softmax(logits / T) with the maximum subtracted (:125-156);
//   5. p <= 1e-10 is dropped (:158-166);
//   6. top-k keeps the k most probable (:309-314);
//   7. top-p keeps the most probable until their sum reaches p (:316-339);
//   8. a uniform draw scaled by the kept sum picks the token whose cumulative range
//      holds it (:168-184).
// The reference sorts the candidates and draws with Go's math/rand.  Here nothing is
// sorted: the k-th largest probability and the top-p cut-off are found by bisection on
// the bit pattern of the probabilities, equal values at a cut-off are kept in index
// order, the cumulative walk runs in index order, and the uniform number comes from
// Philox4x32-10 keyed by the seed and counted by (sequence, step), so a sequence's
// draws do not depend on what else is in the batch.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int SB = 1024;  // threads per row

// ------------------------------------------------------------------ Philox4x32-10
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}
// A uniform double in [0, 1) from (seed, sequence, step).
__device__ double philox_uniform(unsigned long long seed, uint32_t sequence, uint32_t step) {
    uint32_t c[4] = {sequence, step, 0u, 0u};
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    unsigned long long bits = ((unsigned long long)(c[0] >> 5) << 26) | (unsigned long long)(c[1] >> 6);
    return (double)bits * (1.0 / 9007199254740992.0);
}

// ------------------------------------------------------------------ block reductions (fixed order)
struct Shared {
    double d[SB / 32];
    float f[SB / 32];
    int i[SB / 32];
    int idx[SB / 32];
    double bd;
    float bf;
    int bi;
    int bidx;
    int scan[SB];
    double dscan[SB];
};

__device__ double block_sum_d(double v, Shared& sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh.d[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < SB / 32; ++w) t += sh.d[w];
        sh.bd = t;
    }
    __syncthreads();
    return sh.bd;
}
__device__ int block_sum_i(int v, Shared& sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh.i[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < SB / 32; ++w) t += sh.i[w];
        sh.bi = t;
    }
    __syncthreads();
    return sh.bi;
}
// Maximum value, lowest index among equals; NaN never wins.
__device__ void block_argmax(float v, int idx, Shared& sh, float& out_v, int& out_i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi >= 0 && (idx < 0 || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { sh.f[threadIdx.x >> 5] = v; sh.idx[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float bv = sh.f[0];
        int bi = sh.idx[0];
        for (int w = 1; w < SB / 32; ++w) {
            float ov = sh.f[w];
            int oi = sh.idx[w];
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        sh.bf = bv;
        sh.bidx = bi;
    }
    __syncthreads();
    out_v = sh.bf;
    out_i = sh.bidx;
}

// Count of weights >= the value with bit pattern `bits` (weights are >= 0, so their
// bit patterns order like the values).
__device__ int count_ge(const float* w, int V, uint32_t bits, Shared& sh) {
    int c = 0;
    for (int i = threadIdx.x; i < V; i += SB) c += (__float_as_uint(w[i]) >= bits && w[i] > 0.f) ? 1 : 0;
    return block_sum_i(c, sh);
}
__device__ double mass_ge(const float* w, int V, uint32_t bits, Shared& sh) {
    double m = 0.0;
    for (int i = threadIdx.x; i < V; i += SB) m += (__float_as_uint(w[i]) >= bits) ? (double)w[i] : 0.0;
    return block_sum_d(m, sh);
}

// Drop every weight below `cut`; of the weights equal to `cut` keep the first n_eq in index order.
__device__ void apply_cut(float* w, int V, float cut, int n_eq, Shared& sh) {
    const int chunk = (V + SB - 1) / SB;
    const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
    int mine = 0;
    for (int i = lo; i < hi; ++i) mine += (w[i] == cut) ? 1 : 0;
    __syncthreads();
    sh.scan[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int t = 0; t < SB; ++t) { int c = sh.scan[t]; sh.scan[t] = run; run += c; }
    }
    __syncthreads();
    int before = sh.scan[threadIdx.x];
    for (int i = lo; i < hi; ++i) {
        float v = w[i];
        if (v < cut) w[i] = 0.f;
        else if (v == cut) { if (before >= n_eq) w[i] = 0.f; ++before; }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(SB)
sample_kernel(const float* __restrict__ logits, float* __restrict__ scratch, int* __restrict__ out, int V,
              float temperature, int top_k, float top_p, float penalty, const int* __restrict__ history,
              int hist_stride, const int* __restrict__ hist_len, unsigned long long seed,
              const int* __restrict__ rng_sequence, const int* __restrict__ rng_step, int step_offset) {
    __shared__ Shared sh;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* z_in = logits + (size_t)row * V;
    float* w = scratch + (size_t)row * V;

    // 1. any value that is not finite -> first finite index.
    int bad = 0, first_ok = V;
    for (int i = tid; i < V; i += SB) {
        float v = z_in[i];
        if (isfinite(v)) first_ok = min(first_ok, i); else bad = 1;
        w[i] = v;
    }
    bad = block_sum_i(bad, sh);
    if (bad) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) first_ok = min(first_ok, __shfl_xor_sync(0xffffffffu, first_ok, o));
        __syncthreads();
        if ((tid & 31) == 0) sh.i[tid >> 5] = first_ok;
        __syncthreads();
        if (tid == 0) {
            int f = V;
            for (int k = 0; k < SB / 32; ++k) f = min(f, sh.i[k]);
            out[row] = f < V ? f : 0;
        }
        return;
    }
    // 2. repetition penalty over the distinct ids of the history.
    if (penalty > 1.0f && history != nullptr) {
        const int* h = history + (size_t)row * hist_stride;
        int n = hist_len[row];
        __syncthreads();
        if (tid < n) {
            int id = h[tid];
            bool first = id >= 0 && id < V;
            for (int j = 0; j < tid && first; ++j) first = h[j] != id;
            if (first) {
                float v = w[id];
                w[id] = v > 0.f ? v / penalty : v * penalty;
            }
        }
        __syncthreads();
    }
    // 3. greedy.
    float best = -CUDART_INF_F;
    int best_i = -1;
    for (int i = tid; i < V; i += SB) {
        float v = w[i];
        if (best_i < 0 || v > best) { best = v; best_i = i; }
    }
    float zmax;
    int imax;
    block_argmax(best, best_i, sh, zmax, imax);
    if (temperature == 0.f) {
        if (tid == 0) out[row] = imax;
        return;
    }
    // 4. weights e^((z - max) / T) and their sum; 5. drop p <= 1e-10.
    double part = 0.0;
    const float inv_t = 1.0f / temperature;
    for (int i = tid; i < V; i += SB) {
        float e = expf((w[i] - zmax) * inv_t);
        w[i] = e;
        part += (double)e;
    }
    const double total = block_sum_d(part, sh);
    const float floor_w = (float)(1e-10 * total);
    int kept = 0;
    for (int i = tid; i < V; i += SB) {
        if (w[i] <= floor_w) w[i] = 0.f; else ++kept;
    }
    kept = block_sum_i(kept, sh);
    if (kept == 0) {  // cannot happen for finite logits (the maximum has weight 1); mirrors the fallback
        if (tid == 0) out[row] = imax;
        return;
    }
    // 6. top-k: the k-th largest weight by bisection on the bit pattern.
    if (top_k > 0 && top_k < kept) {
        uint32_t lo = 0u, hi = 0x7f800000u;   // count_ge(lo) >= k > count_ge(hi)
        while (hi - lo > 1u) {
            uint32_t mid = lo + (hi - lo) / 2u;
            if (count_ge(w, V, mid, sh) >= top_k) lo = mid; else hi = mid;
        }
        float cut = __uint_as_float(lo);
        int above = count_ge(w, V, lo + 1u, sh);
        apply_cut(w, V, cut, top_k - above, sh);
    }
    // 7. top-p: the weight at which the falling cumulative sum reaches top_p.
    if (top_p > 0.f && top_p < 1.f) {
        const double need = (double)top_p * total;
        if (mass_ge(w, V, 1u, sh) >= need) {
            uint32_t lo = 1u, hi = 0x7f800000u;   // mass_ge(lo) >= need > mass_ge(hi)
            while (hi - lo > 1u) {
                uint32_t mid = lo + (hi - lo) / 2u;
                if (mass_ge(w, V, mid, sh) >= need) lo = mid; else hi = mid;
            }
            float cut = __uint_as_float(lo);
            double above = mass_ge(w, V, lo + 1u, sh);
            int n_eq = (int)ceil((need - above) / (double)cut);
            apply_cut(w, V, cut, max(n_eq, 1), sh);
        }
    }
    // 8. draw in index order.
    const int chunk = (V + SB - 1) / SB;
    const int lo_i = tid * chunk, hi_i = min(V, lo_i + chunk);
    double mine = 0.0;
    for (int i = lo_i; i < hi_i; ++i) mine += (double)w[i];
    __syncthreads();
    sh.dscan[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        double run = 0.0;
        for (int t = 0; t < SB; ++t) { double c = sh.dscan[t]; sh.dscan[t] = run; run += c; }
        double u = philox_uniform(seed, (uint32_t)rng_sequence[row], (uint32_t)(rng_step[row] + step_offset));
        sh.bd = u * run;
        sh.bi = -1;
        // The chunk whose range holds r: the last one whose start is <= r and that has weight.
        sh.bidx = 0;
    }
    __syncthreads();
    const double r = sh.bd;
    const double start = sh.dscan[tid];
    if (mine > 0.0 && r >= start && r < start + mine) {
        double acc = start;
        int pick = -1;
        for (int i = lo_i; i < hi_i; ++i) {
            float v = w[i];
            if (v > 0.f) {
                acc += (double)v;
                pick = i;
                if (r < acc) break;
            }
        }
        sh.bi = pick;
    }
    __syncthreads();
    if (tid == 0) {
        int pick = sh.bi;
        if (pick < 0) pick = imax;   // r fell on a rounding gap: the most probable token is always kept
        out[row] = pick;
    }
}

}  // namespace

// logits [rows, V] float32; scratch [rows, V] float32 (overwritten); out [rows] int32.
// history [rows, hist_stride] with hist_len[rows] valid ids each (null: no penalty).
// rng_sequence / rng_step [rows]: the counter of each row's draw (unused for temperature 0); step_offset is added
// to every row's step, so a caller whose rows all advance together keeps one array and passes the step here.
LQ_EXPORT int lq_sample(const float* logits, float* scratch, int* out, int rows, int V, float temperature, int top_k,
                        float top_p, float penalty, const int* history, int hist_stride, const int* hist_len,
                        unsigned long long seed, const int* rng_sequence, const int* rng_step, int step_offset,
                        cudaStream_t stream) {
    if (rows <= 0) return LQ_OK;
    if (V <= 0 || temperature < 0.f) return LQ_BAD_SIZE;
    if (temperature > 0.f && (!rng_sequence || !rng_step)) return LQ_BAD_SIZE;
    if (hist_stride > SB) return LQ_BAD_SIZE;
    sample_kernel<<<rows, SB, 0, stream>>>(logits, scratch, out, V, temperature, top_k, top_p, penalty, history,
                                           hist_stride, hist_len, seed, rng_sequence, rng_step, step_offset);
    return lq_launch_status();
}
