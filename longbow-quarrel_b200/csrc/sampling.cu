// Choosing the next token from a row of logits on the device.
//
// Two kernels make the same decisions.  sample_cluster_kernel is the one that runs: a thread-block cluster
// of eight blocks takes a row, each block holds an eighth of the row's weights in its shared memory, so the
// logits are read from memory once and every later pass (the maximum, the sum, the search for the top-k and
// top-p cut-offs, the draw) runs out of shared memory; the blocks add up their partial results through
// distributed shared memory, in rank order, so a row's result does not depend on the rest of the batch.
// sample_kernel (one block per row, weights in a scratch row in global memory) takes the vocabularies
// that do not fit a cluster's shared memory, and is the twin that the other is tested against.
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


// ------------------------------------------------------------------ a cluster per row
constexpr int CB = 512;              // threads per block of the cluster
// Element i of a block's part lies at word i + i / 32 of its shared memory: a thread that walks its own run of
// consecutive elements (the cut-offs' ties and the draw go in index order) then meets no other lane's bank.
#define AT(i) ((i) + ((i) >> 5))
constexpr int CLUSTER_MAX = 8;       // blocks per row (the largest cluster size that every device offers)

struct ClusterShared {
    // What a block contributes to a sum over the cluster, in two sets used in turn (a block may write its next
    // contribution while a slower one still reads the last).
    double d[2];
    int i[2];
    float f[2];
    int idx[2];
    int hist[2][256];
    double wd[CB / 32];
    int wi[CB / 32];
    float wf[CB / 32];
    int widx[CB / 32];
    double dscan[CB];
    int pick;
    int bcast_i;
    double bcast_d;
};

struct Cluster {
    ClusterShared* sh;
    unsigned rank, size;
    int turn;

    __device__ __forceinline__ void sync() const {
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    // The same variable in the shared memory of block `r` of the cluster.
    template <typename T> __device__ __forceinline__ const T* remote(const T* p, unsigned r) const {
        uint32_t local = (uint32_t)__cvta_generic_to_shared(p), mapped;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(mapped) : "r"(local), "r"(r));
        return reinterpret_cast<const T*>((uintptr_t)mapped);
    }
    __device__ __forceinline__ double ld_d(const double* p, unsigned r) const {
        double v;
        asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"((uint32_t)(uintptr_t)remote(p, r)) : "memory");
        return v;
    }
    __device__ __forceinline__ int ld_i(const int* p, unsigned r) const {
        int v;
        asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"((uint32_t)(uintptr_t)remote(p, r)) : "memory");
        return v;
    }
    __device__ __forceinline__ float ld_f(const float* p, unsigned r) const {
        float v;
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"((uint32_t)(uintptr_t)remote(p, r)) : "memory");
        return v;
    }

    // Sums over all threads of all blocks, the blocks added in rank order; every thread gets the result.
    __device__ double sum_d(double v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) sh->wd[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < CB / 32; ++w) t += sh->wd[w];
            sh->d[turn] = t;
        }
        sync();
        double total = 0.0;
        for (unsigned r = 0; r < size; ++r) total += ld_d(&sh->d[turn], r);
        turn ^= 1;
        return total;
    }
    __device__ int sum_i(int v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) sh->wi[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < CB / 32; ++w) t += sh->wi[w];
            sh->i[turn] = t;
        }
        sync();
        int total = 0;
        for (unsigned r = 0; r < size; ++r) total += ld_i(&sh->i[turn], r);
        turn ^= 1;
        return total;
    }
    __device__ int min_i(int v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
        if ((threadIdx.x & 31) == 0) sh->wi[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = sh->wi[0];
            for (int w = 1; w < CB / 32; ++w) t = min(t, sh->wi[w]);
            sh->i[turn] = t;
        }
        sync();
        int total = ld_i(&sh->i[turn], 0);
        for (unsigned r = 1; r < size; ++r) total = min(total, ld_i(&sh->i[turn], r));
        turn ^= 1;
        return total;
    }
    // Maximum value, lowest index among equals (idx < 0: no candidate).
    __device__ void argmax(float v, int idx, float& out_v, int& out_i) {
        auto better = [](float ov, int oi, float v, int idx) { return oi >= 0 && (idx < 0 || ov > v || (ov == v && oi < idx)); };
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, v, o);
            int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(ov, oi, v, idx)) { v = ov; idx = oi; }
        }
        if ((threadIdx.x & 31) == 0) { sh->wf[threadIdx.x >> 5] = v; sh->widx[threadIdx.x >> 5] = idx; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float bv = sh->wf[0];
            int bi = sh->widx[0];
            for (int w = 1; w < CB / 32; ++w)
                if (better(sh->wf[w], sh->widx[w], bv, bi)) { bv = sh->wf[w]; bi = sh->widx[w]; }
            sh->f[turn] = bv;
            sh->idx[turn] = bi;
        }
        sync();
        out_v = ld_f(&sh->f[turn], 0);
        out_i = ld_i(&sh->idx[turn], 0);
        for (unsigned r = 1; r < size; ++r) {
            float ov = ld_f(&sh->f[turn], r);
            int oi = ld_i(&sh->idx[turn], r);
            if (better(ov, oi, out_v, out_i)) { out_v = ov; out_i = oi; }
        }
        turn ^= 1;
    }
};

// The k-th largest weight of the row (weights are >= 0, so their bit patterns order like the values): the four
// bytes of its bit pattern are found from the top down, each from a count of the weights that share the bytes
// found so far, by the value of their next byte.  Counts are whole numbers: no order of summation matters.
__device__ uint32_t kth_largest_bits(const float* w, int n, int k, Cluster& c) {
    uint32_t prefix = 0u;
    int want = k;                                        // the rank still looked for among the weights that match
    for (int byte = 3; byte >= 0; --byte) {
        int* hist = c.sh->hist[c.turn];
        for (int b = threadIdx.x; b < 256; b += CB) hist[b] = 0;
        __syncthreads();
        const int shift = byte * 8;
        for (int i = threadIdx.x; i < n; i += CB) {
            const float v = w[AT(i)];
            const uint32_t bits = __float_as_uint(v);
            if (v > 0.f && (byte == 3 || (bits >> (shift + 8)) == (prefix >> (shift + 8))))
                atomicAdd(&hist[(bits >> shift) & 255u], 1);
        }
        __syncthreads();
        c.sync();
        // Every block adds the blocks' counts (thread b takes value b of the byte) and walks down from 255.
        if (threadIdx.x < 256) {
            int t = 0;
            for (unsigned r = 0; r < c.size; ++r) t += c.ld_i(&c.sh->hist[c.turn][threadIdx.x], r);
            c.sh->dscan[threadIdx.x] = (double)t;        // whole numbers far below 2^53
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int above = 0, digit = 0;
            for (int b = 255; b >= 0; --b) {
                const int here = (int)c.sh->dscan[b];
                if (above + here >= want) { digit = b; break; }
                above += here;
            }
            c.sh->bcast_i = digit;
            c.sh->bcast_d = (double)above;
        }
        __syncthreads();
        prefix |= (uint32_t)c.sh->bcast_i << shift;
        want -= (int)c.sh->bcast_d;
        c.turn ^= 1;
        __syncthreads();
    }
    return prefix;
}

// Drop every weight of this block's part below `cut`; of the weights equal to `cut` keep the first n_eq of the
// whole row in index order.
__device__ void cluster_apply_cut(float* w, int n, float cut, int n_eq, Cluster& c) {
    const int chunk = (n + CB - 1) / CB;
    const int lo = threadIdx.x * chunk, hi = min(n, lo + chunk);
    int mine = 0;
    for (int i = lo; i < hi; ++i) mine += (w[AT(i)] == cut) ? 1 : 0;
    c.sh->dscan[threadIdx.x] = (double)mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int t = 0; t < CB; ++t) { int x = (int)c.sh->dscan[t]; c.sh->dscan[t] = (double)run; run += x; }
        c.sh->i[c.turn] = run;                           // equals in this block's part
    }
    __syncthreads();
    c.sync();
    int before = (int)c.sh->dscan[threadIdx.x];
    for (unsigned r = 0; r < c.rank; ++r) before += c.ld_i(&c.sh->i[c.turn], r);     // equals in the parts before this one
    c.turn ^= 1;
    for (int i = lo; i < hi; ++i) {
        const float v = w[AT(i)];
        if (v < cut) w[AT(i)] = 0.f;
        else if (v == cut) { if (before >= n_eq) w[AT(i)] = 0.f; ++before; }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(CB)
sample_cluster_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, int part, float temperature,
                      int top_k, float top_p, float penalty, const int* __restrict__ history, int hist_stride,
                      const int* __restrict__ hist_len, unsigned long long seed, const int* __restrict__ rng_sequence,
                      const int* __restrict__ rng_step, int step_offset) {
    extern __shared__ __align__(16) float w[];           // this block's part of the row
    __shared__ ClusterShared sh;
    Cluster c;
    c.sh = &sh;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(c.rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(c.size));
    c.turn = 0;
    const int row = blockIdx.x / c.size, tid = threadIdx.x;
    const int base = c.rank * part;
    const int n = max(0, min(part, V - base));
    const float* z_in = logits + (size_t)row * V + base;

    // 1. any value that is not finite -> first finite index.
    int bad = 0, first_ok = V;
    if ((((size_t)row * V + base) & 3) == 0) {
        // Four logits a load: enough bytes on their way for the one pass over memory that the kernel makes.
        const float4* z4 = reinterpret_cast<const float4*>(z_in);
        for (int q = tid; q < n / 4; q += CB) {
            const float4 v4 = __ldg(z4 + q);
            const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = 4 * q + e;
                if (isfinite(v[e])) first_ok = min(first_ok, base + i); else bad = 1;
                w[AT(i)] = v[e];
            }
        }
        for (int i = n / 4 * 4 + tid; i < n; i += CB) {
            const float v = z_in[i];
            if (isfinite(v)) first_ok = min(first_ok, base + i); else bad = 1;
            w[AT(i)] = v;
        }
    } else {
        for (int i = tid; i < n; i += CB) {
            const float v = z_in[i];
            if (isfinite(v)) first_ok = min(first_ok, base + i); else bad = 1;
            w[AT(i)] = v;
        }
    }
    __syncthreads();
    bad = c.sum_i(bad);
    if (bad) {
        first_ok = c.min_i(first_ok);
        if (c.rank == 0 && tid == 0) out[row] = first_ok < V ? first_ok : 0;
        c.sync();                                        // no block leaves while another still reads its shared memory
        return;
    }
    // 2. repetition penalty over the distinct ids of the history (each block changes the ids of its part).
    if (penalty > 1.0f && history != nullptr) {
        const int* h = history + (size_t)row * hist_stride;
        const int hn = hist_len[row];
        if (tid < hn) {
            const int id = h[tid];
            bool first = id >= base && id < base + n;
            for (int j = 0; j < tid && first; ++j) first = h[j] != id;
            if (first) {
                const float v = w[AT(id - base)];
                w[AT(id - base)] = v > 0.f ? v / penalty : v * penalty;
            }
        }
        __syncthreads();
    }
    // 3. greedy.
    float best = -CUDART_INF_F;
    int best_i = -1;
    for (int i = tid; i < n; i += CB) {
        const float v = w[AT(i)];
        if (best_i < 0 || v > best) { best = v; best_i = base + i; }
    }
    float zmax;
    int imax;
    c.argmax(best, best_i, zmax, imax);
    if (temperature == 0.f) {
        if (c.rank == 0 && tid == 0) out[row] = imax;
        c.sync();
        return;
    }
    // 4. weights e^((z - max) / T) and their sum; 5. drop p <= 1e-10.
    double partial = 0.0;
    const float inv_t = 1.0f / temperature;
    for (int i = tid; i < n; i += CB) {
        const float e = expf((w[AT(i)] - zmax) * inv_t);
        w[AT(i)] = e;
        partial += (double)e;
    }
    const double total = c.sum_d(partial);
    const float floor_w = (float)(1e-10 * total);
    int kept = 0;
    for (int i = tid; i < n; i += CB) {
        if (w[AT(i)] <= floor_w) w[AT(i)] = 0.f; else ++kept;
    }
    __syncthreads();
    kept = c.sum_i(kept);
    if (kept == 0) {  // cannot happen for finite logits (the maximum has weight 1); mirrors the fallback
        if (c.rank == 0 && tid == 0) out[row] = imax;
        c.sync();
        return;
    }
    // 6. top-k: the k-th largest weight, byte by byte.
    if (top_k > 0 && top_k < kept) {
        const uint32_t cut_bits = kth_largest_bits(w, n, top_k, c);
        int above = 0;
        for (int i = tid; i < n; i += CB) above += (__float_as_uint(w[AT(i)]) > cut_bits) ? 1 : 0;
        above = c.sum_i(above);
        cluster_apply_cut(w, n, __uint_as_float(cut_bits), top_k - above, c);
    }
    // 7. top-p: the weight at which the falling cumulative sum reaches top_p, by bisection on the bit pattern
    // (sums of doubles in a fixed order: the same cut-off in every run).
    if (top_p > 0.f && top_p < 1.f) {
        const double need = (double)top_p * total;
        auto mass_ge = [&](uint32_t bits) {
            double m = 0.0;
            for (int i = tid; i < n; i += CB) m += (__float_as_uint(w[AT(i)]) >= bits) ? (double)w[AT(i)] : 0.0;
            return c.sum_d(m);
        };
        if (mass_ge(1u) >= need) {
            uint32_t lo = 1u, hi = 0x3f800001u;          // mass_ge(lo) >= need > mass_ge(hi); no weight exceeds 1
            while (hi - lo > 1u) {
                const uint32_t mid = lo + (hi - lo) / 2u;
                if (mass_ge(mid) >= need) lo = mid; else hi = mid;
            }
            const float cut = __uint_as_float(lo);
            const double above = mass_ge(lo + 1u);
            const int n_eq = (int)ceil((need - above) / (double)cut);
            cluster_apply_cut(w, n, cut, max(n_eq, 1), c);
        }
    }
    // 8. draw in index order: the parts in rank order, inside a part each thread's run of weights.
    const int chunk = (n + CB - 1) / CB;
    const int lo_i = tid * chunk, hi_i = min(n, lo_i + chunk);
    double mine = 0.0;
    for (int i = lo_i; i < hi_i; ++i) mine += (double)w[AT(i)];
    sh.dscan[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        double run = 0.0;
        for (int t = 0; t < CB; ++t) { const double x = sh.dscan[t]; sh.dscan[t] = run; run += x; }
        sh.d[c.turn] = run;                              // weight of this block's part
        sh.pick = -1;
    }
    __syncthreads();
    c.sync();
    double before = 0.0, all = 0.0;
    for (unsigned r = 0; r < c.size; ++r) {
        const double x = c.ld_d(&sh.d[c.turn], r);
        if (r < c.rank) before += x;
        all += x;
    }
    c.turn ^= 1;
    const double u = philox_uniform(seed, (uint32_t)rng_sequence[row], (uint32_t)(rng_step[row] + step_offset));
    const double r = u * all;
    const double start = before + sh.dscan[tid];
    if (mine > 0.0 && r >= start && r < start + mine) {
        double acc = start;
        int pick = -1;
        for (int i = lo_i; i < hi_i; ++i) {
            const float v = w[AT(i)];
            if (v > 0.f) {
                acc += (double)v;
                pick = base + i;
                if (r < acc) break;
            }
        }
        sh.pick = pick;
    }
    __syncthreads();
    c.sync();
    if (c.rank == 0 && tid == 0) {
        int pick = -1;
        for (unsigned q = 0; q < c.size && pick < 0; ++q) pick = c.ld_i(&sh.pick, q);
        out[row] = pick >= 0 ? pick : imax;              // r fell on a rounding gap: the most probable token is always kept
    }
    c.sync();
}

}  // namespace

namespace {
int cluster_size(int V) { return V >= 2048 ? CLUSTER_MAX : 1; }
int cluster_part(int V) { const int size = cluster_size(V); return ((V + size - 1) / size + 3) / 4 * 4; }
// Whether a row of V logits fits the shared memory of a cluster (set up on first use).
bool fits_cluster(int V) {
    static int smem_limit = -1;
    if (smem_limit < 0) {
        int dev = 0, optin = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        smem_limit = optin - (int)sizeof(ClusterShared) - 1024;
        if (smem_limit > 0 &&
            cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_limit) != cudaSuccess) {
            (void)cudaGetLastError();
            smem_limit = 0;
        }
    }
    return (long)(cluster_part(V) + cluster_part(V) / 32 + 1) * (long)sizeof(float) <= (long)smem_limit;
}
}  // namespace

// Whether lq_sample needs a scratch row per row of logits for this vocabulary (1) or not (0).
LQ_EXPORT int lq_sample_needs_scratch(int V) { return V > 0 && fits_cluster(V) ? 0 : 1; }

// One block per row with the weights in `scratch` serves rows too long for a cluster's shared memory
// (lq_sample_one_block asks for that kernel whatever the size, for comparing the two).
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
    if (hist_stride > SB || hist_stride > CB) return LQ_BAD_SIZE;
    // A cluster per row where the row fits the cluster's shared memory (scratch null asks for that path only).
    const int size = cluster_size(V);
    const int part = cluster_part(V);
    const size_t smem = (size_t)(part + part / 32 + 1) * sizeof(float);
    if (fits_cluster(V)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)rows * size);
        cfg.blockDim = dim3(CB);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = size;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, out, V, part, temperature, top_k, top_p, penalty,
                                           history, hist_stride, hist_len, seed, rng_sequence, rng_step, step_offset);
        return e == cudaSuccess ? LQ_OK : (int)e;
    }
    if (!scratch) return LQ_BAD_SIZE;
    sample_kernel<<<rows, SB, 0, stream>>>(logits, scratch, out, V, temperature, top_k, top_p, penalty, history,
                                           hist_stride, hist_len, seed, rng_sequence, rng_step, step_offset);
    return lq_launch_status();
}

LQ_EXPORT int lq_sample_one_block(const float* logits, float* scratch, int* out, int rows, int V, float temperature,
                                  int top_k, float top_p, float penalty, const int* history, int hist_stride,
                                  const int* hist_len, unsigned long long seed, const int* rng_sequence,
                                  const int* rng_step, int step_offset, cudaStream_t stream) {
    if (rows <= 0) return LQ_OK;
    if (V <= 0 || temperature < 0.f || !scratch || hist_stride > SB) return LQ_BAD_SIZE;
    if (temperature > 0.f && (!rng_sequence || !rng_step)) return LQ_BAD_SIZE;
    sample_kernel<<<rows, SB, 0, stream>>>(logits, scratch, out, V, temperature, top_k, top_p, penalty, history,
                                           hist_stride, hist_len, seed, rng_sequence, rng_step, step_offset);
    return lq_launch_status();
}
