// y = x . W^T on the fifth-generation tensor cores (tcgen05) for many rows of x
// (prefill): bfloat16 operands, float32 accumulation in tensor memory.
//
// One persistent block per SM walks over 128 x BN output tiles.  Inside a block
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor) of the x tile [128, 64] and
//               the W tile [BN, 64] into a ring of shared-memory stages (128-byte swizzle);
//   warp 1      one lane issues tcgen05.mma (M 128, N BN, K 16; four per stage) into one of
//               two accumulators in tensor memory, and frees a stage with tcgen05.commit;
//   warps 2..5  read a finished accumulator with tcgen05.ld (each thread one row) and store
//               it, while the next tile's products already run into the other accumulator; with
//               many rows the stores go through shared memory and leave as TMA stores of whole
//               lines (for the residual as TMA adds into it).
// Stages and accumulators are handed over through mbarriers.  Every wait is bounded: after
// about two seconds a role records a code in the status word, leaves its loop, and the
// block still waits (bounded) for its copies in flight, frees its tensor memory and ends.
//
// Epilogues: bfloat16 store; float32 store; float32 residual add in place; SwiGLU over
// weight rows interleaved in blocks of 8 (8 gate rows, then their 8 up rows); q/k/v (head sizes 64
// and 128): q and k rotated by the cos/sin tables at each row's position, q stored, k and v written
// into the row's cache page -- no rotation kernel and no buffer of unrotated q/k/v in between.
//
// Few rows and a narrow weight give fewer tiles than SMs, and the product is then bound by
// reading W: the contraction is cut into `splits` ranges, a block's piece of work is (tile, range),
// the pieces' float32 results go to scratch memory and a second kernel adds them in the order of K
// and applies the epilogue.  With W as the N side, one tcgen05.mma consumes 8 KB of W.
//
// Reference counterpart: the per-row linear_f16 kernels and the library GEMM of
// internal/device/metal.go:886-964; its CUDA path calls cublasSgemmEx (internal/device/cuda.go:293-318).
#include "gemm_tc_epilogue.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int UMMA_K = 16;
constexpr int N_THREADS = 192;
using namespace tc;       // mbarriers with bounded waits, TMA, tcgen05 wrappers, descriptors, status word

// AROWS: rows of x that a stage holds, 128 or (for at most 64 rows of x) 64.  With 64 the products still
// read 128 rows: the upper 64 are whatever follows in shared memory, and give rows of the accumulator
// that are never stored -- the stage is 8 KB smaller, so more stages of W are on their way.
// STAGED: the epilogue warps have two buffers of 32 rows x 128 bytes each, from which their stores go out as
// whole lines (TMA); without them a thread stores its own row, 16 bytes at a time.
template <int BN, int STAGES, int AROWS, bool STAGED>
struct Smem {
    alignas(1024) uint8_t a[STAGES][AROWS * BK * 2];
    alignas(1024) uint8_t b[STAGES][BN * BK * 2];
    alignas(1024) uint8_t stage[STAGED ? (AROWS == BM ? 4 : 2) : 1][STAGED ? 2 * STAGE_BUF_BYTES : 16];
    alignas(8) uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
};

// ------------------------------------------------------------------ epilogue of 32 columns of one row
// n_lim: the tile's columns end there (at most N); columns from n_lim on are not stored.
// pre (EPI_RESID, or null): the residual of these 32 columns, loaded beforehand (only asked for whole chunks
// of a matrix whose rows are 16-byte aligned, the case in which this function would load float4s itself).
template <int EPI>
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], void* Cout,
                                            const float* residual, int m, int n, int M, int N, int n_lim,
                                            const float4* pre = nullptr) {
    if (m >= M || n >= n_lim) return;
    if (EPI == EPI_SWIGLU) {
        // 32 columns = [8 gate, 8 up, 8 gate, 8 up] -> 16 outputs at column n / 2 of [M, N / 2].
        const int NO = N >> 1, no = n >> 1, no_lim = n_lim >> 1;
        float o[16];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float g = __uint_as_float(r[h * 16 + i]), u = __uint_as_float(r[h * 16 + 8 + i]);
                o[h * 8 + i] = u * (g / (1.0f + __expf(-g)));
            }
        __nv_bfloat16* dst = (__nv_bfloat16*)Cout + (size_t)m * NO + no;
        if (no + 16 <= no_lim && (NO & 7) == 0) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
            d4[0] = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
            d4[1] = make_uint4(pack2(o[8], o[9]), pack2(o[10], o[11]), pack2(o[12], o[13]), pack2(o[14], o[15]));
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (no + i < no_lim) dst[i] = __float2bfloat16_rn(o[i]);
        }
        return;
    }
    const bool whole = n + 32 <= n_lim;
    if (EPI == EPI_BF16) {
        __nv_bfloat16* dst = (__nv_bfloat16*)Cout + (size_t)m * N + n;
        if (whole && (N & 7) == 0) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                d4[i] = make_uint4(pack2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                                   pack2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                                   pack2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                                   pack2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (n + i < n_lim) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
        }
    } else {
        float* dst = (float*)Cout + (size_t)m * N + n;
        const float* res = (EPI == EPI_RESID) ? residual + (size_t)m * N + n : nullptr;
        if (whole && (N & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                       __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                if (EPI == EPI_RESID) {
                    float4 q = pre ? pre[i] : reinterpret_cast<const float4*>(res)[i];
                    v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
                }
                reinterpret_cast<float4*>(dst)[i] = v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (n + i < n_lim) dst[i] = __uint_as_float(r[i]) + (EPI == EPI_RESID ? res[i] : 0.f);
        }
    }
}

// ------------------------------------------------------------------ the kernel
// Whether the epilogue of a kernel with these parameters can go through shared memory and TMA stores:
// tiles of 128 or 256 columns and not the q/k/v epilogue, whose rows go to cache pages of their own; with
// 64-row stages (at most 64 rows of x) only the float32 store of 256-column tiles, which the ranges of K use.
template <int BN, int EPI, int AROWS> struct StagedEpilogue {
    static constexpr bool value = (AROWS == BM && (BN == 128 || BN == 256) && EPI != EPI_QKV) ||
                                  (AROWS == 64 && BN == 256 && EPI == EPI_F32);
};

template <int BN, int STAGES, int EPI, int AROWS>
__global__ void __launch_bounds__(N_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, int staged, void* Cout, const float* residual, int M, int N, int K, int splits,
               int plane_rows, const QkvArgs qkv) {
    extern __shared__ uint8_t smem_raw[];
    constexpr bool STAGED = StagedEpilogue<BN, EPI, AROWS>::value;
    using S = Smem<BN, STAGES, AROWS, STAGED>;
    S& sm = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    // A piece of work is (tile, range of K): piece = tile * splits + range.  With splits > 1 the kernel
    // is the float32-store one and Cout the scratch [splits, plane_rows, N] (plane_rows: M rounded up to 32, so
    // that a warp's box of 32 rows stays inside its range's plane).
    const int total = m_tiles * n_tiles * splits;
    const int n_kb = (K + BK - 1) / BK;
    constexpr uint32_t STAGE_BYTES = (AROWS + BN) * BK * 2;
    constexpr uint32_t ACC_COLS = BN <= 128 ? 128 : 256;   // columns of tensor memory per accumulator (BN of them used)
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sm.full[s]), 1); mbar_init(smem_u32(&sm.empty[s]), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&sm.acc_full[a]), 1); mbar_init(smem_u32(&sm.acc_empty[a]), 4); }
        mbar_fence_init();
        prefetch_map(&map_a);
        prefetch_map(&map_b);
        if (STAGED && staged) prefetch_map(&map_c);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sm.tmem_base), TMEM_COLS);
    }
    pdl_launch_dependents();
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = sm.tmem_base;
    pdl_wait();     // barriers and tensor memory were set up while the kernel ahead was draining

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int piece = blockIdx.x; piece < total && ok; piece += gridDim.x) {
                const int tile = piece / splits, range = piece % splits;
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                const int kb_lo = (int)((long)n_kb * range / splits), kb_hi = (int)((long)n_kb * (range + 1) / splits);
                for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&sm.empty[s]), ((it / STAGES) & 1) ^ 1)) { give_up(1); ok = false; break; }
                    const uint32_t full = smem_u32(&sm.full[s]);
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(smem_u32(sm.a[s]), &map_a, kb * BK, m0, full);
                    tma_load_2d(smem_u32(sm.b[s]), &map_b, kb * BK, n0, full);
                }
            }
            if (!ok) {
                // Copies that were started must land before the block's shared memory goes away.
                for (uint32_t back = 1; back <= (uint32_t)STAGES && back <= it; ++back) {
                    uint32_t j = it - back;
                    mbar_wait(smem_u32(&sm.full[j % STAGES]), (j / STAGES) & 1);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(BM, BN, false);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int piece = blockIdx.x; piece < total && ok; piece += gridDim.x, ++t) {
                const int range = piece % splits;
                const int kb_lo = (int)((long)n_kb * range / splits), kb_hi = (int)((long)n_kb * (range + 1) / splits);
                const uint32_t acc = t & 1;
                if (!mbar_wait(smem_u32(&sm.acc_empty[acc]), ((t >> 1) & 1) ^ 1)) { give_up(2); ok = false; break; }
                fence_after();
                const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
                for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&sm.full[s]), (it / STAGES) & 1)) { give_up(3); ok = false; break; }
                    fence_after();
                    const uint64_t da = desc_k_major(smem_u32(sm.a[s])), db = desc_k_major(smem_u32(sm.b[s]));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)   // 32 bytes further along K: 2 units of 16 bytes
                        mma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
                    commit(smem_u32(&sm.empty[s]));      // the stage is free once these products have read it
                }
                if (ok) commit(smem_u32(&sm.acc_full[acc]));
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        const int quarter = warp & 3;                     // the 32 lanes of tensor memory this warp may read
        uint32_t t = 0;
        int stage_buf = 0;
        bool ok = true;
        for (int piece = blockIdx.x; piece < total && ok; piece += gridDim.x, ++t) {
            const int tile = piece / splits, range = piece % splits;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            void* dst = splits > 1 ? (void*)((float*)Cout + (size_t)range * plane_rows * N) : Cout;
            const uint32_t acc = t & 1;
            const int m = m0 + quarter * 32 + lane;
            const int n_lim = n0 + BN < N ? n0 + BN : N;
            // The residual that the tile is added to is known before the products are done: its first 32 columns
            // are requested now and each further chunk while the one before it is added and stored.
            float4 pre[8];
            auto fetch = [&](int c) -> bool {
                if constexpr (EPI == EPI_RESID) {
                    const int n = n0 + c * 32;
                    if (m >= M || n + 32 > n_lim || (N & 3)) return false;
#pragma unroll
                    for (int i = 0; i < 8; ++i) pre[i] = reinterpret_cast<const float4*>(residual + (size_t)m * N + n)[i];
                    return true;
                } else {
                    return false;
                }
            };
            bool fetched = !(STAGED && staged) && fetch(0);
            if (!mbar_wait(smem_u32(&sm.acc_full[acc]), (t >> 1) & 1)) { give_up(4); ok = false; break; }
            fence_after();
            const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if (EPI == EPI_QKV) {
                qkv_epilogue(taddr, BN, qkv, (__nv_bfloat16*)Cout, m, M, n0, N);
            } else if (STAGED && staged) {
                if constexpr (STAGED) {
                    if (m0 + quarter * 32 < M)          // (with 64-row stages only the first two warps hold rows of x)
                        staged_epilogue<EPI>(taddr, BN, sm.stage[quarter], stage_buf, &map_c,
                                             (splits > 1 ? range * plane_rows : 0) + m0 + quarter * 32, n0, N, lane);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < (BN + 31) / 32; ++c) {      // a last half chunk reads columns that are not stored
                    uint32_t r[32];
                    ld32(taddr + c * 32, r);
                    wait_ld();
                    if (EPI == EPI_RESID) {
                        float4 now[8];
                        const bool have = fetched;
#pragma unroll
                        for (int i = 0; i < 8; ++i) now[i] = pre[i];
                        fetched = c + 1 < (BN + 31) / 32 && fetch(c + 1);
                        store_chunk<EPI>(r, dst, residual, m, n0 + c * 32, M, N, n_lim, have ? now : nullptr);
                    } else {
                        store_chunk<EPI>(r, dst, residual, m, n0 + c * 32, M, N, n_lim);
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.acc_empty[acc]));
        }
        if (STAGED && staged && lane == 0) bulk_wait<0>();      // this warp's stores are done before the block ends
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ adding the ranges of K
// part [splits, M, N] float32 -> the epilogue of their sum, the ranges added in their order.
// One thread makes four neighbouring outputs.
template <int EPI>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int splits, int plane_rows, void* Cout,
                                                            const float* residual, int M, int N, const QkvArgs qkv) {
    pdl_launch_dependents();
    pdl_wait();
    const int NO = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? N >> 1 : N;    // output columns (for q/k/v: pairs)
    const int groups = (NO + 3) >> 2;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)M * groups) return;
    const int m = (int)(idx / groups), c = (int)(idx % groups) * 4;
    const size_t plane = (size_t)plane_rows * N;
    auto sum4 = [&](int col, float (&v)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = 0.f;
        const float* p = part + (size_t)m * N + col;
        if (col + 4 <= N && (N & 3) == 0) {
            for (int s = 0; s < splits; ++s) {
                float4 q = __ldcg(reinterpret_cast<const float4*>(p + s * plane));
                v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
            }
        } else {
            for (int s = 0; s < splits; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (col + i < N) v[i] += __ldcg(p + s * plane + i);
        }
    };
    float v[4];
    if (EPI == EPI_QKV) {
        // pairs c..c+3 of one head: elements j..j+3 of its first half and their partners in the second half
        const int hd = qkv.hd, half = hd >> 1;
        const int head = c / half, j = c % half;
        float u[4];
        sum4(head * hd + j, v);
        sum4(head * hd + half + j, u);
        const int pos = qkv.tok_pos[m];
        if (qkv.cos_t && head < qkv.H + qkv.Hkv) {
            const float4 cs = *reinterpret_cast<const float4*>(qkv.cos_t + (size_t)pos * half + j);
            const float4 sn = *reinterpret_cast<const float4*>(qkv.sin_t + (size_t)pos * half + j);
            const float cc[4] = {cs.x, cs.y, cs.z, cs.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float y0 = v[i] * cc[i] - u[i] * ss[i], y1 = v[i] * ss[i] + u[i] * cc[i];
                v[i] = y0;
                u[i] = y1;
            }
        }
        __nv_bfloat16* row = qkv_dest(qkv, (__nv_bfloat16*)Cout, m, head, pos);
        *reinterpret_cast<uint2*>(row + j) = make_uint2(pack2(v[0], v[1]), pack2(v[2], v[3]));
        *reinterpret_cast<uint2*>(row + half + j) = make_uint2(pack2(u[0], u[1]), pack2(u[2], u[3]));
        return;
    }
    if (EPI == EPI_SWIGLU) {
        // outputs c..c+3 lie in one block of 8: their gate columns and, 8 further, their up columns
        const int gcol = (c >> 3) * 16 + (c & 7);
        float u[4];
        sum4(gcol, v);
        sum4(gcol + 8, u);
        __nv_bfloat16* dst = (__nv_bfloat16*)Cout + (size_t)m * NO + c;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (c + i < NO) dst[i] = __float2bfloat16_rn(u[i] * (v[i] / (1.0f + __expf(-v[i]))));
        return;
    }
    sum4(c, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (c + i >= N) break;
        const size_t o = (size_t)m * N + c + i;
        if (EPI == EPI_BF16) ((__nv_bfloat16*)Cout)[o] = __float2bfloat16_rn(v[i]);
        else if (EPI == EPI_F32) ((float*)Cout)[o] = v[i];
        else ((float*)Cout)[o] = residual[o] + v[i];
    }
}

template <int EPI>
int launch_reduce(const float* part, int splits, void* C, const float* residual, int M, int N, const QkvArgs& qkv,
                  cudaStream_t stream) {
    const int plane_rows = (M + 31) / 32 * 32;
    const int NO = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? N >> 1 : N;
    const long threads = (long)M * ((NO + 3) >> 2);
    return launch_pdl(splitk_reduce_kernel<EPI>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream, part, splits,
                      plane_rows, C, residual, M, N, qkv);
}

// ------------------------------------------------------------------ host side
// A row-major bf16 matrix [rows, K] as a 2-D tensor map with boxes of [box_rows, 64].
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    return make_map_bf16(map, base, rows, K, K, box_rows);
}

template <int BN, int STAGES, int EPI, int AROWS>
int launch_epi(const CUtensorMap& ma, const CUtensorMap& mb, void* C, const float* residual, int M, int N, int K,
               int n_sms, int splits, const QkvArgs& qkv, cudaStream_t stream) {
    constexpr bool STAGED = StagedEpilogue<BN, EPI, AROWS>::value;
    constexpr size_t smem = sizeof(Smem<BN, STAGES, AROWS, STAGED>) + 1024;
    static_assert(smem <= 232448, "more shared memory than a block may have");
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, EPI, AROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        configured = true;
    }
    int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * splits;
    int grid = tiles < n_sms ? tiles : n_sms;
    // The epilogue goes through shared memory and TMA stores when the output's rows are 16-byte aligned
    // (and, for the residual, when the sums are added in place).
    CUtensorMap mc{};
    int staged = 0;
    const int plane_rows = (M + 31) / 32 * 32;          // rows of one range's plane of the scratch
    if constexpr (STAGED)
        staged = staged_map<EPI>(&mc, C, residual, splits > 1 ? (long)splits * plane_rows : M, EPI == EPI_SWIGLU ? N / 2 : N);
    return launch_pdl(gemm_tc_kernel<BN, STAGES, EPI, AROWS>, dim3(grid), dim3(N_THREADS), smem, stream, ma, mb, mc, staged, C, residual,
                      M, N, K, splits, plane_rows, qkv);
}

// ALL: every epilogue; otherwise only the two that products with many columns have (SwiGLU, float32 store).
template <int BN, int STAGES, int AROWS = BM, bool ALL = true>
int launch_bn(const void* A, const void* W, void* C, const float* residual, int M, int N, int K, int epi, int n_sms,
              int splits, float* scratch, cudaStream_t stream, const QkvArgs& qkv = QkvArgs{}) {
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, M, K, AROWS);
    if (rc != LQ_OK) return rc;
    rc = make_map(&mb, W, N, K, BN);
    if (rc != LQ_OK) return rc;
    if (splits > 1) {
        rc = launch_epi<BN, STAGES, EPI_F32, AROWS>(ma, mb, scratch, nullptr, M, N, K, n_sms, splits, QkvArgs{}, stream);
        if (rc != LQ_OK) return rc;
        switch (epi) {
            case EPI_BF16: return launch_reduce<EPI_BF16>(scratch, splits, C, residual, M, N, qkv, stream);
            case EPI_F32: return launch_reduce<EPI_F32>(scratch, splits, C, residual, M, N, qkv, stream);
            case EPI_RESID: return launch_reduce<EPI_RESID>(scratch, splits, C, residual, M, N, qkv, stream);
            case EPI_SWIGLU: return launch_reduce<EPI_SWIGLU>(scratch, splits, C, residual, M, N, qkv, stream);
            case EPI_QKV: return launch_reduce<EPI_QKV>(scratch, splits, C, residual, M, N, qkv, stream);
        }
        return LQ_BAD_DTYPE;
    }
    if constexpr (ALL && (BN == 128 || BN == 256)) {
        if (epi == EPI_QKV) return launch_epi<BN, STAGES, EPI_QKV, AROWS>(ma, mb, C, residual, M, N, K, n_sms, 1, qkv, stream);
    }
    if constexpr (ALL) {
        if (epi == EPI_BF16) return launch_epi<BN, STAGES, EPI_BF16, AROWS>(ma, mb, C, residual, M, N, K, n_sms, 1, qkv, stream);
        if (epi == EPI_RESID) return launch_epi<BN, STAGES, EPI_RESID, AROWS>(ma, mb, C, residual, M, N, K, n_sms, 1, qkv, stream);
    }
    if (epi == EPI_F32) return launch_epi<BN, STAGES, EPI_F32, AROWS>(ma, mb, C, residual, M, N, K, n_sms, 1, qkv, stream);
    if (epi == EPI_SWIGLU) return launch_epi<BN, STAGES, EPI_SWIGLU, AROWS>(ma, mb, C, residual, M, N, K, n_sms, 1, qkv, stream);
    return LQ_BAD_DTYPE;
}

int sm_count() {
    static int n_sms = 0;
    if (!n_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return n_sms;
}

// Into how many ranges the contraction is cut: only when 128 x 256 tiles alone leave most SMs idle
// (few rows, narrow weight); then as many as fill the SMs once, each at least MIN_KB steps of 64 long.
constexpr int MIN_KB = 6;
constexpr int MAX_SPLITS = 16;
int plan_splits(int M, int N, int K) {
    const long tiles = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    const int n_kb = (K + BK - 1) / BK;
    if (tiles * 3 > sm_count() * 2) return 1;
    long s = sm_count() / tiles;
    if (s > n_kb / MIN_KB) s = n_kb / MIN_KB;
    if (s > MAX_SPLITS) s = MAX_SPLITS;
    return s < 1 ? 1 : (int)s;
}

// The choice of tile shape and of ranges of K for a product, and its launch.
int gemm_tc_dispatch(const void* A, const void* W, void* C, const float* residual, int M, int N, int K, int epi,
                            float* scratch, const QkvArgs& qkv, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LQ_OK;
    if (K <= 0 || K % 8 != 0) return LQ_BAD_SIZE;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return LQ_BAD_SIZE;
    if (epi == EPI_SWIGLU && N % 16 != 0) return LQ_BAD_SIZE;
    if (epi == EPI_RESID && residual == nullptr) return LQ_BAD_SIZE;
    const int n_sms = sm_count();
    const int splits = plan_splits(M, N, K);
    if (splits > 1) {
        if (!scratch || ((uintptr_t)scratch & 15)) return LQ_BAD_SIZE;
        if (M <= 64) return launch_bn<256, 5, 64>(A, W, C, residual, M, N, K, epi, n_sms, splits, scratch, stream, qkv);
        return launch_bn<256, 4>(A, W, C, residual, M, N, K, epi, n_sms, splits, scratch, stream, qkv);
    }
    long tiles256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    if (M <= 64) {
        // At most 64 rows: one row of tiles, bound by reading W: the tile width whose rounds over the SMs read
        // the least (rounds x width), so that no round leaves most SMs idle.  28672 columns: 138 tiles of 208 in
        // one round instead of 224 tiles of 128 in two.  The two epilogues that products with many columns have
        // choose among all widths; the others (q/k/v, residual) have few columns in the models at hand and take
        // 256 or 128.  As many stages as the shared memory holds.
        int best = (tiles256 >= n_sms || epi == EPI_QKV) ? 256 : 128;
        if (epi == EPI_SWIGLU || epi == EPI_F32) {
            static const int widths[] = {256, 224, 208, 192, 176, 160, 144, 128};
            long best_cost = -1;
            for (int w : widths) {
                const long tiles = (N + w - 1) / w, cost = (tiles + n_sms - 1) / n_sms * w;
                if (best_cost < 0 || cost < best_cost) { best = w; best_cost = cost; }
            }
        }
#define LQ_W(w, st, all) case w: return launch_bn<w, st, 64, all>(A, W, C, residual, M, N, K, epi, n_sms, 1, nullptr, stream, qkv)
        switch (best) {
            LQ_W(256, 5, true); LQ_W(224, 6, false); LQ_W(208, 6, false); LQ_W(192, 7, false); LQ_W(176, 7, false);
            LQ_W(160, 8, false); LQ_W(144, 8, false); LQ_W(128, 9, true);
        }
#undef LQ_W
    }
    // Many rows: wide tiles when they still fill the GPU, narrower ones otherwise.
    if (tiles256 >= n_sms) return launch_bn<256, 4>(A, W, C, residual, M, N, K, epi, n_sms, 1, nullptr, stream, qkv);
    return launch_bn<128, 6>(A, W, C, residual, M, N, K, epi, n_sms, 1, nullptr, stream, qkv);
}

}  // namespace

// A [M, K] and W [N, K] bfloat16, row-major, 16-byte aligned, K % 8 == 0.
// For EPI_SWIGLU, N counts the interleaved gate and up rows (N % 16 == 0) and C is [M, N / 2].
// scratch: lq_gemm_tc_scratch_floats(M, N, K) floats (0: unused): a plane of M rounded up to 32 rows for each range of K.
LQ_EXPORT int lq_gemm_tc(const void* A, const void* W, void* C, const float* residual, int M, int N, int K, int epi,
                         float* scratch, cudaStream_t stream) {
    if (epi < EPI_BF16 || epi > EPI_SWIGLU) return LQ_BAD_DTYPE;
    return gemm_tc_dispatch(A, W, C, residual, M, N, K, epi, scratch, QkvArgs{}, stream);
}

// The q/k/v projection with its epilogue fused: X [M, K] . W^T for W [(H + 2 Hkv) hd, K]; q and k are rotated
// by the cos/sin tables at each row's position (tables null: no rotation); q goes to q_out [M, H hd], k and v go
// into the row's cache page.  hd is 64 or 128.  scratch: lq_gemm_tc_scratch_floats(M, (H + 2 Hkv) hd, K) floats
// when that number is above 1.
LQ_EXPORT int lq_gemm_tc_qkv(const void* X, const void* W, void* q_out, int M, int K, const float* cos_t,
                             const float* sin_t, const int* tok_pos, const int* tok_seq, const int* slots,
                             const int* page_table, int pt_stride, void* k_pages, void* v_pages, int H, int Hkv, int hd,
                             int page_size, float* scratch, cudaStream_t stream) {
    if (M <= 0) return LQ_OK;
    if ((hd != 64 && hd != 128) || H <= 0 || Hkv <= 0 || page_size <= 0) return LQ_BAD_SIZE;
    if (((uintptr_t)q_out & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return LQ_BAD_SIZE;
    if (cos_t && (((uintptr_t)cos_t & 15) || ((uintptr_t)sin_t & 15))) return LQ_BAD_SIZE;
    const QkvArgs a{cos_t, sin_t, tok_pos, tok_seq, slots, page_table, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
                    pt_stride, H, Hkv, hd, page_size};
    return gemm_tc_dispatch(X, W, q_out, nullptr, M, (H + 2 * Hkv) * hd, K, EPI_QKV, scratch, a, stream);
}

LQ_EXPORT int lq_gemm_tc_splits(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    return plan_splits(M, N, K);
}

// Floats of scratch that a product of these sizes needs (0 when the contraction is not cut).
LQ_EXPORT long lq_gemm_tc_scratch_floats(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int splits = plan_splits(M, N, K);
    return splits > 1 ? (long)splits * ((M + 31) / 32 * 32) * N : 0;
}

// The status word of the bounded waits: 0, or the code of the first wait that gave up
// (1 producer, 2 accumulator free, 3 stage full, 4 accumulator full).  Reading it resets it.
LQ_EXPORT int lq_gemm_tc_status() { return tc::status_read(); }

// The same word in host memory that the device writes through (readable without a CUDA call, so polling
// it never waits for work that is queued); null when it could not be set up.
LQ_EXPORT int* lq_gemm_tc_status_word() { return tc::status_word(); }
