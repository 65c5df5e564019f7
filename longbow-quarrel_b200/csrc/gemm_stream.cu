// y = x . W^T for few rows of x (decoding), as one even stream of W through every SM.
//
// With at most 64 tokens every weight is used once and the product is bound by reading W.
// W [N, K] is cut into units of 128 rows x 64 columns; the units, in row-tile-major order, are
// dealt out to one persistent block per SM in equal contiguous shares, whatever N and K are
// (a block's share may start and end in the middle of a row tile).  Inside a block
//   warp 0      one lane keeps a ring of shared-memory stages full with TMA loads
//               (cp.async.bulk.tensor, 128-byte swizzle) of a W unit and the matching
//               [tokens, 64] piece of x -- the loads never wait for arithmetic, so HBM
//               sees a steady stream;
//   warp 1      one lane issues tcgen05.mma with W as the M side (128 rows) and the tokens
//               as the N side (16, 32 or 64), accumulating in tensor memory;
//   warps 2..5  read a finished accumulator (each thread one row of W, all tokens) and
//               either store it (the block had the whole row tile) or park it in scratch
//               memory; the block that parks last for a row tile adds the parked pieces in
//               the order of K, so the sum does not depend on which block that was.
// The four 16-column steps of a unit accumulate into four separate accumulators (a product then
// never waits for its predecessor); the epilogue adds them.
// The cut depends on N, K and the number of SMs only, never on the number of tokens, so a
// token's result does not depend on what else is in the batch.
//
// Weights are written by no kernel: a block loads its first stages of W before the kernel
// ahead of it on the stream is known to have finished (programmatic dependent launch) and
// waits only before it touches x.  Every wait on a barrier is bounded.
//
// Epilogues: bfloat16 store; float32 store; float32 residual add in place; SwiGLU over
// weight rows interleaved in blocks of 8 (8 gate rows, then their 8 up rows).
//
// Reference counterpart: the mat-vec kernels linear_f16 / linear_f16_f32
// (internal/device/kernels.metal:105-132,1084-1106).
#include "common.cuh"
#include <cuda.h>

#define EPI_BF16 0
#define EPI_F32 1
#define EPI_RESID 2
#define EPI_SWIGLU 3

namespace {

constexpr int TILE_N = 128;            // rows of W per unit (the M side of the mma)
constexpr int BK = 64;                 // columns per unit: 64 bf16 = 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int N_THREADS = 192;
constexpr int MAX_TILES = 4096;        // counters of the row tiles
constexpr int MAX_BLOCKS = 256;
constexpr unsigned long long WAIT_NS = 2000000000ull;

__device__ int g_status = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = globaltimer();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try(bar, parity)) return true;
        if (globaltimer() - t0 > WAIT_NS) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major tile with 128-byte rows, swizzled in 8-row groups of 1024 bytes (as TMA writes it).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// bf16 x bf16 -> f32, both operands K-major, M 128, N n.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);
}

template <int TOK>
struct Cfg {
    static constexpr int STAGE_BYTES = (TILE_N + TOK) * BK * 2;
    static constexpr int STAGES = (180 * 1024) / STAGE_BYTES;
};

template <int TOK>
struct Smem {
    alignas(1024) uint8_t w[Cfg<TOK>::STAGES][TILE_N * BK * 2];
    alignas(1024) uint8_t x[Cfg<TOK>::STAGES][TOK * BK * 2];
    alignas(8) uint64_t full[Cfg<TOK>::STAGES];
    uint64_t empty[Cfg<TOK>::STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int last_flag;
};

// The block that holds unit u when `total` units are dealt to `G` blocks in equal shares.
__device__ __forceinline__ int block_of_unit(long u, long total, int G) { return (int)(((u + 1) * G + total - 1) / total) - 1; }

// One row n of the result for tokens 0..M-1, v[m] = (x_m . W_n).
template <int TOK, int EPI>
__device__ __forceinline__ void store_row(const float (&v)[TOK], void* Cout, const float* residual, int n, int lane,
                                          int M, int N) {
    if (EPI == EPI_SWIGLU) {
        // Rows alternate 8 gate, 8 up: lane l and lane l ^ 8 hold a gate row and its up row.
        const int NO = N >> 1;
        const bool is_gate = (lane & 8) == 0;
        const int f = (n >> 4) * 8 + (n & 7);
#pragma unroll
        for (int m = 0; m < TOK; ++m) {
            if (m >= M) break;
            float other = __shfl_xor_sync(0xffffffffu, v[m], 8);
            if (is_gate && n < N) {
                float g = v[m], u = other;
                ((__nv_bfloat16*)Cout)[(size_t)m * NO + f] = __float2bfloat16_rn(u * (g / (1.0f + expf(-g))));
            }
        }
        return;
    }
    if (n >= N) return;
    float r[TOK];
    if (EPI == EPI_RESID) {
        // All loads before any store: the output is the residual itself, so a load after a store
        // would have to wait for it.
#pragma unroll
        for (int m = 0; m < TOK; ++m) r[m] = m < M ? __ldcg(residual + (size_t)m * N + n) : 0.f;
    }
#pragma unroll
    for (int m = 0; m < TOK; ++m) {
        if (m >= M) break;
        size_t o = (size_t)m * N + n;
        if (EPI == EPI_BF16) ((__nv_bfloat16*)Cout)[o] = __float2bfloat16_rn(v[m]);
        else if (EPI == EPI_F32) ((float*)Cout)[o] = v[m];
        else ((float*)Cout)[o] = r[m] + v[m];
    }
}

template <int TOK, int EPI>
__global__ void __launch_bounds__(N_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   void* Cout, const float* residual, int M, int N, int K, float* part, int* counters) {
    extern __shared__ uint8_t smem_raw[];
    using S = Smem<TOK>;
    constexpr int STAGES = Cfg<TOK>::STAGES;
    constexpr uint32_t STAGE_BYTES = Cfg<TOK>::STAGE_BYTES;
    constexpr int CHAINS = BK / UMMA_K;                     // one accumulator per 16-column step of a unit
    constexpr uint32_t ACC_COLS = CHAINS * TOK;             // columns of one accumulator set
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;            // two sets: 128, 256 or 512 columns
    S& sm = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = (K + BK - 1) / BK;
    const long total = (long)((N + TILE_N - 1) / TILE_N) * KB;
    const int G = gridDim.x, c = blockIdx.x;
    const long u0 = total * c / G, u1 = total * (c + 1) / G;
    const int n_units = (int)(u1 - u0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sm.full[s]), 1); mbar_init(smem_u32(&sm.empty[s]), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&sm.acc_full[a]), 1); mbar_init(smem_u32(&sm.acc_empty[a]), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            const int pre = n_units < STAGES ? n_units : STAGES;
            for (int it = 0; it < pre; ++it) {          // weights first: they depend on no kernel
                const long u = u0 + it;
                const uint32_t full = smem_u32(&sm.full[it]);
                mbar_expect_tx(full, STAGE_BYTES);
                tma_load_2d(smem_u32(sm.w[it]), &map_w, (int)(u % KB) * BK, (int)(u / KB) * TILE_N, full);
            }
            pdl_wait();
            for (int it = 0; it < pre; ++it)
                tma_load_2d(smem_u32(sm.x[it]), &map_x, (int)((u0 + it) % KB) * BK, 0, smem_u32(&sm.full[it]));
            bool ok = true;
            int it = pre;
            for (; it < n_units; ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&sm.empty[s]), ((it / STAGES) & 1) ^ 1)) { atomicExch(&g_status, 1); ok = false; break; }
                const long u = u0 + it;
                const uint32_t full = smem_u32(&sm.full[s]);
                mbar_expect_tx(full, STAGE_BYTES);
                tma_load_2d(smem_u32(sm.w[s]), &map_w, (int)(u % KB) * BK, (int)(u / KB) * TILE_N, full);
                tma_load_2d(smem_u32(sm.x[s]), &map_x, (int)(u % KB) * BK, 0, full);
            }
            if (!ok) {
                for (int back = 1; back <= STAGES && back <= it; ++back) {
                    int j = it - back;
                    mbar_wait(smem_u32(&sm.full[j % STAGES]), (j / STAGES) & 1);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            pdl_wait();
            constexpr uint32_t idesc = instr_desc(TOK);
            uint32_t seg = 0;
            bool ok = true;
            uint32_t d_tmem = tmem_base;
            for (int it = 0; it < n_units && ok; ++it) {
                const long u = u0 + it;
                const int kb = (int)(u % KB);
                const bool first = (it == 0) || kb == 0;
                if (first) {
                    const uint32_t acc = seg & 1;
                    if (!mbar_wait(smem_u32(&sm.acc_empty[acc]), ((seg >> 1) & 1) ^ 1)) { atomicExch(&g_status, 2); ok = false; break; }
                    tc_fence_after();
                    d_tmem = tmem_base + acc * ACC_COLS;
                }
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&sm.full[s]), (it / STAGES) & 1)) { atomicExch(&g_status, 3); ok = false; break; }
                tc_fence_after();
                const uint64_t da = smem_desc(smem_u32(sm.w[s])), db = smem_desc(smem_u32(sm.x[s]));
                // The four products of a unit go to four accumulators, so that a product never waits
                // for the one issued just before it; the epilogue adds the four.
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma(d_tmem + k * TOK, da + 2 * k, db + 2 * k, idesc, first ? 0u : 1u);
                tc_commit(smem_u32(&sm.empty[s]));
                if (kb == KB - 1 || it == n_units - 1) {
                    tc_commit(smem_u32(&sm.acc_full[seg & 1]));
                    ++seg;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        pdl_wait();
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t seg = 0;
        bool ok = true;
        long u = u0;
        while (u < u1 && ok) {
            const int tile = (int)(u / KB), kb_lo = (int)(u % KB);
            const int kb_hi = (int)((u1 - u) < (long)(KB - kb_lo) ? kb_lo + (u1 - u) : KB);
            const uint32_t acc = seg & 1;
            if (!mbar_wait(smem_u32(&sm.acc_full[acc]), (seg >> 1) & 1)) { atomicExch(&g_status, 4); ok = false; break; }
            tc_fence_after();
            float v[TOK];
            const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int j = 0; j < TOK / 16; ++j) tc_ld16(taddr + j * 16, reinterpret_cast<uint32_t*>(v) + j * 16);
            tc_wait_ld();
#pragma unroll
            for (int ch = 1; ch < CHAINS; ++ch) {       // add the other chains, in the order of K
                float w[TOK];
#pragma unroll
                for (int j = 0; j < TOK / 16; ++j) tc_ld16(taddr + ch * TOK + j * 16, reinterpret_cast<uint32_t*>(w) + j * 16);
                tc_wait_ld();
#pragma unroll
                for (int m = 0; m < TOK; ++m) v[m] += w[m];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.acc_empty[acc]));     // the accumulator may be written again
            const int n = tile * TILE_N + row_in_tile;
            if (kb_lo == 0 && kb_hi == KB) {
                store_row<TOK, EPI>(v, Cout, residual, n, lane, M, N);
            } else {
                // Part of a row tile: park it.  A block parks at most two pieces, its first and its last.
                const int slot = c * 2 + (u == u0 ? 0 : 1);
                float* mine = part + (size_t)slot * TOK * TILE_N;
#pragma unroll
                for (int m = 0; m < TOK; ++m)
                    if (m < M) mine[m * TILE_N + row_in_tile] = v[m];
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int first_blk = block_of_unit((long)tile * KB, total, G);
                const int last_blk = block_of_unit((long)tile * KB + KB - 1, total, G);
                if (threadIdx.x == 64) {
                    int old = atomicAdd(&counters[tile], 1);
                    int last = (old == last_blk - first_blk);
                    if (last) counters[tile] = 0;
                    sm.last_flag = last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (sm.last_flag) {
                    __threadfence();
#pragma unroll
                    for (int m = 0; m < TOK; ++m) v[m] = 0.f;
                    for (int b = first_blk; b <= last_blk; ++b) {      // in the order of K
                        const long bu0 = total * b / G;
                        const int bslot = b * 2 + ((int)(bu0 / KB) == tile ? 0 : 1);
                        const float* p = part + (size_t)bslot * TOK * TILE_N;
#pragma unroll
                        for (int m = 0; m < TOK; ++m)
                            if (m < M) v[m] += __ldcg(p + m * TILE_N + row_in_tile);
                    }
                    store_row<TOK, EPI>(v, Cout, residual, n, lane, M, N);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");       // last_flag is read before it is written again
            }
            u += kb_hi - kb_lo;
            ++seg;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiled fn = encode_fn();
    if (!fn) return LQ_NO_DRIVER;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? LQ_OK : LQ_BAD_SIZE;
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

template <int TOK, int EPI>
int launch_epi(const CUtensorMap& mw, const CUtensorMap& mx, void* C, const float* residual, int M, int N, int K,
               float* part, int* counters, cudaStream_t stream) {
    constexpr size_t smem = sizeof(Smem<TOK>) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_stream_kernel<TOK, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        configured = true;
    }
    long total = (long)((N + TILE_N - 1) / TILE_N) * ((K + BK - 1) / BK);
    int grid = total < sm_count() ? (int)total : sm_count();
    if (grid > MAX_BLOCKS) grid = MAX_BLOCKS;      // the scratch holds two parked pieces per block
    return launch_pdl(gemm_stream_kernel<TOK, EPI>, dim3(grid), dim3(N_THREADS), smem, stream, mw, mx, C, residual,
                      M, N, K, part, counters);
}

template <int TOK>
int launch_tok(const void* X, const void* W, void* C, const float* residual, int M, int N, int K, int epi, float* part,
               int* counters, cudaStream_t stream) {
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, N, K, TILE_N);
    if (rc != LQ_OK) return rc;
    rc = make_map(&mx, X, M, K, TOK);
    if (rc != LQ_OK) return rc;
    switch (epi) {
        case EPI_BF16: return launch_epi<TOK, EPI_BF16>(mw, mx, C, residual, M, N, K, part, counters, stream);
        case EPI_F32: return launch_epi<TOK, EPI_F32>(mw, mx, C, residual, M, N, K, part, counters, stream);
        case EPI_RESID: return launch_epi<TOK, EPI_RESID>(mw, mx, C, residual, M, N, K, part, counters, stream);
        case EPI_SWIGLU: return launch_epi<TOK, EPI_SWIGLU>(mw, mx, C, residual, M, N, K, part, counters, stream);
    }
    return LQ_BAD_DTYPE;
}

constexpr long COUNTER_BYTES = MAX_TILES * sizeof(int);

}  // namespace

// X [M, K] and W [N, K] bfloat16, row-major, 16-byte aligned; M <= 64, K % 8 == 0, N <= 128 * 4096.
// For EPI_SWIGLU, N counts the interleaved gate and up rows (N % 16 == 0) and C is [M, N / 2].
// scratch: lq_gemm_stream_scratch_bytes() bytes that start zeroed and are used by one product at a
// time (products on one stream follow one another; two streams need two scratch buffers).
LQ_EXPORT int lq_gemm_stream(const void* X, const void* W, void* C, const float* residual, int M, int N, int K,
                             int epi, void* scratch, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LQ_OK;
    if (M > 64 || K <= 0 || K % 8 != 0 || (N + TILE_N - 1) / TILE_N > MAX_TILES) return LQ_BAD_SIZE;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15) || !scratch) return LQ_BAD_SIZE;
    if (epi == EPI_SWIGLU && N % 16 != 0) return LQ_BAD_SIZE;
    if (epi == EPI_RESID && residual == nullptr) return LQ_BAD_SIZE;
    int* counters = (int*)scratch;
    float* part = (float*)((char*)scratch + COUNTER_BYTES);
    if (M <= 16) return launch_tok<16>(X, W, C, residual, M, N, K, epi, part, counters, stream);
    if (M <= 32) return launch_tok<32>(X, W, C, residual, M, N, K, epi, part, counters, stream);
    return launch_tok<64>(X, W, C, residual, M, N, K, epi, part, counters, stream);
}

// Counters of the row tiles, then two parked pieces [64 tokens, 128 rows] for each of up to 256 blocks.
LQ_EXPORT long lq_gemm_stream_scratch_bytes() {
    return COUNTER_BYTES + (long)MAX_BLOCKS * 2 * 64 * TILE_N * sizeof(float);
}

LQ_EXPORT int lq_gemm_stream_status() {
    int v = 0, zero = 0;
    cudaMemcpyFromSymbol(&v, g_status, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
