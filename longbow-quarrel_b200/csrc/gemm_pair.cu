// y = x . W^T for many rows on pairs of SMs: tcgen05.mma with cta_group::2.
//
// Two blocks of a cluster make one 256 x 256 tile.  Each holds 128 rows of x and 128 rows of W per
// stage (half of what a block of gemm_tc holds for a 128 x 256 tile); one thread of the pair's first
// block issues products of M 256, N 256, K 16, which read x from each block's own shared memory and
// the two halves of W from both, and leave each block's 128 rows of the result in its own tensor
// memory.  A product of 128 x 256 x 16 reads 12 KB of operands from one SM's shared memory in 128
// cycles, close to what the shared memory delivers; in a pair each SM reads 8 KB for the same work, and
// the stages, a third smaller, are six deep instead of four.
//
//   warp 0 (both blocks)   one lane issues the TMA loads of its block's halves; all of a stage's bytes
//                          are counted by the first block's barrier;
//   warp 1 (first block)   one lane waits for a stage, issues four products, and frees the stage in
//                          both blocks (tcgen05.commit to both blocks' barriers); after a tile's last
//                          product it tells both blocks' epilogue warps;
//   warps 2..5 (both)      read their block's accumulator and store it through shared memory by TMA
//                          (gemm_tc_epilogue.cuh), then free the accumulator at the first block.
// Two accumulators of 256 columns: the epilogue of one tile runs under the products of the next.
// Every wait is bounded, as in gemm_tc; the blocks of a pair meet at a cluster barrier before either
// uses the other's barriers and before either ends.
//
// Epilogues: bfloat16 store, float32 store, residual add in place, SwiGLU, and q/k/v with rotation and cache
// write (q leaves by TMA too; rows of k and v go to their cache pages from the same buffers).  Outputs whose
// rows are not 16-byte aligned, and all other shapes, are gemm_tc's.
//
// Reference counterpart: the library GEMM of internal/device/cuda.go:293-318 (cublasSgemmEx).
#include "gemm_tc_epilogue.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;                // rows of x per block; a pair's tile has 2 BM
constexpr int BN = 256;                // columns of a tile; each block holds BN / 2 rows of W
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int N_THREADS = 192;
constexpr uint32_t STAGE_BYTES = (BM + BN / 2) * BK * 2;       // one block's share of a stage
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;                    // a shared-memory address with this bit cleared is the same place in the pair's first block

struct Smem {
    alignas(1024) uint8_t a[STAGES][BM * BK * 2];
    alignas(1024) uint8_t b[STAGES][BN / 2 * BK * 2];
    alignas(1024) uint8_t stage[4][2 * STAGE_BUF_BYTES];
    alignas(8) uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A TMA load of this block's half of a pair's operand; its bytes are counted by `bar`, a barrier of the first block.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// Arrives at the barrier at this address in both blocks of the pair once the products issued so far are done.
__device__ __forceinline__ void commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void arrive_at_first(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_MASK) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(N_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, int M, int N, int K, __nv_bfloat16* q_out, const QkvArgs qkv) {
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
    const int total = m_tiles * n_tiles;
    const int n_kb = (K + BK - 1) / BK;
    constexpr uint32_t TMEM_COLS = 2 * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sm.full[s]), 1); mbar_init(smem_u32(&sm.empty[s]), 1); }
        // An accumulator is free again when the four epilogue warps of both blocks have read it.
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&sm.acc_full[a]), 1); mbar_init(smem_u32(&sm.acc_empty[a]), 8); }
        mbar_fence_init();
        prefetch_map(&map_a);
        prefetch_map(&map_b);
        prefetch_map(&map_c);
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(&sm.tmem_base), TMEM_COLS);      // the same warp in both blocks
    pdl_launch_dependents();
    fence_before();
    __syncthreads();
    cluster_sync();             // both blocks' barriers exist before either block's loads or commits reach them
    fence_after();
    const uint32_t tmem_base = sm.tmem_base;
    pdl_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both blocks)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < total && ok; tile += n_pairs) {
                const int m0 = (tile % m_tiles) * 2 * BM + rank * BM, w0 = (tile / m_tiles) * BN + rank * (BN / 2);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&sm.empty[s]), ((it / STAGES) & 1) ^ 1)) { give_up(1); ok = false; break; }
                    const uint32_t full = smem_u32(&sm.full[s]) & PEER_MASK;
                    if (rank == 0) mbar_expect_tx(smem_u32(&sm.full[s]), 2 * STAGE_BYTES);
                    tma_load_2d_pair(smem_u32(sm.a[s]), &map_a, kb * BK, m0, full);
                    tma_load_2d_pair(smem_u32(sm.b[s]), &map_b, kb * BK, w0, full);
                }
            }
            if (!ok && rank == 0) {
                // Copies that were started must land before the pair's shared memory goes away: the first block's
                // barriers count both blocks' bytes, and the second block ends only after the cluster barrier below.
                for (uint32_t back = 1; back <= (uint32_t)STAGES && back <= it; ++back) {
                    uint32_t j = it - back;
                    mbar_wait(smem_u32(&sm.full[j % STAGES]), (j / STAGES) & 1);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (first block of the pair)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = idesc_bf16(2 * BM, BN, false);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int tile = pair; tile < total && ok; tile += n_pairs, ++t) {
                const uint32_t acc = t & 1;
                if (!mbar_wait(smem_u32(&sm.acc_empty[acc]), ((t >> 1) & 1) ^ 1)) { give_up(2); ok = false; break; }
                fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&sm.full[s]), (it / STAGES) & 1)) { give_up(3); ok = false; break; }
                    fence_after();
                    const uint64_t da = desc_k_major(smem_u32(sm.a[s])), db = desc_k_major(smem_u32(sm.b[s]));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    commit_pair(smem_u32(&sm.empty[s]));          // the stage is free in both blocks
                }
                if (ok) commit_pair(smem_u32(&sm.acc_full[acc]));
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5 of both blocks)
        const int quarter = warp & 3;
        uint32_t t = 0;
        int which = 0;
        for (int tile = pair; tile < total; tile += n_pairs, ++t) {
            const int m0 = (tile % m_tiles) * 2 * BM + rank * BM, n0 = (tile / m_tiles) * BN;
            const uint32_t acc = t & 1;
            if (!mbar_wait(smem_u32(&sm.acc_full[acc]), (t >> 1) & 1)) { give_up(4); break; }
            fence_after();
            const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
            if (EPI == EPI_QKV) {
                // BN holds whole heads; q leaves by TMA, rows of k and v go to their cache pages.
                qkv_epilogue_staged(taddr, BN, qkv, &map_c, sm.stage[quarter], which, m0 + quarter * 32, M, n0, N, lane);
            } else if (m0 + quarter * 32 < M) {
                staged_epilogue<EPI>(taddr, BN, sm.stage[quarter], which, &map_c, m0 + quarter * 32, n0, N, lane);
            }
            fence_before();
            __syncwarp();
            if (lane == 0) arrive_at_first(smem_u32(&sm.acc_empty[acc]));
        }
        if (lane == 0) bulk_wait<0>();      // this warp's stores are done before the block ends
    }
    fence_before();
    __syncthreads();
    cluster_sync();             // neither block ends while the other may still read its shared memory or reach its barriers
    if (warp == 1) {
        fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
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

template <int EPI>
int launch(const void* A, const void* W, void* C, const float* residual, int M, int N, int K, cudaStream_t stream,
           const QkvArgs& qkv = QkvArgs{}) {
    CUtensorMap ma, mb, mc{};
    int rc = make_map_bf16(&ma, A, M, K, K, BM);
    if (rc != LQ_OK) return rc;
    rc = make_map_bf16(&mb, W, N, K, K, BN / 2);
    if (rc != LQ_OK) return rc;
    if constexpr (EPI == EPI_QKV) {
        if (make_map_out(&mc, C, 2, M, (long)qkv.H * qkv.hd, (long)qkv.H * qkv.hd, 32) != LQ_OK) return LQ_BAD_SIZE;
    } else {
        if (!staged_map<EPI>(&mc, C, residual, M, EPI == EPI_SWIGLU ? N / 2 : N)) return LQ_BAD_SIZE;
    }
    constexpr size_t smem = sizeof(Smem) + 1024;
    static_assert(smem <= 232448, "more shared memory than a block may have");
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        configured = true;
    }
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(N_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    static const bool pdl = [] { const char* v = getenv("LQ_PDL"); return !(v && v[0] == '0'); }();
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<EPI>, ma, mb, mc, M, N, K, (__nv_bfloat16*)C, qkv);
    return e == cudaSuccess ? LQ_OK : (int)e;
}

}  // namespace

// Whether lq_gemm_pair takes a product of these sizes: enough rows and columns for tiles of 256 x 256 to keep
// five eighths of the pairs of SMs busy (smaller products are gemm_tc's, with its narrower tiles and its cuts
// of K).  Measured, us pairs / gemm_tc at K = 4096: 1024 rows x 4096 columns (64 tiles) 28 / 46, with K = 14336
// 89 / 142; 512 x 4096 (32 tiles) 27 / 30 but with K = 14336 74 / 64; 256 x 4096 (16 tiles) 26 / 23.
LQ_EXPORT int lq_gemm_pair_takes(int M, int N, int K) {
    if (M < 2 * BM || N < BN || K < BK || K % 8 != 0) return 0;
    const long tiles = (long)((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    return tiles * 8 >= (long)(sm_count() / 2) * 5;
}

// A [M, K] and W [N, K] bfloat16, row-major, 16-byte aligned, K % 8 == 0; epi: EPI_BF16, EPI_F32, EPI_RESID
// (C == residual, float32 [M, N], added in place) or EPI_SWIGLU (N counts the interleaved gate and up rows,
// C is [M, N / 2]).  LQ_BAD_SIZE when the output cannot leave by TMA (rows not 16-byte aligned).
LQ_EXPORT int lq_gemm_pair(const void* A, const void* W, void* C, const float* residual, int M, int N, int K, int epi,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LQ_OK;
    if (K <= 0 || K % 8 != 0) return LQ_BAD_SIZE;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return LQ_BAD_SIZE;
    if (epi == EPI_SWIGLU && N % 16 != 0) return LQ_BAD_SIZE;
    switch (epi) {
        case EPI_BF16: return launch<EPI_BF16>(A, W, C, residual, M, N, K, stream);
        case EPI_F32: return launch<EPI_F32>(A, W, C, residual, M, N, K, stream);
        case EPI_RESID: return residual ? launch<EPI_RESID>(A, W, C, residual, M, N, K, stream) : LQ_BAD_SIZE;
        case EPI_SWIGLU: return launch<EPI_SWIGLU>(A, W, C, residual, M, N, K, stream);
    }
    return LQ_BAD_DTYPE;
}

// The q/k/v projection of many rows with its epilogue fused, as lq_gemm_tc_qkv: X [M, K] . W^T for
// W [(H + 2 Hkv) hd, K]; q and k rotated by the tables at each row's position (null: no rotation), q to
// q_out [M, H hd], k and v into the row's cache page.  hd is 64 or 128.
LQ_EXPORT int lq_gemm_pair_qkv(const void* X, const void* W, void* q_out, int M, int K, const float* cos_t,
                               const float* sin_t, const int* tok_pos, const int* tok_seq, const int* slots,
                               const int* page_table, int pt_stride, void* k_pages, void* v_pages, int H, int Hkv, int hd,
                               int page_size, cudaStream_t stream) {
    if (M <= 0) return LQ_OK;
    if ((hd != 64 && hd != 128) || H <= 0 || Hkv <= 0 || page_size <= 0 || K <= 0 || K % 8 != 0) return LQ_BAD_SIZE;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)q_out & 15) || ((uintptr_t)k_pages & 15) ||
        ((uintptr_t)v_pages & 15))
        return LQ_BAD_SIZE;
    if (cos_t && (((uintptr_t)cos_t & 15) || ((uintptr_t)sin_t & 15))) return LQ_BAD_SIZE;
    const QkvArgs a{cos_t, sin_t, tok_pos, tok_seq, slots, page_table, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
                    pt_stride, H, Hkv, hd, page_size};
    return launch<EPI_QKV>(X, W, q_out, nullptr, M, (H + 2 * Hkv) * hd, K, stream, a);
}

LQ_EXPORT int lq_gemm_pair_status() { return tc::status_read(); }
LQ_EXPORT int* lq_gemm_pair_status_word() { return tc::status_word(); }
