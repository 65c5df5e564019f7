// Thin wrappers around the PTX of the fifth-generation tensor cores and of TMA, shared by the
// kernels that use them: mbarriers with bounded waits, tensor-map loads, tcgen05.mma with
// shared-memory descriptors, loads and stores of tensor memory.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace tc {

constexpr unsigned long long WAIT_NS = 2000000000ull;   // a wait gives up after about two seconds

// ------------------------------------------------------------------ the status word of the bounded waits
// A wait that gives up records a code: in device memory, and in a word of mapped host memory that the
// host reads without any CUDA call (polling it cannot wait for, or fall behind, queued work).
__device__ int g_status = 0;
__device__ volatile int* g_status_mapped = nullptr;

// The first code stays: the waits that give up after it are its consequences.
__device__ __forceinline__ void give_up(int code) {
    if (atomicCAS(&g_status, 0, code) != 0) return;
    volatile int* p = g_status_mapped;
    if (p) { *p = code; __threadfence_system(); }
}

// Host: the mapped word, made on first use and announced to the current device (once per device).
static inline int* status_word() {
    static int* host = nullptr;
    static bool told[64] = {};
    static bool failed = false;
    if (failed) return nullptr;
    if (!host) {
        if (cudaHostAlloc((void**)&host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            (void)cudaGetLastError();
            failed = true;
            host = nullptr;
            return nullptr;
        }
        *host = 0;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return host;
    if (!told[dev]) {
        int* dptr = nullptr;
        if (cudaHostGetDevicePointer((void**)&dptr, host, 0) == cudaSuccess &&
            cudaMemcpyToSymbol(g_status_mapped, &dptr, sizeof(dptr)) == cudaSuccess)
            told[dev] = true;
        else
            (void)cudaGetLastError();
    }
    return host;
}

// Host: the code in device memory (a synchronous copy: it waits for the device); reading resets both words.
static inline int status_read() {
    int v = 0, zero = 0;
    cudaMemcpyFromSymbol(&v, g_status, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    int* host = status_word();
    if (host && *host) { if (!v) v = *host; *host = 0; }
    return v;
}

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
// Bounded wait: false when the phase did not complete within WAIT_NS.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = globaltimer();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try(bar, parity)) return true;
        if (globaltimer() - t0 > WAIT_NS) return false;
    }
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// x is the innermost coordinate (elements; its byte offset must be a multiple of 16).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Stores of a box from shared memory (written by threads, then fence_async_shared) to a tensor in global
// memory: plain, or added to what is there (float32).  Elements of the box outside the tensor are not written.
// The inner coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most N of this thread's groups of stores still read their shared memory / are still under way.
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
// Writes of ordinary threads to shared memory become visible to the tensor cores and TMA.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// The same with the A operand in tensor memory: row r of A in lane r, two bfloat16 per 32-bit column, the 16
// elements of one product's K in 8 consecutive columns from a_tmem on.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// 32 lanes x 32 columns: each thread of the warp gets 32 consecutive columns of its lane.
__device__ __forceinline__ void ld32(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void st32(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors for tiles whose rows are 128 bytes, swizzled in 8-row groups of
// 1024 bytes (what a TMA load with 128-byte swizzle writes).
//   K-major operand [rows, 64 elements]: the 64 elements of the contraction are contiguous.
//   MN-major operand [contraction rows, 64 elements of M or N]: consecutive contraction indices are
//   consecutive 128-byte rows; `panel_bytes` is the distance to the next 64 elements of M or N.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                            // leading byte offset: unused with a swizzle
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset: next 8 rows
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // 128-byte swizzle
    return d;
}
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t panel_bytes) {
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((panel_bytes >> 4) & 0x3FFF) << 16;   // leading byte offset: next 64 elements of M or N
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: next 8 contraction rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, A K-major; B K-major or MN-major.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------ host: tensor maps
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiled encode_fn() {
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

// A row-major bf16 matrix [rows, cols] with a row pitch of `pitch` elements, as a 2-D tensor map
// with boxes of [box_rows, 64 columns] and 128-byte swizzle.  pitch * 2 must be a multiple of 16.
static inline int make_map_bf16(CUtensorMap* map, const void* base, long rows, long cols, long pitch, int box_rows) {
    EncodeTiled fn = encode_fn();
    if (!fn) return LQ_NO_DRIVER;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? LQ_OK : LQ_BAD_SIZE;
}

// A row-major matrix [rows, cols] of float32 (elt 4) or bfloat16 (elt 2) with a row pitch of `pitch` elements,
// as a 2-D tensor map with boxes of [box_rows, 128 bytes] and 128-byte swizzle: the target of an epilogue's stores.
static inline int make_map_out(CUtensorMap* map, const void* base, int elt, long rows, long cols, long pitch, int box_rows) {
    EncodeTiled fn = encode_fn();
    if (!fn) return LQ_NO_DRIVER;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * elt};
    cuuint32_t box[2] = {(cuuint32_t)(128 / elt), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, elt == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? LQ_OK : LQ_BAD_SIZE;
}

}  // namespace tc
