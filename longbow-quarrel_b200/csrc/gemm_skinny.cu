// y = x . W^T for few rows of x (decoding: one token for each sequence of the batch).
//
// With at most 64 rows every weight is used once, so the product is bound by
// reading W from HBM.  Each block owns 16 rows of W and all of K (the work of a block on
// its rows is gemm_skinny.cuh's).  A block keeps all of K: measured on B200, cutting K between blocks made every
// shape slower.  An output therefore depends only on its own row of x and W, not on how many
// other rows the batch has.
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
#include "gemm_skinny.cuh"

namespace {

using namespace skinny;

// The weights that the stream reads next (of the product that follows this one): the last blocks of
// this launch ask for their first bytes to be brought into L2, so that HBM stays busy while this
// launch runs out and the next one starts from L2.  ptr null: nothing is asked for.
struct NextWeights {
    const char* ptr;
    unsigned bytes_per_block;   // a multiple of 16
    int first_block;            // blocks from this one on ask for one piece each
};

template <int MT, int EPI>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, void* Cout,
                   const float* residual, int M, int N, int K, const QkvArgs qkv, const NormArgs norm,
                   const NextWeights next) {
    __shared__ Scratch<MT> sm;
    Unit<MT, EPI, false> unit;
    unit.begin(X, W, M, N, K, qkv, blockIdx.x);
    Frags<MT> fa;
    // Weights are written by no kernel, so the first round of them is loaded before the kernel
    // ahead of this one is known to have finished; x and the output wait for pdl_wait().
    unit.first_w(fa);
    pdl_launch_dependents();
    if (next.ptr && (int)blockIdx.x >= next.first_block && threadIdx.x == 0) {
        const char* piece = next.ptr + (size_t)((int)blockIdx.x - next.first_block) * next.bytes_per_block;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(piece), "r"(next.bytes_per_block) : "memory");
    }
    pdl_wait();
    unit.run(fa, sm, Cout, residual, qkv, norm, blockIdx.x, gridDim.x);
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
