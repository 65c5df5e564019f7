// The epilogue that the tcgen05 products share when their output's rows are 16-byte aligned: a warp's
// 32 rows of the accumulator go through a shared-memory buffer of 32 x 128 bytes and leave as one TMA
// store of whole lines (for the residual: one TMA add into the stream, which reads nothing in the SM).
// A thread holds one row of the accumulator, and storing it straight to global memory 16 bytes at a
// time touches 32 lines per instruction: a 128 x 256 float32 tile with its residual then took the four
// epilogue warps 16 us, against 26 us for the tile's products at K = 4096.
#pragma once
#include "tcgen05.cuh"

#define EPI_BF16 0
#define EPI_F32 1
#define EPI_RESID 2
#define EPI_SWIGLU 3
#define EPI_QKV 4       // q, k, v rows: rotate q and k, store k and v into the cache pages

namespace tc {

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int STAGE_BUF_BYTES = 32 * 128;       // one warp's buffer: 32 rows of 128 bytes

// 16-byte piece `piece` (0..7) of row `row` in a buffer of 128-byte rows with the 128-byte swizzle of the tensor maps.
__device__ __forceinline__ uint4* staged_at(uint8_t* buf, int row, int piece) {
    return reinterpret_cast<uint4*>(buf + row * 128 + ((piece ^ (row & 7)) << 4));
}

// Accumulator columns that fill a buffer's 128 bytes per row: 32 floats, 64 bfloat16, or 128 columns of
// interleaved gate and up rows (64 outputs).
template <int EPI> struct StagedCols {
    static constexpr int value = (EPI == EPI_F32 || EPI == EPI_RESID) ? 32 : (EPI == EPI_BF16 ? 64 : 128);
};

// Columns [0, bn) of this warp's 32 lanes of the accumulator at `taddr` go to rows y .. y + 31 of the output
// behind map_c, whose column for accumulator column 0 is n0 (for SwiGLU: output column n0 / 2); columns from
// N on are skipped.  bufs: the warp's two buffers (1024-byte aligned), used in turn; `which` says which is
// next and is kept across calls, as are the stores in flight (wait for them with bulk_wait<0> at the end).
template <int EPI>
__device__ __forceinline__ void staged_epilogue(uint32_t taddr, int bn, uint8_t* bufs, int& which, const CUtensorMap* map_c,
                                                int y, int n0, int N, int lane) {
    constexpr int COLS = StagedCols<EPI>::value;
#pragma unroll 1
    for (int c0 = 0; c0 < bn && n0 + c0 < N; c0 += COLS) {
        uint8_t* buf = bufs + which * STAGE_BUF_BYTES;
        if (lane == 0) bulk_wait_read<1>();            // the store before the last has read this buffer
        __syncwarp();
#pragma unroll
        for (int sub = 0; sub < COLS / 32; ++sub) {
            uint32_t r[32];
            ld32(taddr + c0 + sub * 32, r);
            wait_ld();
            if (EPI == EPI_F32 || EPI == EPI_RESID) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    *staged_at(buf, lane, i) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            } else if (EPI == EPI_BF16) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *staged_at(buf, lane, sub * 4 + i) =
                        make_uint4(pack2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                                   pack2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                                   pack2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                                   pack2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
            } else {
                // 32 columns = [8 gate, 8 up, 8 gate, 8 up] -> 16 outputs
                float o[16];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float gt = __uint_as_float(r[h * 16 + i]), up = __uint_as_float(r[h * 16 + 8 + i]);
                        o[h * 8 + i] = up * (gt / (1.0f + __expf(-gt)));
                    }
                *staged_at(buf, lane, sub * 2) = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
                *staged_at(buf, lane, sub * 2 + 1) = make_uint4(pack2(o[8], o[9]), pack2(o[10], o[11]), pack2(o[12], o[13]), pack2(o[14], o[15]));
            }
        }
        fence_async_shared();
        __syncwarp();
        if (lane == 0) {
            const int x = EPI == EPI_SWIGLU ? (n0 + c0) >> 1 : n0 + c0;
            if (EPI == EPI_RESID) tma_add_2d(map_c, smem_u32(buf), x, y);
            else tma_store_2d(map_c, smem_u32(buf), x, y);
            bulk_commit();
        }
        which ^= 1;
    }
}

// What the q/k/v epilogue needs beside the product: where each row stands and where its cache page is.
// W holds H query heads, then Hkv key heads, then Hkv value heads, hd rows each.
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

// Where elements j .. of head `head` of row m go: q_out, or the row's place in a cache page.
__device__ __forceinline__ __nv_bfloat16* qkv_dest(const QkvArgs& q, __nv_bfloat16* q_out, int m, int head, int pos) {
    if (head < q.H) return q_out + ((size_t)m * q.H + head) * q.hd;
    const int kvh = (head - q.H) % q.Hkv;
    __nv_bfloat16* pages = head < q.H + q.Hkv ? q.k_pages : q.v_pages;
    const int page = q.page_table[(size_t)q.slots[q.tok_seq[m]] * q.pt_stride + pos / q.page_size];
    return pages + (((size_t)page * q.Hkv + kvh) * q.page_size + pos % q.page_size) * q.hd;
}

// Elements j0 + 8 i .. j0 + 8 i + 7 of a head's first half (from a) and their partners in the second half (from b)
// of one row, rotated (heads of q and k, when there are tables) and packed as bfloat16.
__device__ __forceinline__ void rotate_pack(const uint32_t (&a)[32], const uint32_t (&b)[32], const float* cos_row,
                                            const float* sin_row, int j0, int i, uint4& lo, uint4& hi) {
    float x0[8], x1[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { x0[e] = __uint_as_float(a[8 * i + e]); x1[e] = __uint_as_float(b[8 * i + e]); }
    if (cos_row) {
#pragma unroll
        for (int e4 = 0; e4 < 2; ++e4) {
            const float4 c = reinterpret_cast<const float4*>(cos_row + j0)[2 * i + e4];
            const float4 sn = reinterpret_cast<const float4*>(sin_row + j0)[2 * i + e4];
            const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float y0 = x0[4 * e4 + e] * cc[e] - x1[4 * e4 + e] * ss[e];
                const float y1 = x0[4 * e4 + e] * ss[e] + x1[4 * e4 + e] * cc[e];
                x0[4 * e4 + e] = y0;
                x1[4 * e4 + e] = y1;
            }
        }
    }
    lo = make_uint4(pack2(x0[0], x0[1]), pack2(x0[2], x0[3]), pack2(x0[4], x0[5]), pack2(x0[6], x0[7]));
    hi = make_uint4(pack2(x1[0], x1[1]), pack2(x1[2], x1[3]), pack2(x1[4], x1[5]), pack2(x1[6], x1[7]));
}

// 32 elements j0 .. j0+31 of a head's first half (a) and their partners in the second half (b) of one row:
// rotated and stored at dst + j0 and dst + half + j0.
__device__ __forceinline__ void store_qkv_pair(const uint32_t (&a)[32], const uint32_t (&b)[32], __nv_bfloat16* dst,
                                               const float* cos_row, const float* sin_row, int j0, int half) {
    uint4* lo = reinterpret_cast<uint4*>(dst + j0);
    uint4* hi = reinterpret_cast<uint4*>(dst + half + j0);
#pragma unroll
    for (int i = 0; i < 4; ++i) rotate_pack(a, b, cos_row, sin_row, j0, i, lo[i], hi[i]);
}

// The q/k/v epilogue of one thread's row m: columns [0, bn) of its lane of the accumulator at `taddr` are whole
// heads starting at column n0 of W (bn is a multiple of hd); a head's halves are hd / 2 = 32 or 64 columns.
__device__ __forceinline__ void qkv_epilogue(uint32_t taddr, int bn, const QkvArgs& qkv, __nv_bfloat16* q_out, int m, int M,
                                             int n0, int N) {
    const int hd = qkv.hd, half = hd >> 1;
    const int pos = m < M ? qkv.tok_pos[m] : 0;
#pragma unroll 1
    for (int col = 0; col < bn && n0 + col < N; col += hd) {
        const int head = (n0 + col) / hd;
        const bool rotate = qkv.cos_t != nullptr && head < qkv.H + qkv.Hkv;
        __nv_bfloat16* row = m < M ? qkv_dest(qkv, q_out, m, head, pos) : nullptr;
#pragma unroll 1
        for (int j0 = 0; j0 < half; j0 += 32) {
            uint32_t a[32], b[32];
            ld32(taddr + col + j0, a);
            ld32(taddr + col + half + j0, b);
            wait_ld();
            if (m < M)
                store_qkv_pair(a, b, row, rotate ? qkv.cos_t + (size_t)pos * half : nullptr,
                               rotate ? qkv.sin_t + (size_t)pos * half : nullptr, j0, half);
        }
    }
}

// The same through shared memory, for a warp's 32 rows (this thread's row is m = y + lane): a head's rows are put
// into the warp's buffers as 128-byte pieces (head size 128: elements 0..63 in one buffer, 64..127 in the other;
// head size 64: a whole row in one buffer).  Query heads leave as TMA stores into q_out (map_q: [M, H hd]); rows
// of k and v go to their cache pages four rows per instruction, eight lanes writing a row's 128 contiguous bytes.
__device__ __forceinline__ void qkv_epilogue_staged(uint32_t taddr, int bn, const QkvArgs& qkv, const CUtensorMap* map_q,
                                                    uint8_t* bufs, int& which, int y, int M, int n0, int N, int lane) {
    const int hd = qkv.hd, half = hd >> 1;
    const int m = y + lane;
    const int pos = m < M ? qkv.tok_pos[m] : 0;
    const float* cos_row = qkv.cos_t ? qkv.cos_t + (size_t)pos * half : nullptr;
    const float* sin_row = qkv.cos_t ? qkv.sin_t + (size_t)pos * half : nullptr;
#pragma unroll 1
    for (int col = 0; col < bn && n0 + col < N; col += hd) {
        const int head = (n0 + col) / hd;
        const bool rotate = head < qkv.H + qkv.Hkv;
        uint8_t *lo_buf, *hi_buf;
        int hi_piece;                               // where the second half's pieces start in hi_buf
        if (hd == 128) {
            if (lane == 0) bulk_wait_read<0>();     // both buffers are used at once
            lo_buf = bufs; hi_buf = bufs + STAGE_BUF_BYTES; hi_piece = 0;
        } else {
            if (lane == 0) bulk_wait_read<1>();
            lo_buf = hi_buf = bufs + which * STAGE_BUF_BYTES; hi_piece = 4;
            which ^= 1;
        }
        __syncwarp();
#pragma unroll 1
        for (int j0 = 0; j0 < half; j0 += 32) {
            uint32_t a[32], b[32];
            ld32(taddr + col + j0, a);
            ld32(taddr + col + half + j0, b);
            wait_ld();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 lo, hi;
                rotate_pack(a, b, rotate ? cos_row : nullptr, rotate ? sin_row : nullptr, j0, i, lo, hi);
                *staged_at(lo_buf, lane, (j0 >> 3) + i) = lo;
                *staged_at(hi_buf, lane, hi_piece + (j0 >> 3) + i) = hi;
            }
        }
        if (head < qkv.H) {
            fence_async_shared();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(map_q, smem_u32(lo_buf), head * hd, y);
                if (hd == 128) tma_store_2d(map_q, smem_u32(hi_buf), head * hd + 64, y);
                bulk_commit();
            }
        } else {
            __syncwarp();
            const unsigned long long mine = m < M ? (unsigned long long)qkv_dest(qkv, nullptr, m, head, pos) : 0ull;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int r = it * 4 + (lane >> 3), piece = lane & 7;
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xffffffffu, mine, r));
                if (dst) {
                    *reinterpret_cast<uint4*>(dst + piece * 8) = *staged_at(lo_buf, r, piece);
                    if (hd == 128) *reinterpret_cast<uint4*>(dst + 64 + piece * 8) = *staged_at(hi_buf, r, piece);
                }
            }
            __syncwarp();           // all lanes have read the buffers before the next head fills them
        }
    }
}

// Host: whether an output of this epilogue at C (cols columns, for SwiGLU the halved count) can leave by TMA,
// and its tensor map (boxes of 32 rows x 128 bytes).
template <int EPI>
static inline bool staged_map(CUtensorMap* map, void* C, const void* residual, long rows, long cols) {
    const int elt = (EPI == EPI_F32 || EPI == EPI_RESID) ? 4 : 2;
    if (((uintptr_t)C & 15) || (cols * elt) % 16 != 0 || (EPI == EPI_RESID && C != residual)) return false;
    return make_map_out(map, C, elt, rows, cols, cols, 32) == LQ_OK;
}

}  // namespace tc
