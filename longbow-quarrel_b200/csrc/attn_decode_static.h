/* lq_attn_decode_static: split-KV decode attention for callers that cannot allocate.
 *
 * This entry point has no counterpart in the reference (23skdu/longbow-quarrel); it exists for
 * users of this library only.
 *
 * Who needs it.  lq_attn_decode wants two scratch buffers from its caller (the unnormalised
 * partial outputs of the key slices and their running maximum and sum).  Some callers cannot
 * provide them because they cannot call cudaMalloc where they stand: a host program that gave
 * out its whole device-memory budget at start-up and treats any later allocation as a fault;
 * a latency-bound loop that must not pay cudaMalloc's implicit synchronisation of the device,
 * or cannot recover if the allocation fails at that point; a plug-in or callback whose host
 * forbids allocator calls.  For them the scratch lives in this library itself, in a
 * file-scope device array, and the call allocates nothing: no cudaMalloc, no cudaFree, no
 * library routine that allocates (torch's included).
 *
 * The limit.  The array holds LQ_ATTN_STATIC_FLOATS floats (8 MiB).  Every GPU that loads the
 * library holds those 8 MiB from load until the process ends.  A call needs
 * T * H * n_splits * (head_dim + 2) floats plus one counter for each (token, kv head) and is
 * refused with LQ_STATIC_TOO_SMALL (-4), before anything is launched, when that is more;
 * lq_attn_decode_static_floats() gives the capacity.
 * With one slice (n_splits == 1) no scratch is used at all.
 *
 * Sizes the kernel does not take (a head size that is no multiple of 8 or above 128, heads that are no
 * multiple of the kv heads, a page size that is no multiple of 16, more than 32 slices, a q_stride that
 * is no multiple of 8) are refused with -2, likewise before anything is queued.
 *
 * Set-up.  The first call on a device asks the runtime for the array's device address
 * (cudaGetSymbolAddress, with that device current) and keeps it; the name of the array in
 * host code is only a handle, not an address the GPU can use.  Make that first call on each
 * device before any stream capture begins, like any other call that may initialise a module.
 * The array is the current device's, so `stream` must be a stream of the device that is current
 * when the call is made (the call does not check this).
 *
 * Sharing.  All calls on a device use the same array, and it keeps what the last call left in
 * it.  The partial outputs need no clearing: a call writes every element that it later reads
 * (a slice without keys writes "maximum -inf, sum 0").  The counters by which the last block of
 * a (token, kv head) knows that it is the last must start at zero: each call clears the ones
 * it uses with cudaMemsetAsync on its stream before the kernel.  Two calls that overlap on the GPU -- different
 * streams, or different host threads launching on different streams -- race on the array; keep
 * calls on one stream, or order them with events.
 *
 * Arguments and result are those of lq_attn_decode without part_o and part_ml:
 *   q          [T, q_stride] bfloat16 rows whose first H * head_dim elements are the query heads
 *   k_pages, v_pages, page_table, pt_stride, tok_pos, tok_seq, slots   the paged bfloat16 cache
 *   out        [T, H * head_dim] bfloat16
 * Returns 0 when the kernels were launched, -2 for sizes the kernel does not take, -4 when the
 * scratch is too small, a cudaError_t value if the runtime refused (set-up or launch).
 */
#pragma once
#include <cuda_runtime.h>

#define LQ_ATTN_STATIC_FLOATS (2 * 1024 * 1024)
#define LQ_STATIC_TOO_SMALL (-4)

#ifdef __cplusplus
extern "C" {
#endif

int lq_attn_decode_static(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                          const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                          const int* slots, void* out, int T, int H, int Hkv, int head_dim, int page_size,
                          float scale, int window, int n_splits, cudaStream_t stream);

long lq_attn_decode_static_floats(void);

#ifdef __cplusplus
}
#endif
