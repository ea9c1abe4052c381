/* pi_attention_mma_noalloc: the paged tensor-core attention (attention_mma.cu) for callers that cannot
 * allocate device memory.
 *
 * This entry point has no counterpart in the reference engine; it exists for hosts of this library that
 * are not allowed to call cudaMalloc (or any allocator that may end up there) around a launch: code that
 * runs inside another framework's memory plan, a process whose device memory was handed out in full at
 * start-up, or a caller on a path where an allocation could block or fail after the point of no return.
 * Such callers already own the inputs and the output; the only other memory the kernel needs is the
 * scratch in which the split decode attention keeps its per-range partial results.  Here that scratch is a
 * fixed array inside the library's device image instead of a buffer passed in.
 *
 * What that means for the caller:
 *  - Limit.  The array is PI_NOALLOC_SCRATCH_BYTES (8 MiB).  A call needs
 *        tokens * query_heads * max_splits * (head_size + 2) * 4   bytes
 *    and is refused (return -1, text from pi_last_error()) when that is more.  Every GPU on which the
 *    library is loaded holds the array until the process exits, whether or not this entry is used.
 *    The attention library is built once per head size (libpi_attention_mma_d64, ..._d128, ...); each of
 *    those builds carries an array of its own, so a process that loads three of them holds 24 MiB per GPU.
 *  - No allocation.  The call performs no cudaMalloc, cudaFree or other allocating routine.
 *  - First call.  The first call on each device asks the runtime for the array's device address
 *    (cudaGetSymbolAddress, with that device current).  Make that first call outside any stream capture.
 *  - Sharing.  All calls on a device use the same array and it keeps what the last call left.  Nothing in
 *    it needs clearing between calls (each entry is written before it is read), but two calls that can
 *    run at the same time on one GPU - different streams, or different threads - race on it.  Serialise
 *    them, e.g. by launching on one stream.
 *  - Everything else (arguments, results, supported sizes) is exactly pi_attention_mma's; the two scratch
 *    pointers are simply absent.  One difference: has_prompt and has_decode must be 0 or 1 here.
 *    pi_attention_mma's has_decode = 2 ("the partial results are already in the scratch, only merge them")
 *    is refused, because no other kernel can have written this library's private array.
 */
#pragma once
#include <cuda_runtime.h>

#define PI_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

/* bytes of the fixed scratch array (PI_NOALLOC_SCRATCH_BYTES) */
int pi_attention_noalloc_scratch_bytes(void);

/* returns 0, a cudaError_t (> 0), or -1 for refused arguments */
int pi_attention_mma_noalloc(const void* q, int q_stride, const void* kcache, const void* vcache,
                             const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                             const int* seg_start, const int* seg_len, const int* token_seg, void* out, int max_splits,
                             int split_keys, int num_tokens, int num_segments, int max_seg_len, int has_prompt,
                             int has_decode, int nq, int nkv, int page_size, int window, float scale,
                             cudaStream_t stream);

#ifdef __cplusplus
}
#endif
