/* Decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project; it exists for hosts
 * that embed this library under rules the rest of the library does not have to obey.
 *
 * Who needs it: a program that hands the whole GPU to its own memory pool at start-up
 * (a later cudaMalloc would fail or tear a hole in that pool); a control loop with a
 * hard latency bound, for which the device-wide synchronisation hidden in cudaMalloc and
 * cudaFree is not acceptable; a plug-in whose host forbids any allocation after
 * initialisation.  The ordinary entry point, ek_attention_decode_bf16, asks such a caller
 * for two scratch buffers whenever the keys are split over several blocks.  This variant
 * asks for nothing: its scratch is a fixed array that is part of the library image.
 *
 * Contract
 *  - Same arguments and the same result as ek_attention_decode_bf16 without the two
 *    scratch pointers.  The caller still owns and passes every input and the output.
 *  - It calls no cudaMalloc, cudaFree or other allocating routine, ever.
 *  - The scratch array holds EK_NOALLOC_SCRATCH_FLOATS 32-bit values (8 MiB).  Every GPU
 *    that loads the library carries that array until the process exits.  A call needs
 *        n_tokens * n_q_heads * n_splits * (head_dim + 2)
 *    values when n_splits > 1 and none otherwise.  A call that needs more is refused:
 *    nothing is launched, the output is left as it was, one line naming both numbers goes
 *    to stderr, and EK_NOALLOC_TOO_LARGE is returned.  Use fewer splits, fewer tokens per
 *    call, or the ordinary entry point.
 *  - The first call on each device looks up the device address of the array (with that
 *    device current).  Make that first call outside of any stream capture.
 *  - All calls share the one array, and it keeps whatever the previous call left.  The
 *    kernels write every partial result they later read, so nothing has to be cleared
 *    between calls.  Two calls whose kernels can overlap on the GPU (different streams
 *    without an ordering between them) race on the array and give wrong results: keep
 *    the calls of one device in stream order.
 *
 * Returns 0, a cudaError_t value, -2 for sizes the kernel does not take (see
 * ek_attention_decode_bf16), or EK_NOALLOC_TOO_LARGE.
 */
#pragma once
#include <cuda_runtime.h>

#define EK_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define EK_NOALLOC_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C" {
#endif

int ek_attention_decode_bf16_noalloc(void* out, const void* q, int q_row_stride,
                                     const int* positions, const int* token_slot,
                                     const void* k_pages, const void* v_pages,
                                     const int* block_table, int table_stride, int n_tokens,
                                     int n_q_heads, int n_kv_heads, int head_dim, float scale,
                                     int window, int n_splits, int keys_per_split,
                                     cudaStream_t stream);

#ifdef __cplusplus
}
#endif
