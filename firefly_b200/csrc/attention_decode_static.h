/* Split-KV decode attention that allocates nothing.
 *
 * This entry point has no counterpart in the reference engine; it exists for hosts
 * that embed these kernels through the C interface and cannot allocate device
 * memory at call time: a server that handed all free device memory to its own
 * cache pool at start-up (a cudaMalloc would simply fail), or a latency-critical
 * loop in which the device-wide synchronisation that cudaMalloc / cudaFree imply
 * is not acceptable.  The regular entry point, ff_attn_decode, takes its scratch
 * memory (the per-split partial outputs) from the caller; this one keeps it in a
 * fixed array inside the library instead.
 *
 * Limits and rules
 *  - n_seqs * nq * num_splits must not exceed FF_ATTN_STATIC_MAX_PARTIALS; a larger
 *    request is refused with FF_ATTN_STATIC_TOO_LARGE and a line on stderr.
 *  - The array (FF_ATTN_STATIC_MAX_PARTIALS * (head_dim + 2) floats, about 2 MB at
 *    head size 128) is part of the loaded library: every GPU that loads the
 *    library holds it until the process exits.
 *  - The first call on a device looks up the array's device address and raises
 *    the kernels' shared-memory limit.  Make that first call before any stream
 *    capture is begun.
 *  - All calls share the one array, and it keeps the previous call's contents.
 *    Nothing in it has to start at zero: the decode kernel writes every
 *    (sequence, head, split) entry, empty splits included, before the joining
 *    kernel reads it.  Two calls that overlap on the GPU (different streams with no
 *    ordering between them) race on the array; order them.
 *  - No cudaMalloc, cudaFree or allocating library routine is called.
 *
 * Arguments are those of ff_attn_decode without the two scratch pointers:
 * bfloat16 q [tokens, q_stride], cache pages [num_blocks][2][nkv][block_size][D],
 * int32 block_table [n_seqs, max_blocks], cu_q [n_seqs+1], ctx_lens [n_seqs],
 * bfloat16 out [tokens, out_stride]; one query token per sequence.
 * Returns 0, a positive cudaError_t, or a negative FF_* code.
 */
#pragma once
#include <cuda_runtime.h>

#define FF_ATTN_STATIC_MAX_PARTIALS 4096
#define FF_ATTN_STATIC_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C"
#endif
int ff_attn_decode_static(const void* q, int q_stride, const void* cache, const int* block_table,
                          int max_blocks, const int* cu_q, const int* ctx_lens, int n_seqs, void* out,
                          int out_stride, int nq, int nkv, int block_size, int num_blocks, float scale,
                          int window, int num_splits, cudaStream_t stream);
