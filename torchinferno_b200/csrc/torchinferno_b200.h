/* C interface of libtorchinferno_b200.so that is meant for callers outside the Python package.
 *
 * All functions return 0 on success, a positive cudaError_t when a CUDA call failed, or a negative
 * code when the arguments are refused (-2: a size the kernel does not take, -3: alignment,
 * -5: null or inconsistent arguments, -7: more scratch needed than the built-in array holds).
 */
#ifndef TORCHINFERNO_B200_H
#define TORCHINFERNO_B200_H

#include <cuda_runtime_api.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Paged decode attention (bf16, head_dim a multiple of 16 up to 128) that allocates nothing.
 *
 * This entry point has no counterpart in the reference project.  It exists for hosts that cannot
 * allocate device memory when they call: code running under another framework's fixed memory plan,
 * a latency-critical loop that may not enter the allocator, or a plug-in whose host forbids
 * allocation after start-up.  The partial results of the context splits are kept in a 16 MiB array
 * that is part of the library's device image (held by every GPU that loads the library, until exit).
 *
 *   q, out        [n_entries tokens][heads * head_dim] bf16 (entries that bring one token each)
 *   pool          one layer's pages [num_pages][2][kv_heads][page_size][head_dim] bf16
 *   q_start       [n_entries + 1] first token row of each entry; kv_start [n_entries] position of that
 *                 token; slots [n_entries] row of block_table; block_table [rows][table_stride] page ids
 *   num_splits, chunk   the context is cut into num_splits parts of chunk keys (a multiple of 64)
 *   max_kv_len    the longest context of the batch (the largest kv_start + 1); num_splits * chunk must
 *                 cover it, or the call is refused with -2 (keys beyond the parts would be left out)
 *
 * A call needs n_entries * heads * num_splits * (head_dim + 2) floats of the array (none when
 * num_splits is 1); more than tib_decode_attention_noalloc_capacity() is refused with -7.
 * The first call on a device resolves the array's device address; make it before any stream
 * capture.  All calls share the array and it keeps the last call's contents; nothing needs
 * clearing, but calls that overlap on the GPU race on it: order them on a stream or with events.
 * It calls no cudaMalloc, cudaFree or allocating library routine.
 */
int tib_decode_attention_noalloc(const void* q, const void* pool, void* out, const int* q_start,
                                 const int* kv_start, const int* slots, const int* block_table,
                                 int table_stride, int n_entries, int heads, int kv_heads, int head_dim,
                                 int page_size, int64_t page_stride, int num_pages, int window, float scale,
                                 int num_splits, int chunk, int max_kv_len, cudaStream_t stream);

/* Floats of the built-in array a call would use, and how many it holds. */
long long tib_decode_attention_noalloc_need(int n_entries, int heads, int head_dim, int num_splits);
long long tib_decode_attention_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
#endif
