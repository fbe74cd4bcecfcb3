/* Split-KV decode attention without any allocation.
 *
 * This entry point has no counterpart in the reference (pochenai/llm-inference-lab); it is an
 * addition of this library, built from attention_tc.cu for one head size (-DLAB_HEAD_DIM).
 *
 * Who needs it: code that runs where device memory cannot be allocated.  Examples are a
 * plugin inside a host application that owns the whole device heap and forbids cudaMalloc,
 * a callback during which the host forbids allocation, a real-time loop
 * that may not block on the allocator, and a caller that has only raw device pointers and no
 * tensor library.  Such callers still pass the inputs and the output; what they cannot supply
 * is the scratch for the per-split partial results, so that scratch is a fixed array inside
 * the library's device image.
 *
 * Limits and rules:
 *  - requests * n_q * splits * (head size + 2) must not exceed
 *    lab_attention_decode_noalloc_max_floats() (1,048,576 floats = 4 MiB); larger calls return
 *    a negative code that lab_attention_decode_noalloc_strerror() explains.  Every GPU on
 *    which the library is loaded holds those 4 MiB until the process exits.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress);
 *    make that first call outside any stream capture, with the device current.
 *  - All calls share the one array.  It keeps what the last call left; the kernels write every
 *    slot before reading it, so nothing needs clearing.  Two calls that overlap on the GPU
 *    (different streams, no ordering between them) race on it: order them.
 *  - It calls no cudaMalloc, cudaFree or allocating library routine.  Arguments are those of
 *    lab_attention_decode without the scratch pointer; results are the same.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long lab_attention_decode_noalloc_max_floats(void);
const char* lab_attention_decode_noalloc_strerror(int code);

/* out: [rows, out_stride] bf16; q: [rows, q_stride] bf16 (row of request b at q_start[b]);
 * cache_k / cache_v: [num_pages, n_kv, page_size, head size] bf16; q_start: [requests + 1];
 * kv_len: [requests]; block_table: [requests, max_blocks]; only requests that bring exactly one
 * row are served.  Returns 0, a CUDA error code, or a negative code (see strerror above). */
int lab_attention_decode_noalloc(void* out, int out_stride, const void* q, int q_stride, const void* cache_k,
                                 const void* cache_v, const int* q_start, const int* kv_len, const int* block_table,
                                 int max_blocks, int requests, int n_q, int n_kv, int page_size, int num_pages,
                                 int window, float scale, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
