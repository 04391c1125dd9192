/* Split-KV paged decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference.  It exists for embedders of this library that
 * cannot call cudaMalloc where they call us: a host process that has handed the whole GPU to its own pool
 * allocator, a plugin running inside another runtime's allocation-free callback, or a replica that is kept
 * "parked" with all of its memory already promised to weights and the KV pool.  The ordinary entry point
 * (blitz_attn_decode) needs a caller-provided workspace for the partial results of the KV splits; this one
 * keeps that workspace inside the library, in a fixed array in device global memory that every GPU loading
 * the library carries until the process exits.
 *
 * Limits and rules
 *   - The built-in scratch is BLITZ_ATTN_NOALLOC_SCRATCH_BYTES (16 MiB).  A call needs
 *       batch * q_heads * num_splits * (head_dim + 1) * 4 bytes
 *     when num_splits > 1 and nothing otherwise; a larger request is refused with
 *     BLITZ_ATTN_NOALLOC_TOO_LARGE and launches nothing.
 *   - Nothing in the scratch has to start at zero: every (sequence, head, split) slot a call reads is
 *     written by the same call first.  The contents of the previous call stay there otherwise.
 *   - All calls on a device share the one array.  Two calls whose kernels can overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it; issue them on one stream or order them yourself.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that
 *     device current) and raises the kernel's shared-memory limit.  Make that first call outside any stream
 *     capture; later calls do no set-up work.
 *     Host threads may make that first call concurrently: the set-up runs once per device under a lock.
 *   - A process may use devices 0..63 with this entry point; on a higher device ordinal it returns -1.
 *   - No cudaMalloc, cudaFree, or allocating library routine is called, on any call.
 *
 * Arguments are those of blitz_attn_decode without the workspace pointer:
 *   q [batch, >= q_heads*head_dim] (row pitch q_stride elements), kv_layer [max_pages][2][page_size][kv_heads]
 *   [head_dim], CSR page table (indices, indptr[batch+1], last_page_len[batch]), out [batch, q_heads*head_dim]
 *   (row pitch out_stride), dtype 0 = fp16 / 1 = bf16, status = optional device int that receives a non-zero
 *   code if a bounded wait or a page-id check fails.
 * Returns 0, a cudaError_t value, -1 for unsupported shapes, -2 if the TMA descriptor encoder is unavailable,
 * or BLITZ_ATTN_NOALLOC_TOO_LARGE.
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define BLITZ_ATTN_NOALLOC_SCRATCH_BYTES (16u << 20)
#define BLITZ_ATTN_NOALLOC_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C" {
#endif

int blitz_attn_decode_noalloc(const void* q, int64_t q_stride, const void* kv_layer, const int32_t* indices,
                              const int32_t* indptr, const int32_t* last_page_len, void* out, int64_t out_stride,
                              int batch, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages,
                              int num_splits, float sm_scale, int* status, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
