/* Split-key decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project; it exists for hosts
 * that embed the kernels but are not allowed to ask the CUDA allocator for anything:
 * a program whose device memory is owned and handed out entirely by someone else, a
 * plug-in called from inside another framework's callback where cudaMalloc is
 * forbidden, or a latency-bound loop that cannot afford an allocation (cudaMalloc may
 * synchronise the device and has no time bound).  The engine itself does not use it;
 * it passes scratch from its own arena to wllm_attention_mma_decode.
 *
 * Same arguments and results as wllm_attention_mma_decode (see attention_mma.cu), but
 * without the `scratch` pointer: the partial results of the key splits live in a
 * file-scope device array of WLLM_STATIC_SCRATCH_FLOATS floats (4 MiB) that every GPU
 * holding the library keeps until the process exits.
 *
 *   - It calls no cudaMalloc, cudaFree or allocating library routine.
 *   - requests * nq * max_splits * (head_dim + 2) must not exceed
 *     WLLM_STATIC_SCRATCH_FLOATS; otherwise nothing is launched and status 4
 *     (WLLM_SCRATCH_TOO_SMALL) is returned.
 *   - The first call on a device looks up the array's device address (with that
 *     device current) and remembers it; make that first call before any stream
 *     capture begins.  A failed look-up returns status 5 (WLLM_SETUP_FAILED).
 *   - All calls share the one array, and it keeps the last call's contents.  Nothing in
 *     it has to start at zero: every split writes its slot before the merge reads it.
 *     Two calls that overlap on the GPU (different streams, no ordering between them)
 *     race on the array; order them.
 *   - split_keys and max_splits are the caller's plan: every request is cut into parts of split_keys keys,
 *     at most max_splits of them.  A request whose context is longer than split_keys * max_splits is still
 *     computed in full (its parts are widened to fit max_splits), only more slowly than planned.
 *   - Returns 0 once the kernels are enqueued on `stream`, or a status code as the
 *     other entry points do (1000 + cudaError_t for a failed launch).
 */
#pragma once
#include <cuda_runtime.h>

#define WLLM_STATIC_SCRATCH_FLOATS (1 << 20)
#define WLLM_SCRATCH_TOO_SMALL 4
#define WLLM_SETUP_FAILED 5

#ifdef __cplusplus
extern "C" {
#endif

int wllm_attention_mma_decode_static(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                     const void* v_pages, long long pool_pages, const int* req_q_start,
                                     const int* req_q_len, const int* req_ctx_len, const int* block_table,
                                     int max_pages, int requests, int nq, int nkv, int page_size, int window,
                                     float scale, int split_keys, int max_splits, int* status, cudaStream_t stream);

/* Floats of the static array that a call with these sizes would use. */
long long wllm_attention_mma_decode_static_needs(int requests, int nq, int max_splits);

#ifdef __cplusplus
}
#endif
