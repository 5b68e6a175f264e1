// The allocation-free variant of the split-key decode attention: see attention_decode_static.h.
// Compiled per head size like attention_mma.cu (-DHEAD_DIM=...), whose kernels it reuses unchanged.
#include "attention_mma.cu"
#include "attention_decode_static.h"

#include <mutex>

// Partial results of the key splits.  In host code this name is only a handle for the
// symbol, not a device address: the address is looked up once per device below.
static __device__ __align__(256) float g_static_scratch[WLLM_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
static float* g_scratch_addr[MAX_DEVICES];
static std::mutex g_setup_mutex;

// Device address of the array on the current device; looked up on the first call per device.
static int static_scratch(float** addr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return WLLM_SETUP_FAILED;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) return WLLM_SETUP_FAILED;
        g_scratch_addr[dev] = static_cast<float*>(p);
    }
    *addr = g_scratch_addr[dev];
    return WLLM_OK;
}

WLLM_API long long wllm_attention_mma_decode_static_needs(int requests, int nq, int max_splits) {
    return wllm_attention_mma_scratch_floats(requests, nq, max_splits);
}

WLLM_API int wllm_attention_mma_decode_static(const void* q, int q_stride, void* out, int out_stride,
                                              const void* k_pages, const void* v_pages, long long pool_pages,
                                              const int* req_q_start, const int* req_q_len, const int* req_ctx_len,
                                              const int* block_table, int max_pages, int requests, int nq, int nkv,
                                              int page_size, int window, float scale, int split_keys, int max_splits,
                                              int* status, cudaStream_t stream) {
    if (requests <= 0) return WLLM_OK;
    if (nq <= 0 || max_splits < 1) return WLLM_BAD_SIZE;
    if (wllm_attention_mma_scratch_floats(requests, nq, max_splits) > (long long)WLLM_STATIC_SCRATCH_FLOATS)
        return WLLM_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    const int rc = static_scratch(&scratch);
    if (rc != WLLM_OK) return rc;
    return wllm_attention_mma_decode(q, q_stride, out, out_stride, k_pages, v_pages, pool_pages, req_q_start, req_q_len,
                                     req_ctx_len, block_table, max_pages, requests, nq, nkv, page_size, window, scale,
                                     split_keys, max_splits, scratch, status, stream);
}
