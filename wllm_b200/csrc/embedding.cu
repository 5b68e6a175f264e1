// Scaled embedding gather: out[n, :] = float(table[ids[n], :]) * scale, written to the
// 32-bit residual stream.  One block per token, 16-byte loads where the row allows.
// And the patch that lets a step start before the host has seen the previous step's tokens:
// ids[dst[i]] = sampled[src[i]], device to device.
#include "common.cuh"

__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ dst, const int* __restrict__ sampled,
                                    const int* __restrict__ src, int n) {
    pdl_begin();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[dst[i]] = sampled[src[i]];
}

WLLM_API int wllm_patch_tokens(int* ids, const int* dst, const int* sampled, const int* src, int n, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    return wllm_launch(patch_tokens_kernel, (n + 127) / 128, 128, 0, stream, ids, dst, sampled, src, n);
}

template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table, float scale,
                                    float* __restrict__ out, int H, int V) {
    pdl_begin();
    const int row = blockIdx.x;
    int id = ids[row];
    float* o = out + (size_t)row * H;
    if (id < 0 || id >= V) {  // the host checks ids; an id that slips through reads nothing
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = to_f32(src[c]) * scale;
}

WLLM_API int wllm_embed_gather(const int* ids, const void* table, int table_dtype, float scale, float* out,
                               int n, int H, int V, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || V <= 0) return WLLM_BAD_SIZE;
    const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
    if (table_dtype == WLLM_BF16)
        return wllm_launch(embed_gather_kernel<bf16>, n, threads, 0, stream, ids, (const bf16*)table, scale, out, H, V);
    if (table_dtype == WLLM_F32)
        return wllm_launch(embed_gather_kernel<float>, n, threads, 0, stream, ids, (const float*)table, scale, out, H, V);
    return WLLM_BAD_DTYPE;
}
