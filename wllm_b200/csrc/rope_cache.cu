// Rotary position encoding of the query and key heads of a fused q|k|v row, and the
// write of the rotated keys and the values into the pages of the cache.
//
//   angle = float(position) * inv_freq[j],  j < rot_dim/2        (32-bit, sinf/cosf)
//   y[j]         = x[j] * cos - x[j + rot/2] * sin
//   y[j + rot/2] = x[j + rot/2] * cos + x[j] * sin                (pairs j, j + rot/2)
// Dimensions from rot_dim up to head_dim pass through unrotated.  Queries are
// rotated in place.  A token whose slot is negative writes nothing to the cache
// (a layer that reads another layer's cache).
//
// Page layout: [page][kv_head][slot_in_page][head_dim]; `slots[n]` is
// page * page_size + slot_in_page.
#include "common.cuh"

// grid (token, head): head < nq rotates a query head in place, nq <= head < nq + nkv rotates a key head
// into its page, the rest copy a value head into its page.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                     const int* __restrict__ slots, const float* __restrict__ inv_freq,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd,
                                     int rot_dim, int page_size) {
    const int t = blockIdx.x, h = blockIdx.y;
    T* x = qkv + (size_t)t * row_stride + (size_t)h * hd;
    const int slot = slots ? slots[t] : -1;
    T* dst = nullptr;
    if (h >= nq) {
        if (slot < 0) return;
        const int kvh = h < nq + nkv ? h - nq : h - nq - nkv;
        T* pages = h < nq + nkv ? k_pages : v_pages;
        dst = pages + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * hd;
    }
    if (h >= nq + nkv) {
        for (int c = threadIdx.x; c < hd; c += blockDim.x) dst[c] = x[c];
        return;
    }
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[j], &s, &c);
        const float x1 = to_f32(x[j]), x2 = to_f32(x[j + half]);
        const T y1 = from_f32<T>(x1 * c - x2 * s), y2 = from_f32<T>(x2 * c + x1 * s);
        if (dst) { dst[j] = y1; dst[j + half] = y2; }
        else { x[j] = y1; x[j + half] = y2; }
    }
    if (dst)
        for (int c = rot_dim + threadIdx.x; c < hd; c += blockDim.x) dst[c] = x[c];
}

WLLM_API int wllm_rope_kv_write(void* qkv, int dtype, int row_stride, const int* positions, const int* slots,
                                const float* inv_freq, void* k_pages, void* v_pages, int n, int nq, int nkv, int hd,
                                int rot_dim, int page_size, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (hd <= 0 || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || page_size <= 0 || nq <= 0 || nkv <= 0) return WLLM_BAD_SIZE;
    const int threads = hd >= 256 ? 128 : (hd >= 128 ? 64 : 32);
    const dim3 grid(n, nq + 2 * nkv);
    if (dtype == WLLM_BF16)
        rope_kv_write_kernel<bf16><<<grid, threads, 0, stream>>>((bf16*)qkv, row_stride, positions, slots, inv_freq,
                                                               (bf16*)k_pages, (bf16*)v_pages, nq, nkv, hd, rot_dim, page_size);
    else if (dtype == WLLM_F32)
        rope_kv_write_kernel<float><<<grid, threads, 0, stream>>>((float*)qkv, row_stride, positions, slots, inv_freq,
                                                                (float*)k_pages, (float*)v_pages, nq, nkv, hd, rot_dim, page_size);
    else
        return WLLM_BAD_DTYPE;
    return wllm_launch_status();
}
