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

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                     const int* __restrict__ slots, const float* __restrict__ inv_freq,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd,
                                     int rot_dim, int page_size) {
    const int t = blockIdx.x;
    T* row = qkv + (size_t)t * row_stride;
    const float pos = (float)positions[t];
    const int slot = slots ? slots[t] : -1;
    const int half = rot_dim >> 1;
    size_t page_base = 0;
    int off = 0;
    if (slot >= 0) {
        page_base = (size_t)(slot / page_size) * nkv;
        off = slot % page_size;
    }
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[j], &s, &c);
        for (int h = 0; h < nq + nkv; ++h) {
            T* x = row + (size_t)h * hd;
            const float x1 = to_f32(x[j]), x2 = to_f32(x[j + half]);
            const T y1 = from_f32<T>(x1 * c - x2 * s), y2 = from_f32<T>(x2 * c + x1 * s);
            if (h < nq) {
                x[j] = y1;
                x[j + half] = y2;
            } else if (slot >= 0) {
                T* dst = k_pages + ((page_base + (h - nq)) * page_size + off) * hd;
                dst[j] = y1;
                dst[j + half] = y2;
            }
        }
    }
    if (slot < 0) return;
    // unrotated tail of the keys
    for (int idx = threadIdx.x; idx < nkv * (hd - rot_dim); idx += blockDim.x) {
        const int h = idx / (hd - rot_dim), c = rot_dim + idx % (hd - rot_dim);
        k_pages[((page_base + h) * page_size + off) * hd + c] = row[(size_t)(nq + h) * hd + c];
    }
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        const int h = idx / hd, c = idx % hd;
        v_pages[((page_base + h) * page_size + off) * hd + c] = row[(size_t)(nq + nkv + h) * hd + c];
    }
}

WLLM_API int wllm_rope_kv_write(void* qkv, int dtype, int row_stride, const int* positions, const int* slots,
                                const float* inv_freq, void* k_pages, void* v_pages, int n, int nq, int nkv, int hd,
                                int rot_dim, int page_size, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (hd <= 0 || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || page_size <= 0 || nq <= 0 || nkv <= 0) return WLLM_BAD_SIZE;
    const int threads = hd >= 256 ? 128 : (hd >= 128 ? 64 : 32);
    if (dtype == WLLM_BF16)
        rope_kv_write_kernel<bf16><<<n, threads, 0, stream>>>((bf16*)qkv, row_stride, positions, slots, inv_freq,
                                                               (bf16*)k_pages, (bf16*)v_pages, nq, nkv, hd, rot_dim, page_size);
    else if (dtype == WLLM_F32)
        rope_kv_write_kernel<float><<<n, threads, 0, stream>>>((float*)qkv, row_stride, positions, slots, inv_freq,
                                                                (float*)k_pages, (float*)v_pages, nq, nkv, hd, rot_dim, page_size);
    else
        return WLLM_BAD_DTYPE;
    return wllm_launch_status();
}
