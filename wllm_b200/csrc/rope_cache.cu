// Rotary position encoding of the query and key heads of a fused q|k|v row, and the write of the
// rotated keys and the values into the pages of the cache.
//
//   angle = float(position) * inv_freq[j],  j < rot_dim/2        (32-bit, sinf/cosf)
//   y[j]         = x[j] * cos - x[j + rot/2] * sin
//   y[j + rot/2] = x[j + rot/2] * cos + x[j] * sin                (pairs j, j + rot/2)
// Dimensions from rot_dim up to head_dim pass through unrotated.  The rotated queries go to `q_out`
// [n, nq * hd].  The input row may come as `in_splits` partial sums (slabs `in_split_stride` elements
// apart, as the split-K matrix product leaves them), which are added in slab order first.  A token
// whose slot is negative writes nothing to the cache (a layer that reads another layer's cache).
//
// Page layout: [page][kv_head][slot_in_page][head_dim]; `slots[n]` is page * page_size + slot_in_page.
#include "common.cuh"

// grid (token, head): head < nq rotates a query head into q_out, nq <= head < nq + nkv rotates a key head
// into its page, the rest copy a value head into its page.
template <typename TI, typename TO>
__global__ void rope_kv_write_kernel(const TI* __restrict__ qkv, int row_stride, int in_splits, size_t in_split_stride,
                                     TO* __restrict__ q_out, int q_stride, const int* __restrict__ positions,
                                     const int* __restrict__ slots, const float* __restrict__ inv_freq,
                                     TO* __restrict__ k_pages, TO* __restrict__ v_pages, int nq, int nkv, int hd,
                                     int rot_dim, int page_size) {
    pdl_begin();
    const int t = blockIdx.x, h = blockIdx.y;
    const TI* x = qkv + (size_t)t * row_stride + (size_t)h * hd;
    const int slot = slots ? slots[t] : -1;
    TO* dst;
    if (h < nq) {
        dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
    } else {
        if (slot < 0) return;
        const int kvh = h < nq + nkv ? h - nq : h - nq - nkv;
        TO* pages = h < nq + nkv ? k_pages : v_pages;
        dst = pages + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * hd;
    }
    auto in = [&](int c) {     // part 0 + part 1 + ... in order; sixteen loads are in flight at a time
        if (in_splits == 1) return to_f32(x[c]);
        float v = 0.f;
        for (int sp = 0; sp < in_splits; sp += 16) {
            float part[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) part[u] = sp + u < in_splits ? to_f32(x[(size_t)(sp + u) * in_split_stride + c]) : 0.f;
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (sp + u < in_splits) v = (sp + u == 0) ? part[u] : v + part[u];
        }
        return v;
    };
    if (h >= nq + nkv) {
        for (int c = threadIdx.x; c < hd; c += blockDim.x) dst[c] = from_f32<TO>(in(c));
        return;
    }
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[j], &s, &c);
        const float x1 = in(j), x2 = in(j + half);
        dst[j] = from_f32<TO>(x1 * c - x2 * s);
        dst[j + half] = from_f32<TO>(x2 * c + x1 * s);
    }
    for (int c = rot_dim + threadIdx.x; c < hd; c += blockDim.x) dst[c] = from_f32<TO>(in(c));
}

WLLM_API int wllm_rope_kv_write(const void* qkv, int in_dtype, int row_stride, int in_splits, long long in_split_stride,
                                void* q_out, int out_dtype, int q_stride, const int* positions, const int* slots,
                                const float* inv_freq, void* k_pages, void* v_pages, int n, int nq, int nkv, int hd,
                                int rot_dim, int page_size, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (hd <= 0 || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || page_size <= 0 || nq <= 0 || nkv <= 0 || in_splits < 1)
        return WLLM_BAD_SIZE;
    const int threads = hd >= 256 ? 128 : (hd >= 128 ? 64 : 32);
    const dim3 grid(n, nq + 2 * nkv);
#define GO(TI, TO) wllm_launch(rope_kv_write_kernel<TI, TO>, grid, threads, 0, stream, (const TI*)qkv, row_stride, in_splits, \
        (size_t)in_split_stride, (TO*)q_out, q_stride, positions, slots, inv_freq, (TO*)k_pages, (TO*)v_pages, nq, nkv, hd, \
        rot_dim, page_size)
    if (in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16) return GO(bf16, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_BF16) return GO(float, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_F32) return GO(float, float);
#undef GO
    return WLLM_BAD_DTYPE;
}
