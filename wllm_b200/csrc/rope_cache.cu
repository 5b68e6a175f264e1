// Rotary position encoding of the query and key heads of a fused q|k|v row, and the write of the
// rotated keys and the values into the pages of the cache.
//
//   angle = float(position) * inv_freq[j],  j < rot_dim/2        (32-bit, sinf/cosf)
//   y[j]         = x[j] * cos - x[j + rot/2] * sin
//   y[j + rot/2] = x[j + rot/2] * cos + x[j] * sin                (pairs j, j + rot/2)
// or, with `interleaved`, the same rotation of the pairs (2j, 2j + 1).
// Dimensions from rot_dim up to head_dim pass through unrotated.  The rotated queries go to `q_out`
// [n, nq * hd].  The input row may come as `in_splits` partial sums (slabs `in_split_stride` elements
// apart, as the split-K matrix product leaves them), which are added in slab order first.  A token
// whose slot is negative writes nothing to the cache (a layer that reads another layer's cache).
//
// Page layout: [page][kv_head][slot_in_page][head_dim]; `slots[n]` is page * page_size + slot_in_page.
#include "common.cuh"

// Two launch shapes.  Fewer than 1,024 tokens (a decode step, a short prompt): grid (token, head), so that the heads of a token run on
// different SMs; head < nq rotates a query head into q_out, nq <= head < nq + nkv rotates a key head into
// its page, the rest copy a value head into its page.  Many tokens: one CTA a token (ALL_HEADS), which
// computes the sines and cosines of the token's position once and walks the heads with them.
// Positions, slots and frequencies are written by no kernel of the step: the angles are worked out before
// the kernel waits for the product it rotates.
template <typename TI, typename TO, bool ALL_HEADS>
__global__ void rope_kv_write_kernel(const TI* __restrict__ qkv, int row_stride, int in_splits, size_t in_split_stride,
                                     TO* __restrict__ q_out, int q_stride, const int* __restrict__ positions,
                                     const int* __restrict__ slots, const float* __restrict__ inv_freq,
                                     TO* __restrict__ k_pages, TO* __restrict__ v_pages, int nq, int nkv, int hd,
                                     int rot_dim, int page_size, int interleaved) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    // the angle of this thread's first pair (all of them when the block is as wide as half the rotary size)
    float s0 = 0.f, c0 = 1.f;
    if ((int)threadIdx.x < half) sincosf(pos * inv_freq[threadIdx.x], &s0, &c0);
    pdl_wait();
    const int h_lo = ALL_HEADS ? 0 : blockIdx.y, h_hi = ALL_HEADS ? nq + 2 * nkv : blockIdx.y + 1;
    for (int h = h_lo; h < h_hi; ++h) {
        const TI* x = qkv + (size_t)t * row_stride + (size_t)h * hd;
        TO* dst;
        if (h < nq) {
            dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
        } else {
            if (slot < 0) break;
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
            continue;
        }
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float sn = s0, cs = c0;
            if (j != (int)threadIdx.x) sincosf(pos * inv_freq[j], &sn, &cs);
            const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
            const float x1 = in(ia), x2 = in(ib);
            float y1, y2;
            rotate_pair(x1, x2, sn, cs, y1, y2);
            dst[ia] = from_f32<TO>(y1);
            dst[ib] = from_f32<TO>(y2);
        }
        for (int c = rot_dim + threadIdx.x; c < hd; c += blockDim.x) dst[c] = from_f32<TO>(in(c));
    }
}

// Many tokens, bfloat16 in and out, one input tensor, head size and half the rotary size in steps of 8: one
// CTA a token; the token's sines and cosines go to shared memory once; every thread then takes eight
// neighbouring pairs of one head with 16-byte loads and stores, so that a block of 128 threads has the heads
// of a Gemma-2B token in flight at once.  The arithmetic per element is that of the kernel above.
__global__ void rope_kv_write_rows_kernel(const bf16* __restrict__ qkv, int row_stride, bf16* __restrict__ q_out, int q_stride,
                                          const int* __restrict__ positions, const int* __restrict__ slots,
                                          const float* __restrict__ inv_freq, bf16* __restrict__ k_pages,
                                          bf16* __restrict__ v_pages, int nq, int nkv, int hd, int rot_dim, int page_size) {
    extern __shared__ float sc[];            // [half] sines, [half] cosines
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sc[j], &sc[half + j]);
    __syncthreads();
    pdl_wait();
    const bf16* row = qkv + (size_t)t * row_stride;
    auto dst_of = [&](int h) -> bf16* {
        if (h < nq) return q_out + (size_t)t * q_stride + (size_t)h * hd;
        const int kvh = h < nq + nkv ? h - nq : h - nq - nkv;
        bf16* pages = h < nq + nkv ? k_pages : v_pages;
        return pages + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * hd;
    };
    const int heads = slot < 0 ? nq : nq + 2 * nkv;
    // rotated heads: items of eight pairs (j .. j + 7 and their partners)
    const int per_head = half / 8, rotated = min(heads, nq + nkv);
    for (int item = threadIdx.x; item < rotated * per_head; item += blockDim.x) {
        const int h = item / per_head, j = (item % per_head) * 8;
        const bf16* x = row + (size_t)h * hd;
        const uint4 a = *reinterpret_cast<const uint4*>(x + j), b = *reinterpret_cast<const uint4*>(x + j + half);
        const bf16* xa = reinterpret_cast<const bf16*>(&a);
        const bf16* xb = reinterpret_cast<const bf16*>(&b);
        uint4 ya, yb;
        bf16* pa = reinterpret_cast<bf16*>(&ya);
        bf16* pb = reinterpret_cast<bf16*>(&yb);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float x1 = to_f32(xa[e]), x2 = to_f32(xb[e]), sn = sc[j + e], cs = sc[half + j + e];
            float y1, y2;
            rotate_pair(x1, x2, sn, cs, y1, y2);
            pa[e] = from_f32<bf16>(y1);
            pb[e] = from_f32<bf16>(y2);
        }
        bf16* dst = dst_of(h);
        *reinterpret_cast<uint4*>(dst + j) = ya;
        *reinterpret_cast<uint4*>(dst + j + half) = yb;
    }
    // what is not rotated: the tails of the rotated heads and the value heads, eight elements at a time
    const int tail = (hd - rot_dim) / 8, whole = hd / 8;
    const int copies = rotated * tail + (heads - rotated) * whole;
    for (int item = threadIdx.x; item < copies; item += blockDim.x) {
        int h, c;
        if (item < rotated * tail) { h = item / tail; c = rot_dim + (item % tail) * 8; }
        else { const int v = item - rotated * tail; h = rotated + v / whole; c = (v % whole) * 8; }
        *reinterpret_cast<uint4*>(dst_of(h) + c) = *reinterpret_cast<const uint4*>(row + (size_t)h * hd + c);
    }
}

WLLM_API int wllm_rope_kv_write(const void* qkv, int in_dtype, int row_stride, int in_splits, long long in_split_stride,
                                void* q_out, int out_dtype, int q_stride, const int* positions, const int* slots,
                                const float* inv_freq, void* k_pages, void* v_pages, int n, int nq, int nkv, int hd,
                                int rot_dim, int page_size, int interleaved, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (hd <= 0 || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || page_size <= 0 || nq <= 0 || nkv <= 0 || in_splits < 1)
        return WLLM_BAD_SIZE;
    if (n >= 256 && !interleaved && in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16 && in_splits == 1 && hd % 8 == 0 && rot_dim % 16 == 0 &&
        row_stride % 8 == 0 && q_stride % 8 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)q_out & 15) &&
        !((uintptr_t)k_pages & 15) && !((uintptr_t)v_pages & 15))
        return wllm_launch(rope_kv_write_rows_kernel, n, 128, (size_t)rot_dim * sizeof(float), stream, (const bf16*)qkv, row_stride,
                           (bf16*)q_out, q_stride, positions, slots, inv_freq, (bf16*)k_pages, (bf16*)v_pages, nq, nkv, hd,
                           rot_dim, page_size);
    const int threads = hd >= 256 ? 128 : (hd >= 128 ? 64 : 32);
    // One CTA a token once the tokens alone fill the SMs several times over; below that a CTA a head, which keeps a
    // token's heads (and the partial sums each has to add) on different SMs: 256 tokens x 10 heads of 4 parts took
    // 24 us a layer as 256 CTAs and take 6 as 2,560.
    const bool all_heads = n >= 1024;
    const dim3 grid(n, all_heads ? 1 : nq + 2 * nkv);
#define GO2(TI, TO, A) wllm_launch(rope_kv_write_kernel<TI, TO, A>, grid, threads, 0, stream, (const TI*)qkv, row_stride, in_splits, \
        (size_t)in_split_stride, (TO*)q_out, q_stride, positions, slots, inv_freq, (TO*)k_pages, (TO*)v_pages, nq, nkv, hd, \
        rot_dim, page_size, interleaved)
#define GO(TI, TO) (all_heads ? GO2(TI, TO, true) : GO2(TI, TO, false))
    if (in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16) return GO(bf16, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_BF16) return GO(float, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_F32) return GO(float, float);
#undef GO
#undef GO2
    return WLLM_BAD_DTYPE;
}
