// Attention over the paged cache, one warp per (token, query head), every size.
//
// A token at position p of request r attends to the keys first..p of r, where
// first = 0, or p - window + 1 when the layer has a window; the keys are found
// through the request's row of the block table.  The keys and values of this
// step's own tokens are already in the pages when the kernel runs, so a portion
// of a prompt, a whole prompt and a single decoded token are the same case.
//
// Scores, softmax statistics and the output accumulate in 32-bit (expf, no fast
// math), in an order that is a function of the keys' absolute positions alone:
//   chunk    64 keys that start at an absolute multiple of 64.  Its partial result
//            (max m, sum l, output o) starts from nothing and takes the chunk's keys
//            in tiles of 32 (absolute multiples of 32) with the running-maximum rule.
//   row      the chunks' partial results merged one after the other in ascending
//            order:  m' = max(m, mc), l = l e^(m-m') + lc e^(mc-m'), o likewise.
// So a token's output depends on its own query and keys only: not on what else is
// in the batch, nor on how the sequence was cut into steps, nor on which pages hold
// it, nor on which of the two kernels below computed it, bit for bit:
//   walk     one warp per (token, head) takes the row's chunks in turn.  Steps of
//            many rows (prompts and their portions).
//   split    one warp per (token, head, chunk) leaves its partial result in scratch
//            memory and a second kernel merges a row's chunks in order.  Steps of few
//            rows over long contexts (decoding), where a walk would leave most SMs idle.
//
// Used for the 32-bit path at every size, and for bfloat16 at the sizes that the
// tensor-core kernels refuse.
#include "common.cuh"

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    __device__ static void load(const bf16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            out[2 * i] = f.x; out[2 * i + 1] = f.y;
        }
    }
};

constexpr int WARPS = 4;
constexpr int CHUNK = 64;

// The partial result of one chunk of one row (every lane holds m and l; lane x holds o of the dimensions e*32+x).
template <typename T, int NE>
__device__ __forceinline__ void chunk_partial(const float* __restrict__ qs, const T* __restrict__ k_pages,
                                              const T* __restrict__ v_pages, const int* __restrict__ table, int nkv,
                                              int kvh, int hd, int page_size, int first, int pos, int chunk, float scale,
                                              int lane, float& m, float& l, float (&o)[NE]) {
    m = -INFINITY;
    l = 0.f;
#pragma unroll
    for (int e = 0; e < NE; ++e) o[e] = 0.f;
    const int lo = max(chunk * CHUNK, (first >> 5) << 5), hi = min(chunk * CHUNK + CHUNK - 1, pos);
    for (int tile = lo; tile <= hi; tile += 32) {
        const int key = tile + lane;
        const bool valid = key >= first && key <= pos;
        float s = -INFINITY;
        int row = -1;  // index of the key's row of head_dim elements inside the pool
        if (valid) {
            const int page = table[key / page_size];
            row = (page * nkv + kvh) * page_size + key % page_size;
            const T* kr = k_pages + (size_t)row * hd;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            float kv[Vec<T>::N];
#pragma unroll 8
            for (int d = 0; d < hd; d += Vec<T>::N) {
                Vec<T>::load(kr + d, kv);
#pragma unroll
                for (int i = 0; i < Vec<T>::N; ++i) acc[i & 3] = fmaf(qs[d + i], kv[i], acc[i & 3]);
            }
            s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int e = 0; e < NE; ++e) o[e] *= corr;
        // values of four keys are requested before the first of them is used; a key outside the row's range
        // (only at its two ends) adds fma(0, v, o) = o with the values of a key inside it
        const int count = min(32, pos - tile + 1);
        const int safe = __shfl_sync(0xffffffffu, row, min(31, pos - tile));     // the row's last key of this tile: always valid
        for (int j0 = 0; j0 < count; j0 += 4) {
            float pj[4], vj[4][NE];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = min(j0 + u, 31);
                pj[u] = j0 + u < count ? __shfl_sync(0xffffffffu, p, j) : 0.f;
                const int rj = __shfl_sync(0xffffffffu, row, j);
                const T* vr = v_pages + (size_t)(rj < 0 || j0 + u >= count ? safe : rj) * hd;
#pragma unroll
                for (int e = 0; e < NE; ++e) {
                    const int d = e * 32 + lane;
                    vj[u][e] = d < hd ? to_f32(vr[d]) : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int e = 0; e < NE; ++e) o[e] = fmaf(pj[u], vj[u][e], o[e]);
        }
        m = m_new;
    }
}

// (m, l, o) <- (m, l, o) merged with the next chunk's (mc, lc, oc).  From the empty state (m = -inf, l = 0,
// o = 0) the result is the chunk's own, exactly: e^(-inf) = 0 and e^0 = 1.
template <int NE>
__device__ __forceinline__ void merge_chunk(float& m, float& l, float (&o)[NE], float mc, float lc, const float (&oc)[NE]) {
    const float m_new = fmaxf(m, mc);
    const float a = expf(m - m_new), b = expf(mc - m_new);
    l = fmaf(lc, b, l * a);
#pragma unroll
    for (int e = 0; e < NE; ++e) o[e] = fmaf(oc[e], b, o[e] * a);
    m = m_new;
}

template <typename T, int NE>
__device__ __forceinline__ void store_row(T* __restrict__ orow, int hd, int lane, float l, const float (&o)[NE]) {
    const float inv_l = 1.0f / l;
#pragma unroll
    for (int e = 0; e < NE; ++e) {
        const int d = e * 32 + lane;
        if (d < hd) orow[d] = from_f32<T>(o[e] * inv_l);
    }
}

// SPLIT false: grid (items / WARPS), the warp walks its row's chunks and writes the row.
// SPLIT true:  grid (items / WARPS, max_chunks), the warp of (item, slot) computes chunk first_chunk + slot of its
//              row and writes m, l, o[hd] to scratch[(item * max_chunks + slot) * (hd + 2)]; the warp of the last
//              slot also takes whatever chunks lie beyond it (merged in order), so that no key is dropped when a
//              row has more chunks than the caller's bound promised.
template <typename T, int NE, bool SPLIT>  // head_dim <= 32 * NE
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                            const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                            const int* __restrict__ token_req, const int* __restrict__ positions,
                            const int* __restrict__ block_table, int max_pages, int n_tokens, int nq, int nkv, int hd,
                            int page_size, int window, float scale, float* __restrict__ scratch, int max_chunks) {
    extern __shared__ float q_smem[];
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * WARPS + warp;
    if (item >= n_tokens * nq) return;
    const int token = item / nq, head = item % nq;
    const int kvh = head / (nq / nkv);
    const int pos = positions[token];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int first_chunk = first / CHUNK, last_chunk = pos / CHUNK;
    int c0 = first_chunk, c1 = last_chunk;
    if (SPLIT) {
        c0 = first_chunk + (int)blockIdx.y;
        if (c0 > last_chunk) return;
        if ((int)blockIdx.y < max_chunks - 1) c1 = c0;
    }
    const int* table = block_table + (size_t)token_req[token] * max_pages;
    float* qs = q_smem + warp * hd;
    const T* qrow = q + (size_t)token * q_stride + (size_t)head * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f, o[NE];
#pragma unroll
    for (int e = 0; e < NE; ++e) o[e] = 0.f;
    for (int chunk = c0; chunk <= c1; ++chunk) {
        float mc, lc, oc[NE];
        chunk_partial<T, NE>(qs, k_pages, v_pages, table, nkv, kvh, hd, page_size, first, pos, chunk, scale, lane, mc, lc, oc);
        merge_chunk<NE>(m, l, o, mc, lc, oc);
    }
    if (SPLIT) {
        float* dst = scratch + ((size_t)item * max_chunks + blockIdx.y) * (hd + 2);
        if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
        for (int e = 0; e < NE; ++e) {
            const int d = e * 32 + lane;
            if (d < hd) dst[2 + d] = o[e];
        }
    } else {
        store_row<T, NE>(out + (size_t)token * out_stride + (size_t)head * hd, hd, lane, l, o);
    }
}

template <typename T, int NE>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simt_merge_kernel(T* __restrict__ out, int out_stride, const int* __restrict__ positions, int n_tokens,
                                  int nq, int hd, int window, const float* __restrict__ scratch, int max_chunks) {
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * WARPS + warp;
    if (item >= n_tokens * nq) return;
    const int token = item / nq, head = item % nq;
    const int pos = positions[token];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int slots = min(max_chunks, pos / CHUNK - first / CHUNK + 1);
    float m = -INFINITY, l = 0.f, o[NE];
#pragma unroll
    for (int e = 0; e < NE; ++e) o[e] = 0.f;
    for (int s = 0; s < slots; ++s) {
        const float* src = scratch + ((size_t)item * max_chunks + s) * (hd + 2);
        float oc[NE];
#pragma unroll
        for (int e = 0; e < NE; ++e) {
            const int d = e * 32 + lane;
            oc[e] = d < hd ? src[2 + d] : 0.f;
        }
        merge_chunk<NE>(m, l, o, src[0], src[1], oc);
    }
    store_row<T, NE>(out + (size_t)token * out_stride + (size_t)head * hd, hd, lane, l, o);
}

template <typename T>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                  const int* token_req, const int* positions, const int* block_table, int max_pages, int n_tokens,
                  int nq, int nkv, int hd, int page_size, int window, float scale, float* scratch, int max_chunks,
                  cudaStream_t stream) {
    const int blocks = (n_tokens * nq + WARPS - 1) / WARPS;
    const size_t smem = (size_t)WARPS * hd * sizeof(float);
    const bool split = scratch != nullptr && max_chunks > 1;
#define GO(NE) do { \
        if (!split) \
            return wllm_launch(paged_attention_simt_kernel<T, NE, false>, blocks, WARPS * 32, smem, stream, \
                (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages, token_req, positions, \
                block_table, max_pages, n_tokens, nq, nkv, hd, page_size, window, scale, scratch, max_chunks); \
        const int st = wllm_launch(paged_attention_simt_kernel<T, NE, true>, dim3(blocks, max_chunks), WARPS * 32, smem, \
                stream, (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages, token_req, \
                positions, block_table, max_pages, n_tokens, nq, nkv, hd, page_size, window, scale, scratch, max_chunks); \
        if (st != WLLM_OK) return st; \
        return wllm_launch(paged_attention_simt_merge_kernel<T, NE>, blocks, WARPS * 32, 0, stream, (T*)out, out_stride, \
                positions, n_tokens, nq, hd, window, (const float*)scratch, max_chunks); \
    } while (0)
    if (hd <= 64) GO(2);
    if (hd <= 128) GO(4);
    if (hd <= 256) GO(8);
    GO(16);
#undef GO
}

// scratch (may be null) and max_chunks: with scratch of n_tokens * nq * max_chunks * (hd + 2) floats and
// max_chunks > 1 the split kernels run; max_chunks must be at least the number of chunks of 64 keys that any
// row of the step touches, or the results, still right, are no longer bit-equal to the walk's.
WLLM_API int wllm_paged_attention_simt(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                       const void* v_pages, int dtype, const int* token_req, const int* positions,
                                       const int* block_table, int max_pages, int n_tokens, int nq, int nkv, int hd,
                                       int page_size, int window, float scale, float* scratch, int max_chunks,
                                       cudaStream_t stream) {
    if (n_tokens <= 0) return WLLM_OK;
    // rows are read with 16-byte loads: head sizes come in steps of 16 up to 512
    if (hd <= 0 || hd > 512 || hd % 16 != 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || max_pages <= 0)
        return WLLM_BAD_SIZE;
    if (scratch != nullptr && (max_chunks < 1 || max_chunks > 65535)) return WLLM_BAD_SIZE;
    if (dtype == WLLM_BF16) {
        if (q_stride % 8 != 0) return WLLM_BAD_ALIGN;
        return launch<bf16>(q, q_stride, out, out_stride, k_pages, v_pages, token_req, positions, block_table, max_pages,
                            n_tokens, nq, nkv, hd, page_size, window, scale, scratch, max_chunks, stream);
    }
    if (dtype == WLLM_F32)
        return launch<float>(q, q_stride, out, out_stride, k_pages, v_pages, token_req, positions, block_table, max_pages,
                             n_tokens, nq, nkv, hd, page_size, window, scale, scratch, max_chunks, stream);
    return WLLM_BAD_DTYPE;
}
