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
//   tiled    a CTA takes 32 rows of one (request, key/value head) and brings every tile
//            of 32 keys and values into shared memory once for all of them; each warp
//            runs its four rows against the tile with the walk's arithmetic.  Portions
//            of prompts, where neighbouring rows read the same keys.
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
#pragma unroll 16
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
        l = fmaf(l, corr, warp_sum(p));
#pragma unroll
        for (int e = 0; e < NE; ++e) o[e] *= corr;
        // values of eight keys are requested before the first of them is used; a key outside the row's range
        // (only at its two ends) adds fma(0, v, o) = o with the values of a key inside it
        const int count = min(32, pos - tile + 1);
        const int safe = __shfl_sync(0xffffffffu, row, min(31, pos - tile));     // the row's last key of this tile: always valid
        constexpr int VA = NE <= 8 ? 8 : 4;      // value rows asked for together
        for (int j0 = 0; j0 < count; j0 += VA) {
            float pj[VA], vj[VA][NE];
#pragma unroll
            for (int u = 0; u < VA; ++u) {
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
            for (int u = 0; u < VA; ++u)
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
    // The merges of a row are one chain, in chunk order; the loads are not: a group of chunks is asked for at once and
    // then merged one after the other (one load's latency a chunk made this kernel the longest of a 32-bit decode
    // step: 149 us for 85 chunks of a row).
    constexpr int AHEAD = NE <= 8 ? 8 : 4;
    for (int s0 = 0; s0 < slots; s0 += AHEAD) {
        float mc[AHEAD], lc[AHEAD], oc[AHEAD][NE];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const float* src = scratch + ((size_t)item * max_chunks + min(s0 + u, slots - 1)) * (hd + 2);
            mc[u] = src[0];
            lc[u] = src[1];
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                const int d = e * 32 + lane;
                oc[u][e] = d < hd ? src[2 + d] : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < AHEAD; ++u)
            if (s0 + u < slots) merge_chunk<NE>(m, l, o, mc[u], lc[u], oc[u]);
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

// --------------------------------------------------------------------------------------
// tiled: grid (tiles of 32 rows, kv heads, requests); rows of a request are (token, head of the group)
// --------------------------------------------------------------------------------------
constexpr int TL_WARPS = 8, TL_RPW = 4, TL_ROWS = TL_WARPS * TL_RPW;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;          // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

template <typename T, int NE>
__global__ void __launch_bounds__(TL_WARPS * 32)
paged_attention_simt_tiled_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                  const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                  const int* __restrict__ req_q_start, const int* __restrict__ req_q_len,
                                  const int* __restrict__ req_ctx_len, const int* __restrict__ block_table, int max_pages,
                                  int nq, int nkv, int hd, int page_size, int window, float scale) {
    constexpr int VN = Vec<T>::N;                  // elements of a 16-byte piece
    extern __shared__ __align__(16) unsigned char tl_smem[];
    pdl_begin();
    const int g = blockIdx.y, r = blockIdx.z;
    const int q_len = req_q_len[r], rep = nq / nkv, rows = q_len * rep;
    const int m0 = blockIdx.x * TL_ROWS;
    if (m0 >= rows) return;
    const int ctx = req_ctx_len[r], q_start = req_q_start[r], pos0 = ctx - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kld = hd + VN;                       // a key's row in shared memory: the head and one piece of padding (banks)
    float* qs = reinterpret_cast<float*>(tl_smem);                          // [32 rows][hd] float
    T* ks = reinterpret_cast<T*>(qs + TL_ROWS * hd);                        // [2][32 keys][kld]
    T* vs = ks + 2 * 32 * kld;                                              // [2][32 keys][hd]
    const int* table = block_table + (size_t)r * max_pages;

    // this warp's rows: position, first key, where they are stored
    int pos_r[TL_RPW], first_r[TL_RPW];
#pragma unroll
    for (int i = 0; i < TL_RPW; ++i) {
        const int m = m0 + warp * TL_RPW + i;
        pos_r[i] = m < rows ? pos0 + m / rep : -1;                          // a row past the end takes no key
        first_r[i] = window > 0 ? max(0, pos_r[i] - window + 1) : 0;
    }
    for (int idx = threadIdx.x; idx < TL_ROWS * hd; idx += blockDim.x) {
        const int m = m0 + idx / hd, d = idx % hd;
        qs[idx] = m < rows ? to_f32(q[(size_t)(q_start + m / rep) * q_stride + (size_t)(g * rep + m % rep) * hd + d]) : 0.f;
    }
    // the keys that the CTA's rows see, in tiles of 32 at absolute multiples of 32
    const int last_m = min(rows, m0 + TL_ROWS) - 1;
    const int key_hi = pos0 + last_m / rep + 1;                              // one past the last row's position
    const int key_lo = window > 0 ? max(0, pos0 + m0 / rep - window + 1) : 0;
    const int t_lo = key_lo >> 5, t_hi = (key_hi + 31) >> 5;

    auto load_tile = [&](int t, int stage) {
        const int pieces = hd / VN;                // 16-byte pieces of a key's row
        for (int c = threadIdx.x; c < 32 * pieces; c += blockDim.x) {
            const int kl = c / pieces, piece = c % pieces, key = t * 32 + kl;
            const bool valid = key >= key_lo && key < key_hi;           // others are zero: their weight is zero, their values must be numbers
            size_t row = 0;
            if (valid) row = ((size_t)table[key / page_size] * nkv + g) * page_size + key % page_size;
            cp_async_16(ks + ((size_t)stage * 32 + kl) * kld + piece * VN, k_pages + row * hd + piece * VN, valid);
            cp_async_16(vs + ((size_t)stage * 32 + kl) * hd + piece * VN, v_pages + row * hd + piece * VN, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float m_t[TL_RPW], l_t[TL_RPW], o_t[TL_RPW][NE];      // the rows' results so far (finished chunks)
    float m_c[TL_RPW], l_c[TL_RPW], o_c[TL_RPW][NE];      // the chunk in progress
    bool open_c[TL_RPW];
#pragma unroll
    for (int i = 0; i < TL_RPW; ++i) {
        m_t[i] = m_c[i] = -INFINITY; l_t[i] = l_c[i] = 0.f; open_c[i] = false;
#pragma unroll
        for (int e = 0; e < NE; ++e) o_t[i][e] = o_c[i][e] = 0.f;
    }
    if (t_lo < t_hi) load_tile(t_lo, 0);
    for (int t = t_lo; t < t_hi; ++t) {
        const int stage = (t - t_lo) & 1;
        if (t + 1 < t_hi) load_tile(t + 1, stage ^ 1); else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();                          // tile t is here for everyone (and the queries, the first time)
        const T* kt = ks + (size_t)stage * 32 * kld;
        const T* vt = vs + (size_t)stage * 32 * hd;
        const int tile = t * 32, key = tile + lane;
        // a row takes part in the tiles from its first key's to its own position's, as in the walk
        bool act[TL_RPW], any = false;
#pragma unroll
        for (int i = 0; i < TL_RPW; ++i) {
            act[i] = !(tile > pos_r[i] || tile + 31 < first_r[i]);
            any = any || act[i];
        }
        if (any) {
            // scores of the warp's four rows against this lane's key: the key's row is read once for the four
            // (a row that sits this tile out is computed along and dropped; every number it meets is finite)
            const T* kr = kt + (size_t)lane * kld;
            const float* qw = qs + (size_t)(warp * TL_RPW) * hd;
            float acc[TL_RPW][4];
#pragma unroll
            for (int i = 0; i < TL_RPW; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll 4
            for (int d = 0; d < hd; d += VN) {
                float kv[VN];
                Vec<T>::load(kr + d, kv);
#pragma unroll
                for (int i = 0; i < TL_RPW; ++i) {
                    float qv[VN];
#pragma unroll
                    for (int u = 0; u < VN; u += 4) {
                        const float4 t4 = *reinterpret_cast<const float4*>(qw + (size_t)i * hd + d + u);
                        qv[u] = t4.x; qv[u + 1] = t4.y; qv[u + 2] = t4.z; qv[u + 3] = t4.w;
                    }
#pragma unroll
                    for (int u = 0; u < VN; ++u) acc[i][u & 3] = fmaf(qv[u], kv[u], acc[i][u & 3]);
                }
            }
            float p[TL_RPW];
#pragma unroll
            for (int i = 0; i < TL_RPW; ++i) {
                p[i] = 0.f;
                if (!act[i]) continue;
                const bool valid = key >= first_r[i] && key <= pos_r[i];
                const float s = valid ? ((acc[i][0] + acc[i][1]) + (acc[i][2] + acc[i][3])) * scale : -INFINITY;
                const float m_new = fmaxf(m_c[i], warp_max(s));
                p[i] = valid ? expf(s - m_new) : 0.f;
                const float corr = expf(m_c[i] - m_new);
                l_c[i] = fmaf(l_c[i], corr, warp_sum(p[i]));
#pragma unroll
                for (int e = 0; e < NE; ++e) o_c[i][e] *= corr;
                m_c[i] = m_new;
                open_c[i] = true;
            }
            // values: a key's row is read once for the four rows; a weight of 0 (a key outside a row's range, a row
            // that sits the tile out) adds fma(0, v, o) = o
#pragma unroll 2
            for (int j = 0; j < 32; ++j) {
                float v[NE];
#pragma unroll
                for (int e = 0; e < NE; ++e) {
                    const int d = e * 32 + lane;
                    v[e] = d < hd ? to_f32(vt[(size_t)j * hd + d]) : 0.f;
                }
#pragma unroll
                for (int i = 0; i < TL_RPW; ++i) {
                    const float pj = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
                    for (int e = 0; e < NE; ++e) o_c[i][e] = fmaf(pj, v[e], o_c[i][e]);
                }
            }
        }
        // the end of a chunk of 64 keys (or of the row): its result joins the row's
        const bool chunk_ends = ((t + 1) & (CHUNK / 32 - 1)) == 0 || t + 1 == t_hi;
#pragma unroll
        for (int i = 0; i < TL_RPW; ++i) {
            if (open_c[i] && (chunk_ends || tile + 32 > pos_r[i])) {
                merge_chunk<NE>(m_t[i], l_t[i], o_t[i], m_c[i], l_c[i], o_c[i]);
                m_c[i] = -INFINITY; l_c[i] = 0.f; open_c[i] = false;
#pragma unroll
                for (int e = 0; e < NE; ++e) o_c[i][e] = 0.f;
            }
        }
        __syncthreads();                          // everyone is done with this stage before the tile after next lands in it
    }
#pragma unroll
    for (int i = 0; i < TL_RPW; ++i) {
        const int m = m0 + warp * TL_RPW + i;
        if (m < rows)
            store_row<T, NE>(out + (size_t)(q_start + m / rep) * out_stride + (size_t)(g * rep + m % rep) * hd, hd, lane, l_t[i], o_t[i]);
    }
}

template <typename T>
static int launch_tiled(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                        const int* req_q_start, const int* req_q_len, const int* req_ctx_len, const int* block_table,
                        int max_pages, int requests, int max_q_len, int nq, int nkv, int hd, int page_size, int window,
                        float scale, cudaStream_t stream) {
    const int rep = nq / nkv;
    const dim3 grid((max_q_len * rep + TL_ROWS - 1) / TL_ROWS, nkv, requests);
    const size_t smem = (size_t)TL_ROWS * hd * sizeof(float) + 2 * 32 * ((size_t)(hd + Vec<T>::N) + hd) * sizeof(T);
#define GO(NE) do { \
        static bool raised = false; \
        if (!raised) { \
            const cudaError_t e = cudaFuncSetAttribute(paged_attention_simt_tiled_kernel<T, NE>, \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max); \
            if (e != cudaSuccess) return 1000 + (int)e; \
            raised = true; \
        } \
        return wllm_launch(paged_attention_simt_tiled_kernel<T, NE>, grid, TL_WARPS * 32, smem, stream, (const T*)q, q_stride, \
                           (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages, req_q_start, req_q_len, req_ctx_len, \
                           block_table, max_pages, nq, nkv, hd, page_size, window, scale); \
    } while (0)
    const int smem_max = TL_ROWS * 256 * (int)sizeof(float) + 2 * 32 * ((256 + Vec<T>::N) + 256) * (int)sizeof(T);
    if (hd <= 64) GO(2);
    if (hd <= 128) GO(4);
    GO(8);
#undef GO
}

// The tiled kernel for the requests of a step (all of them: a request with one token is a tile with few rows).
// Head sizes up to 256; the result is the walk's bit for bit.
WLLM_API int wllm_paged_attention_simt_tiled(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                             const void* v_pages, int dtype, const int* req_q_start, const int* req_q_len,
                                             const int* req_ctx_len, const int* block_table, int max_pages, int requests,
                                             int max_q_len, int nq, int nkv, int hd, int page_size, int window, float scale,
                                             cudaStream_t stream) {
    if (requests <= 0 || max_q_len <= 0) return WLLM_OK;
    if (hd <= 0 || hd > 256 || hd % 16 != 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || max_pages <= 0 ||
        nkv > 65535 || requests > 65535)
        return WLLM_BAD_SIZE;
    if (dtype == WLLM_BF16) {
        if (q_stride % 8 != 0) return WLLM_BAD_ALIGN;
        return launch_tiled<bf16>(q, q_stride, out, out_stride, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len,
                                  block_table, max_pages, requests, max_q_len, nq, nkv, hd, page_size, window, scale, stream);
    }
    if (dtype == WLLM_F32)
        return launch_tiled<float>(q, q_stride, out, out_stride, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len,
                                   block_table, max_pages, requests, max_q_len, nq, nkv, hd, page_size, window, scale, stream);
    return WLLM_BAD_DTYPE;
}
