// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// 32-bit accumulation), compiled for one head size: -DHEAD_DIM=<multiple of 16, <= 256>.
//
// Two kernels share the tile code.
//
//   decode   one CTA per (request with one new token, kv head, split of its keys).  The
//            query heads of the kv head's group are the rows of one 16-row tile, so the
//            keys are read once for the whole group.  The four warps take different
//            16-key slices of every 64-key tile and merge at the end.  Splits of
//            `split_keys` keys give a long context to many SMs; each writes its partial
//            (max, sum, unnormalised output) to scratch and a second kernel merges them
//            in split order.  A request with a single split writes its output directly.
//   prefill  one CTA per (request with several new tokens, kv head, tile of 128 rows),
//            rows = (token, query head of the group); the eight warps own 16 rows each and
//            walk all 64-key tiles up to the causal edge.
//
// Keys and values come straight from the pages through the request's block table
// ([page][kv_head][slot][head_dim] layout), by 16-byte cp.async into a swizzled,
// multi-stage ring in shared memory; rows outside a request's keys are zero-filled.
// Scores, the running maximum and sum and the output accumulate in 32-bit; the
// exponentials are exp2 of log2(e)-scaled scores.  Which requests each kernel serves is
// read from q_len on the device (1: decode, more: prefill), so a captured graph stays
// valid when the batch changes its contents but not its shape.
#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif

constexpr int HD = HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head sizes in steps of 16 up to 256");
constexpr int HDP = (HD + 63) / 64 * 64;   // row length in shared memory (elements): whole 128-byte groups
constexpr int ROWB = HDP * 2;              // bytes per shared-memory row
constexpr int CPR = HD / 8;                // 16-byte chunks of a row that carry data
constexpr int BN = 64;                     // keys per tile
constexpr int KT = HD / 16;                // k-steps of q.k over the head size
constexpr int NTO = HD / 8;                // 8-wide column tiles of the output
constexpr int NWARPS = 4;
constexpr int NTHREADS = NWARPS * 32;
constexpr int TILE_BYTES = BN * ROWB;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * ROWB + ((((chunk & ~7) | ((chunk ^ row) & 7))) << 4));
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// One 64-key tile of keys AND values of kv head `g` into shared memory (all threads of the CTA).
// Each warp first reads the tile's page ids (at most four pages of 16 keys) with one load and hands
// them out by shuffle, so the copies that follow depend on no further load.
template <int NT>
__device__ __forceinline__ void load_kv_tile(uint32_t k_dst, uint32_t v_dst, const bf16* __restrict__ k_pages,
                                             const bf16* __restrict__ v_pages, const int* __restrict__ table,
                                             int tile_start, int key_lo, int key_hi, int g, int nkv, int page_size,
                                             int page_shift) {
    const int lane = threadIdx.x & 31;
    const int first_page = tile_start >> page_shift;
    const int last_page = (min(tile_start + BN, key_hi) - 1) >> page_shift;
    int my_page = 0;
    if (first_page + lane <= last_page) my_page = table[first_page + lane];
#pragma unroll
    for (int it = 0; it < (BN * CPR + NT - 1) / NT; ++it) {
        const int idx = threadIdx.x + it * NT;
        const int row = idx / CPR, chunk = idx % CPR;
        const int key = tile_start + row;
        const int page = __shfl_sync(0xffffffffu, my_page, ((key >> page_shift) - first_page) & 31);
        if (BN * CPR % NT != 0 && idx >= BN * CPR) continue;
        const bool valid = key >= key_lo && key < key_hi;
        const size_t off = valid ? ((size_t)(page * nkv + g) * page_size + (key & (page_size - 1))) * HD + chunk * 8 : 0;
        cp_async16(k_dst + swz(row, chunk), k_pages + off, valid);
        cp_async16(v_dst + swz(row, chunk), v_pages + off, valid);
    }
}

// Rows of the query tile: row m of a (request, kv head) is (token m / rep, head g*rep + m % rep).
template <int NT>
__device__ __forceinline__ void load_q_tile(uint32_t dst, const bf16* __restrict__ q, int q_stride, int q_start, int q_len,
                                            int row0, int nrows, int g, int rep) {
    for (int idx = threadIdx.x; idx < nrows * CPR; idx += NT) {
        const int row = idx / CPR, chunk = idx % CPR;
        const int m = row0 + row;
        const bool valid = m < q_len * rep;
        const bf16* src = q;
        if (valid) src = q + (size_t)(q_start + m / rep) * q_stride + (size_t)(g * rep + m % rep) * HD + chunk * 8;
        cp_async16(dst + swz(row, chunk), src, valid);
    }
}

// Running state of the 16 rows of a warp: rows r = lane/4 and r + 8.
struct RowState {
    float m[2], l[2];      // running max (log2 units) and this thread's share of the running sum
    float o[NTO][4];
};

// One warp: its 16 query rows (at q_rows in shared memory) against NKEYS keys of a tile
// that start at shared-memory row `key0`; `pos_r[i]`/`first_r[i]` bound the keys each of the
// thread's two rows may see; `key_base` is the absolute index of tile row 0.
template <int NKEYS>
__device__ __forceinline__ void warp_tile(RowState& st, uint32_t q_rows, uint32_t k_tile, uint32_t v_tile, int key0,
                                          int key_base, const int (&pos_r)[2], const int (&first_r)[2], float scale2) {
    constexpr int NT = NKEYS / 8;
    const int lane = threadIdx.x & 31;
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_chunk = lane >> 4;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_chunk = (lane >> 3) & 1;
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) {
        uint32_t a[4];
        ldsm4(q_rows + swz(a_row, kt * 2 + a_chunk), a);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            ldsm4(k_tile + swz(key0 + np * 16 + b_row, kt * 2 + b_chunk), b);
            mma16816(s[2 * np], a, b[0], b[1]);
            mma16816(s[2 * np + 1], a, b[2], b[3]);
        }
    }
    // mask, scale to log2 units, running max
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int key = key_base + key0 + n * 8 + (lane & 3) * 2 + (c & 1);
            const int i = c >> 1;
            const bool ok = key <= pos_r[i] && key >= first_r[i];
            s[n][c] = ok ? s[n][c] * scale2 : -INFINITY;
            mx[i] = fmaxf(mx[i], s[n][c]);
        }
    float corr[2], base[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(st.m[i], mx[i]);
        base[i] = m_new == -INFINITY ? 0.f : m_new;          // a row that has seen no key yet
        corr[i] = exp2f(st.m[i] - base[i]);                  // exp2(-inf) = 0 for the first keys
        st.m[i] = m_new;
        st.l[i] *= corr[i];
    }
#pragma unroll
    for (int n = 0; n < NTO; ++n) {
        st.o[n][0] *= corr[0]; st.o[n][1] *= corr[0];
        st.o[n][2] *= corr[1]; st.o[n][3] *= corr[1];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            s[n][c] = exp2f(s[n][c] - base[c >> 1]);
            st.l[c >> 1] += s[n][c];
        }
    // O += P V, 16 keys per k-step
    const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_chunk = lane >> 4;
#pragma unroll
    for (int kk = 0; kk < NKEYS / 16; ++kk) {
        uint32_t p[4];
        p[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        p[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        p[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        p[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int np = 0; np < NTO / 2; ++np) {
            uint32_t b[4];
            ldsm4t(v_tile + swz(key0 + kk * 16 + v_row, np * 2 + v_chunk), b);
            mma16816(st.o[2 * np], p, b[0], b[1]);
            mma16816(st.o[2 * np + 1], p, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ void init_state(RowState& st) {
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
#pragma unroll
    for (int n = 0; n < NTO; ++n) st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.f;
}

// --------------------------------------------------------------------------------------
// decode: grid (max_splits, nkv, requests)
// --------------------------------------------------------------------------------------
constexpr int DEC_STAGES = 3;
constexpr int DEC_SMEM = 16 * ROWB + DEC_STAGES * 2 * TILE_BYTES;

__global__ void __launch_bounds__(NTHREADS)
decode_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
              const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages, const int* __restrict__ req_q_start,
              const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len, const int* __restrict__ block_table,
              int max_pages, int nq, int nkv, int page_size, int window, float scale2, int split_keys, int max_splits,
              float* __restrict__ part_o, float* __restrict__ part_ml) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int split = blockIdx.x, g = blockIdx.y, r = blockIdx.z;
    if (req_q_len[r] != 1) return;
    const int ctx = req_ctx_len[r], pos = ctx - 1;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int num_splits = (ctx + split_keys - 1) / split_keys;
    if (split >= num_splits) return;
    const int key_lo = max(split * split_keys, first), key_hi = min(ctx, (split + 1) * split_keys);
    const int rep = nq / nkv, token = req_q_start[r];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_table + (size_t)r * max_pages;
    const uint32_t q_s = smem_u32(smem), kv_s = q_s + 16 * ROWB;

    RowState st;
    init_state(st);
    const bool empty = key_lo >= key_hi;     // the window starts behind this split
    const int t0 = key_lo / BN, t1 = empty ? t0 : (key_hi + BN - 1) / BN;   // tiles [t0, t1)
    load_q_tile<NTHREADS>(q_s, q, q_stride, token, 1, 0, 16, g, rep);
    const int page_shift = 31 - __clz(page_size);
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
        if (t0 + s < t1)
            load_kv_tile<NTHREADS>(kv_s + (2 * s) * TILE_BYTES, kv_s + (2 * s + 1) * TILE_BYTES, k_pages, v_pages, table,
                                   (t0 + s) * BN, key_lo, key_hi, g, nkv, page_size, page_shift);
        cp_commit();
    }
    const int first_r[2] = {key_lo, key_lo};
    for (int t = t0; t < t1; ++t) {
        cp_wait<DEC_STAGES - 2>();
        __syncthreads();
        const int nxt = t + DEC_STAGES - 1;
        if (nxt < t1) {
            const int s = (nxt - t0) % DEC_STAGES;
            load_kv_tile<NTHREADS>(kv_s + (2 * s) * TILE_BYTES, kv_s + (2 * s + 1) * TILE_BYTES, k_pages, v_pages, table,
                                   nxt * BN, key_lo, key_hi, g, nkv, page_size, page_shift);
        }
        cp_commit();
        const int s = (t - t0) % DEC_STAGES;
        const int hi_r[2] = {min(pos, key_hi - 1), min(pos, key_hi - 1)};
        warp_tile<16>(st, q_s, kv_s + (2 * s) * TILE_BYTES, kv_s + (2 * s + 1) * TILE_BYTES, warp * 16, t * BN, hi_r,
                      first_r, scale2);
    }
    cp_wait<0>();
    __syncthreads();

    // merge the four warps through shared memory (the tile ring is free now)
    float* sm_o = reinterpret_cast<float*>(smem);                  // [warp][16][HD]
    float* sm_ml = sm_o + NWARPS * 16 * HD;                         // [warp][16][2]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
        st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
    }
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < NTO; ++n) {
        float* o0 = sm_o + ((size_t)(warp * 16 + r0) * HD) + n * 8 + c0;
        float* o1 = sm_o + ((size_t)(warp * 16 + r0 + 8) * HD) + n * 8 + c0;
        o0[0] = st.o[n][0]; o0[1] = st.o[n][1];
        o1[0] = st.o[n][2]; o1[1] = st.o[n][3];
    }
    if ((lane & 3) == 0) {
        sm_ml[(warp * 16 + r0) * 2] = st.m[0];      sm_ml[(warp * 16 + r0) * 2 + 1] = st.l[0];
        sm_ml[(warp * 16 + r0 + 8) * 2] = st.m[1];  sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = st.l[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rep * HD; idx += NTHREADS) {
        const int row = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, sm_ml[(w * 16 + row) * 2]);
        const float base = M == -INFINITY ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float f = exp2f(sm_ml[(w * 16 + row) * 2] - base);
            L += sm_ml[(w * 16 + row) * 2 + 1] * f;
            O += sm_o[(size_t)(w * 16 + row) * HD + d] * f;
        }
        const int head = g * rep + row;
        if (num_splits == 1) {
            out[(size_t)token * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(O / L);
        } else {
            const size_t slot = ((size_t)r * nq + head) * max_splits + split;
            part_o[slot * HD + d] = O;
            if (d == 0) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
        }
    }
}

// merge of the splits: grid (nq, requests).  The splits' weights exp2(m_s - M) are computed once into
// shared memory; every thread then sums its output columns over the splits in split order.
constexpr int MERGE_MAX_SPLITS = 256;
__global__ void merge_kernel(bf16* __restrict__ out, int out_stride, const int* __restrict__ req_q_start,
                             const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len, int nq,
                             int split_keys, int max_splits, const float* __restrict__ part_o,
                             const float* __restrict__ part_ml) {
    __shared__ float w[MERGE_MAX_SPLITS];
    __shared__ float inv_l;
    const int head = blockIdx.x, r = blockIdx.y;
    if (req_q_len[r] != 1) return;
    const int num_splits = (req_ctx_len[r] + split_keys - 1) / split_keys;
    if (num_splits <= 1) return;
    const size_t slot0 = ((size_t)r * nq + head) * max_splits;
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int s = threadIdx.x; s < num_splits; s += 32) M = fmaxf(M, part_ml[(slot0 + s) * 2]);
        M = warp_max(M);
        const float base = M == -INFINITY ? 0.f : M;
        float L = 0.f;
        for (int s = threadIdx.x; s < num_splits; s += 32) {
            const float f = exp2f(part_ml[(slot0 + s) * 2] - base);
            w[s] = f;
            L += part_ml[(slot0 + s) * 2 + 1] * f;
        }
        L = warp_sum(L);
        if (threadIdx.x == 0) inv_l = 1.0f / L;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float O = 0.f;
#pragma unroll 4
        for (int s = 0; s < num_splits; ++s) O += part_o[(slot0 + s) * HD + d] * w[s];
        out[(size_t)req_q_start[r] * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(O * inv_l);
    }
}

// --------------------------------------------------------------------------------------
// prefill: grid (row tiles, nkv, requests); heavier (later) row tiles first
// --------------------------------------------------------------------------------------
constexpr int PRE_WARPS = 8;
constexpr int PRE_THREADS = PRE_WARPS * 32;
constexpr int BM = PRE_WARPS * 16;
constexpr int PRE_STAGES = 2;
constexpr int PRE_SMEM = BM * ROWB + PRE_STAGES * 2 * TILE_BYTES;

__global__ void __launch_bounds__(PRE_THREADS)
prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
               const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages, const int* __restrict__ req_q_start,
               const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len, const int* __restrict__ block_table,
               int max_pages, int nq, int nkv, int page_size, int window, float scale2, int skip_single) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int g = blockIdx.y, r = blockIdx.z;
    const int q_len = req_q_len[r];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;
    const int rep = nq / nkv, rows = q_len * rep;
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int row0 = tile * BM;
    if (row0 >= rows) return;
    const int ctx = req_ctx_len[r], q_start = req_q_start[r], pos0 = ctx - q_len;   // position of the request's first new token
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_table + (size_t)r * max_pages;
    const uint32_t q_s = smem_u32(smem), kv_s = q_s + BM * ROWB;

    // keys this CTA needs: from the first row's window start to the last row's position
    const int last_row = min(rows, row0 + BM) - 1;
    const int pos_hi = pos0 + last_row / rep;
    const int pos_lo = pos0 + row0 / rep;
    const int key_lo = window > 0 ? max(0, pos_lo - window + 1) : 0, key_hi = pos_hi + 1;
    const int t0 = key_lo / BN, t1 = (key_hi + BN - 1) / BN;

    int pos_r[2], first_r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = row0 + warp * 16 + (lane >> 2) + i * 8;
        pos_r[i] = m < rows ? pos0 + m / rep : -1;                      // a row past the end sees no key
        first_r[i] = window > 0 ? max(0, pos_r[i] - window + 1) : 0;
    }
    RowState st;
    init_state(st);
    const int page_shift = 31 - __clz(page_size);
    load_q_tile<PRE_THREADS>(q_s, q, q_stride, q_start, q_len, row0, BM, g, rep);
    for (int s = 0; s < PRE_STAGES - 1; ++s) {
        if (t0 + s < t1)
            load_kv_tile<PRE_THREADS>(kv_s + (2 * s) * TILE_BYTES, kv_s + (2 * s + 1) * TILE_BYTES, k_pages, v_pages, table,
                                      (t0 + s) * BN, key_lo, key_hi, g, nkv, page_size, page_shift);
        cp_commit();
    }
    for (int t = t0; t < t1; ++t) {
        cp_wait<PRE_STAGES - 2>();
        __syncthreads();
        const int nxt = t + PRE_STAGES - 1;
        if (nxt < t1) {
            const int s = (nxt - t0) % PRE_STAGES;
            load_kv_tile<PRE_THREADS>(kv_s + (2 * s) * TILE_BYTES, kv_s + (2 * s + 1) * TILE_BYTES, k_pages, v_pages, table,
                                      nxt * BN, key_lo, key_hi, g, nkv, page_size, page_shift);
        }
        cp_commit();
        const int s = (t - t0) % PRE_STAGES;
        // a warp whose rows all end before this tile has nothing to add
        const int warp_hi = pos0 + min(rows - 1, row0 + warp * 16 + 15) / rep;
        if (t * BN <= warp_hi && row0 + warp * 16 < rows)
            warp_tile<BN>(st, q_s + warp * 16 * ROWB, kv_s + (2 * s) * TILE_BYTES, kv_s + (2 * s + 1) * TILE_BYTES, 0,
                          t * BN, pos_r, first_r, scale2);
    }
    cp_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
        st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = row0 + warp * 16 + (lane >> 2) + i * 8;
        if (m >= rows) continue;
        const float inv = 1.0f / st.l[i];
        bf16* dst = out + (size_t)(q_start + m / rep) * out_stride + (size_t)(g * rep + m % rep) * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NTO; ++n) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(st.o[n][2 * i] * inv, st.o[n][2 * i + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = v;
        }
    }
}

// --------------------------------------------------------------------------------------
// entry points
// --------------------------------------------------------------------------------------
WLLM_API int wllm_attention_mma_head_dim() { return HD; }

// Floats of scratch the decode path needs for `requests` requests: partial outputs and (max, sum) pairs.
WLLM_API long long wllm_attention_mma_scratch_floats(int requests, int nq, int max_splits) {
    return (long long)requests * nq * max_splits * (HD + 2);
}

static int check_common(const void* q, int q_stride, const void* out, int out_stride, int nq, int nkv, int page_size) {
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size < 16 || (page_size & (page_size - 1))) return WLLM_BAD_SIZE;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 3)) return WLLM_BAD_ALIGN;
    return WLLM_OK;
}

// Tokens of requests with q_len == 1.  `scratch` holds wllm_attention_mma_scratch_floats(...) floats.
WLLM_API int wllm_attention_mma_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                       const void* v_pages, const int* req_q_start, const int* req_q_len,
                                       const int* req_ctx_len, const int* block_table, int max_pages, int requests,
                                       int nq, int nkv, int page_size, int window, float scale, int split_keys,
                                       int max_splits, float* scratch, cudaStream_t stream) {
    if (requests <= 0) return WLLM_OK;
    const int bad = check_common(q, q_stride, out, out_stride, nq, nkv, page_size);
    if (bad) return bad;
    if (nq / nkv > 16 || split_keys < BN || split_keys % BN != 0 || max_splits < 1 || max_splits > MERGE_MAX_SPLITS)
        return WLLM_BAD_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)requests * nq * max_splits * HD;
    decode_kernel<<<dim3(max_splits, nkv, requests), NTHREADS, DEC_SMEM, stream>>>(
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages, req_q_start,
        req_q_len, req_ctx_len, block_table, max_pages, nq, nkv, page_size, window, scale * LOG2E, split_keys,
        max_splits, part_o, part_ml);
    int status = wllm_launch_status();
    if (status || max_splits == 1) return status;
    merge_kernel<<<dim3(nq, requests), HD >= 256 ? 256 : (HD >= 128 ? 128 : 64), 0, stream>>>(
        (bf16*)out, out_stride, req_q_start, req_q_len, req_ctx_len, nq, split_keys, max_splits, part_o, part_ml);
    return wllm_launch_status();
}

// Tokens of requests with q_len > 1 (and of those with q_len == 1 too unless skip_single).
WLLM_API int wllm_attention_mma_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                        const void* v_pages, const int* req_q_start, const int* req_q_len,
                                        const int* req_ctx_len, const int* block_table, int max_pages, int requests,
                                        int max_q_len, int nq, int nkv, int page_size, int window, float scale,
                                        int skip_single, cudaStream_t stream) {
    if (requests <= 0 || max_q_len <= 0) return WLLM_OK;
    const int bad = check_common(q, q_stride, out, out_stride, nq, nkv, page_size);
    if (bad) return bad;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PRE_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    const int tiles = (max_q_len * (nq / nkv) + BM - 1) / BM;
    prefill_kernel<<<dim3(tiles, nkv, requests), PRE_THREADS, PRE_SMEM, stream>>>(
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages, req_q_start,
        req_q_len, req_ctx_len, block_table, max_pages, nq, nkv, page_size, window, scale * LOG2E, skip_single);
    return wllm_launch_status();
}
